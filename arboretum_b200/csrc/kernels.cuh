// Launchers of the level-loop kernels.  All of them enqueue on the given stream
// and never synchronise; sizes that depend on the data (node sizes, work-item
// counts) live in device memory and are read by the kernels themselves.
#pragma once
#include <cuda_runtime.h>

#include "common.cuh"
#include "gain.cuh"

namespace arb {

constexpr int kHistWords = 8192;      // words of one shared-memory histogram plane
constexpr int kHistThreads = 512;     // threads of a histogram CTA
constexpr int kHistCtasPerSm = 2;     // resident histogram CTAs per SM (32 warps: the row gather
                                      // of the levels below the root needs them to hide its latency)
constexpr int kMaxLevels = 16;
constexpr int kCounterStride = 32;    // words between two counters that many CTAs add to
constexpr int kMinItemRows = 256;     // smallest piece a node's row list is cut into
constexpr int kItemsPerCta = 6;       // items a histogram CTA gets at least (evens out the shares)

// Geometry of the binned matrix and of the histograms built from it.
//   bins : row-major, `pitch` bytes per row, feature f of row r at
//          bins[r * pitch + f * bin_bytes]; pitch is a multiple of 32.
//   tiles: TW consecutive features; TW * BINS == kHistWords, so one tile of one
//          node is kHistWords (g, h) pairs: hist[((node * NT + tile) * BINS + bin) * TW + lane]
struct Geometry {
  const unsigned char *bins;
  size_t pitch;
  int bin_bytes;
  int F;        // all features: dense ones first, then the categorical ones
  int n_dense;  // features below this id split by `bin <= b`, the others by `bin == b`
  int TW, NT, BINS;
  int hist_size;  // bins a split may use (config value); id hist_size = missing
  // optional feature-major copy bins_cm[f * cm_rows + row] (nullptr: absent): the row
  // descend step reads one feature of every row, which is sequential in this layout
  const unsigned char *bins_cm = nullptr;
  size_t cm_rows = 0;
  // 0: row-major, the tiles of a row lie side by side in its `pitch` bytes.  Otherwise the
  // matrix is kept tile by tile (uint8 bins only): tile t starts `tile_stride` bytes after tile
  // t - 1 and holds one 32-byte chunk per row (`pitch` = 32), so that the rows a tile's
  // histogram reads lie back to back however many tiles the matrix has.
  size_t tile_stride = 0;
};

// The driver's tensor map of a row-major uint8 bin matrix (bytes of a padded row x rows), with
// which the uint8 histogram kernel gathers rows through the TMA unit.  Opaque here so that only
// the histogram's translation unit needs the driver's header.
struct alignas(64) RowGatherMap {
  unsigned char opaque[128];
};
// false: no map (ARBORETUM_TMA_GATHER is not set in the environment, the driver's encoder is
// not available, the matrix has 2^31 rows or more): the kernel then gathers with cp.async
bool make_row_gather_map(RowGatherMap *out, const unsigned char *bins, size_t pitch, size_t rows);

struct HistLaunch {
  Geometry geo;
  const unsigned *rowid;  // nullptr: positions are row ids (root level)
  const void *grad;       // quantised gradients: int2[N] (pair) or int[N]
  bool pair;
  const WorkItem *items;  // every item has at most 2^(31 - quant_bits) rows
  const int *n_items;
  const int *item_slot = nullptr;  // per item: the run it belongs to (neighbouring items of one node
                                   // that one CTA takes and whose rows together fit an int32 plane);
                                   // nullptr: every item is a run of its own
  int max_items;
  int grid_x = 0;  // CTAs per feature tile; must be what the plan kernel cut the runs for when
                   // item_slot is given (0: from max_items)
  int *partials;  // [run][tile][2][kHistWords] int32 planes, written here
  const void *list_grad = nullptr;  // gradient records in list order (position p of `rowid` <->
                                    // record p), or nullptr: gathered from `grad` by row id.
                                    // Read by the uint8 kernel only.
  const RowGatherMap *row_map = nullptr;  // map of geo.bins (host pointer), or nullptr
  int *status = nullptr;  // device word, set to 1 when a wait on a TMA gather ran out (needed with
                          // row_map)
};
void launch_hist(const HistLaunch &a, cudaStream_t s);
int hist_grid_x(int max_items, int NT);

// (g, h) pair updates per second of the histogram kernels' two shared-memory reductions
// alone, on the current device: the ceiling their inner loop runs against
double measure_shared_atomic_peak(int steps, cudaStream_t s);

// planes of the items of every built node -> the level's int64 histogram
struct ReduceLaunch {
  const int *partials;
  const int *item_first;  // n_build + 1: the planes of built node b are [first[b], first[b+1])
  const int *build_node;  // node index (inside the level) of built node b; nullptr: level_hist
                          // holds the built nodes only, in build order
  int n_build;
  int NT;
  long long *level_hist;
  const long long *parent_hist;  // level above, for the subtraction
  bool subtract;      // also write sibling = parent - built
  int level_nodes;    // nodes of the level (size of level_hist)
  const int *built_child;  // per parent: which child was built (for the subtraction)
  bool accumulate = false;  // add into level_hist (cleared by the caller): row chunks of one level
};
void launch_reduce(const ReduceLaunch &a, cudaStream_t s);

// The built nodes' histograms alone (what row shards exchange) -> the level's buffer:
// built child = compact[parent], sibling = parent - compact[parent]
void launch_expand(const long long *compact, const long long *parent_hist, long long *level_hist,
                   const int *built_child, int n_parents, int NT, cudaStream_t s);

// sibling = parent - built child, for every parent of the level above
void launch_subtract(long long *level_hist, const long long *parent_hist, const int *built_child,
                     int n_parents, int NT, cudaStream_t s);

struct SplitLaunch {
  Geometry geo;
  const long long *hist;       // level buffer
  const long long *count_hist = nullptr;  // same layout, second word of a pair = rows ((g, h)
                                          // objectives with min_leaf_size > 1), or nullptr
  const unsigned *node_begin;  // L+1 prefix counts of this level
  const unsigned char *feature_active;  // F flags: evaluated at this level
  const int *feature_size;     // bins in use per feature
  const int *cat_candidates = nullptr;  // per feature: bins a one-vs-rest split may name
                                        // (categorical features), 0 for dense ones; or nullptr
  // The histogram may cover a subset of the columns (the columns a tree samples, copied side
  // by side): feature_map[j] is the feature behind column j of `geo`, ascending; records,
  // feature_active and cat_candidates speak of features.  nullptr: column j is feature j.
  const int *feature_map = nullptr;
  unsigned long long *keys;    // max_nodes packed (gain, feature, bin) maxima followed by
                               // max_nodes u32 arrival counters; zeroed by the plan kernel of the
                               // level (PlanBuffers::split_scratch)
  int max_nodes;
  NodeRec *rec;                // L records out
  const NodeRec *parent_rec;   // level above (nullptr at the root)
  const QuantScale *qs;
  GainParams gp;
  bool pair;
  int L;
};
void launch_split(const SplitLaunch &a, cudaStream_t s);

// out[r][j] = bins[r][map[j]] for j < n_cols (bin_bytes each), rows of `out_pitch` bytes whose
// padding is zeroed: the columns a tree samples, side by side.  With the feature-major copy
// bins_cm[f * n + r] at hand (uint8, n a multiple of 16) only the wanted columns are read.
// `tile_major` (needs bins_cm, uint8, n a multiple of 16): the copy is written tile by tile,
// tile t at out + t * n * 32 with 32 bytes per row (see Geometry::tile_stride).
void launch_compact_columns(const unsigned char *bins, size_t pitch, int bin_bytes, size_t n, const int *map,
                            int n_cols, unsigned char *out, size_t out_pitch, cudaStream_t s,
                            const unsigned char *bins_cm = nullptr, bool tile_major = false);
// whether launch_compact_columns can write the tile-by-tile layout for this matrix
bool compact_columns_tile_major_ok(int bin_bytes, size_t n, const unsigned char *bins_cm);

// --- node assignment and row lists ---------------------------------------------
struct PlanBuffers {
  WorkItem *hist_items;
  int *n_hist_items;
  int *hist_item_first;   // per built node: its first item; max_nodes + 1 entries
  int *item_slot;         // per item: its run (see HistLaunch); max_items entries
  int *slot_first;        // per built node: its first run; max_nodes + 1 entries
  int *built_child;       // per parent: 0 = left child built, 1 = right child
  unsigned *list_base;    // per node of the level: where its row list starts (0xffffffff: none)
  unsigned *cursor;       // per node of the level, kCounterStride words apart: rows written to
                          // its list so far
  unsigned *scratch_begin, *scratch_len;  // per built node: list start / length; max_nodes + 1
  int *scratch_node;      // per built node: its node index inside the level
  // cleared by the plan kernel for the kernels that follow it (instead of memsets of their own):
  unsigned *right_count;  //   the descend step's counters, one per node, kCounterStride apart
  unsigned *split_scratch;  // the split search's keys and arrival counters
  int split_scratch_words;
};

// Every row steps from its node to a child (or, below the last level, into a leaf).
struct DescendLaunch {
  Geometry geo;
  const NodeRec *rec;        // split records of the level the rows stand on
  int L;                     // nodes of that level
  unsigned short *node_of;   // per row: its node inside the level; becomes the child's (L == 1:
                             // not read, every row stands on the root)
  unsigned *child_count;     // per node (kCounterStride words apart): its rows that went right;
                             // added to here, cleared by the plan kernel before (PlanBuffers::
                             // right_count); nullptr = the final step,
  const float *leaf_w;       //   which adds leaf_w[child] to
  float *yhat;               //   yhat[row] instead
  size_t n;
};
void launch_descend(const DescendLaunch &a, cudaStream_t s);

// Prefix counts of a level, the children to build, their lists and the histogram work items.
struct LevelPlanLaunch {
  const unsigned *child_count;  // per parent (kCounterStride apart): rows that went right, from
                                // launch_descend; nullptr at the root
  const unsigned *parent_begin; // L / 2 + 1 prefix counts of the level above
  unsigned *node_begin;         // L + 1 prefix counts, written here (read at the root)
  NodeRec *parent_rec;          // L / 2 records of the level above: left_count += lefts
  int L;
  int item_rows;                // rows per work item
  int hist_grid_x;              // CTAs per feature tile of the histogram launch: each takes a
                                // contiguous share of the items
  int items_per_run;            // items of `item_rows` rows that fit an int32 plane together
  bool use_trick;               // build one child per parent, the other is parent - built
  bool by_hessian;              // choose it by the hessian sums (row shards, row chunks)
  PlanBuffers pb;
  int max_items;
};
void launch_plan_level(const LevelPlanLaunch &a, cudaStream_t s);

// rows of the built nodes -> list[pb.list_base[node] + ...]; with list_grad != nullptr their
// gradient records (int2 if pair, else int) are copied to the same positions of list_grad
void launch_gather_lists(const unsigned short *node_of, size_t n, int L, const PlanBuffers &pb,
                         unsigned *list, const void *grad, void *list_grad, bool pair,
                         cudaStream_t s);

// --- objective, leaves, prediction ----------------------------------------------
// Gradients of the round in two passes over (y, yhat).  emit = false: the largest |g| and h
// go to qs (multi:softmax also stores its float gradients); emit = true, after
// launch_finish_scales: grad receives the fixed-point integers int2[N] (pair) or int[N].
// The integers are dithered (see to_fixed in objective.cu): row0 = index of the first row in
// the whole data set, round = the boosting round.
void launch_gradients(int objective, int K, size_t n, const float *y, const unsigned char *label,
                      const float *yhat, void *grad, QuantScale *qs, bool emit, cudaStream_t s,
                      unsigned long long row0, unsigned round, int quant_bits);
// reg:linear only, between the two passes of launch_gradients: the tail counts of |g| below
// the round's maximum (QuantScale::tail)
void launch_gradient_tails(size_t n, const float *y, const float *yhat, QuantScale *qs, cudaStream_t s);
// stage 0: the scales from the maxima (and, `tails`, from the tail counts); stage 1: only this
// rank's scale exponent into qs->neg_s (row shards then take the maximum over the ranks);
// stage 2: the scales from qs->neg_s
void launch_finish_scales(QuantScale *qs, int K, int quant_bits, bool pair, cudaStream_t s, bool tails = false,
                          int stage = 0);
// float gradients -> fixed-point integers, in place, rounded to nearest
// (g_q = rint(g * sg), h_q = max(1, rint(h * sh)))
void launch_quantize_grads(void *grad, size_t n, bool pair, const QuantScale *qs, int quant_bits,
                           cudaStream_t s);

struct LeafLaunch {
  const NodeRec *last_rec;
  int L;  // nodes of the last level
  float *leaf_w;  // 2L
  const QuantScale *qs;
  float mcw;
  unsigned mls;
  float lambda, alpha, mlw, eta;
  bool pair;
  bool counts = false;  // last_rec carries true row counts (lcnt, tcnt)
};
void launch_leaf_weights(const LeafLaunch &a, cudaStream_t s);

// inference over raw fp32 rows (RegTree::Predict of the reference, on the device)
struct PackedTree {  // device arrays of one forest
  const int *fid;        // [trees][nodes]
  const float *thr;      // [trees][nodes]
  const float *weights;  // [trees][leaves]
  const int *label;      // [trees]
  const unsigned *category = nullptr;  // [trees][nodes], read for nodes with fid >= F
};
// out[label * plane_stride + row] += leaf weight (plane_stride 0 = n).  A node with fid >= F
// tests the categorical column fid - F of `cat` (row-major [n][ccol]) for equality.
void launch_predict(const float *X, size_t n, int F, PackedTree t, int first_tree, int n_trees,
                    int depth, float *out /*[K][plane_stride]*/, cudaStream_t s, size_t plane_stride = 0,
                    const unsigned *cat = nullptr, int ccol = 0);
void launch_fill(float *dst, size_t n, float value, cudaStream_t s);
void launch_fill_u32(unsigned *dst, size_t n, unsigned value, cudaStream_t s);
void launch_link(int objective, int K, size_t n, const float *internal /*[K][n]*/,
                 float *out /*[n][K]*/, cudaStream_t s);

// --- quantizer ---------------------------------------------------------------------
// thresholds of one sorted column (device) -> thr[hist_size]
void launch_thresholds(const float *sorted, size_t n, int hist_size, float *thr, unsigned *scratch,
                       cudaStream_t s);
// the same for nf columns of n sorted values each (sorted_cols[c * n + i]): thresholds of
// column c to thr + c * hist_size; scratch of nf x thresholds_scratch_words(n) words
void launch_thresholds_columns(const float *sorted_cols, size_t n, int nf, int hist_size, float *thr,
                               unsigned *scratch, cudaStream_t s);
size_t thresholds_scratch_words(size_t n);
// bin every (row, feature) of a row-major fp32 matrix
void launch_binning(const float *X, size_t n, int F, const float *thr /*[F][hist_size]*/,
                    const int *fsize, int hist_size, bool missing_bin, unsigned char *bins,
                    size_t pitch, int bin_bytes, cudaStream_t s);
// bin ids of the categorical columns ([n][ccol], BIN_T wide) into columns f0 .. f0 + ccol - 1
// of the padded row-major bin matrix
void launch_place_columns(const void *src, size_t n, int ccol, int f0, unsigned char *bins, size_t pitch,
                          int bin_bytes, cudaStream_t s, bool by_column = false);
// row-major padded bins -> feature-major copy
void launch_transpose_bins(const unsigned char *bins, size_t pitch, int bin_bytes, size_t n, int F,
                           unsigned char *bins_cm, cudaStream_t s);
// caller's unpadded uint8 rows -> the padded row-major layout (pitch a multiple of 4)
void launch_pad_rows(const unsigned char *raw, int F, size_t n, unsigned char *bins, size_t pitch,
                     cudaStream_t s);
void launch_u8_to_f32(const unsigned char *src, float *dst, size_t count, cudaStream_t s);
// columns [f0, f0 + nf) of a row-major fp32 matrix as contiguous columns out[(f - f0) * n + row]
void launch_transpose_columns(const float *X, size_t n, int F, int f0, int nf, float *out,
                              cudaStream_t s);
// sorts n fp32 keys (radix order); tmp sizes itself on first use unless it already holds
// sort_floats_temp_bytes(n) bytes
size_t sort_floats_temp_bytes(size_t n);
void sort_floats(const float *in, float *out, size_t n, DevBuf &tmp, cudaStream_t s);
// nf columns of n values each, cols[c * n + r], every column sorted in place in the same
// order sort_floats gives, in one pass of the library's sort over 64-bit (column, value) keys;
// keys_a and keys_b hold n * nf keys each, tmp grows to sort_columns_temp_bytes(n, nf)
size_t sort_columns_temp_bytes(size_t n, int nf);
void sort_columns(float *cols, size_t n, int nf, unsigned long long *keys_a, unsigned long long *keys_b,
                  DevBuf &tmp, cudaStream_t s);

}  // namespace arb
