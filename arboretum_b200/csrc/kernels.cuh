// Launchers of the level-loop kernels.  All of them enqueue on the given stream
// and never synchronise; sizes that depend on the data (node sizes, work-item
// counts) live in device memory and are read by the kernels themselves.
#pragma once
#include <cuda_runtime.h>

#include "common.cuh"
#include "gain.cuh"

namespace arb {

constexpr int kHistWords = 8192;      // words of one shared-memory histogram plane
constexpr int kHistThreads = 256;     // threads of a histogram CTA
constexpr int kPartRows = 2048;       // rows of one partition work item
constexpr int kPartThreads = 256;
constexpr int kMaxLevels = 16;
constexpr int kMinItemRows = 2048;    // smallest piece a node's row list is cut into

// Geometry of the binned matrix and of the histograms built from it.
//   bins : row-major, `pitch` bytes per row, feature f of row r at
//          bins[r * pitch + f * bin_bytes]; pitch is a multiple of 32.
//   tiles: TW consecutive features; TW * BINS == kHistWords, so one tile of one
//          node is kHistWords (g, h) pairs: hist[((node * NT + tile) * BINS + bin) * TW + lane]
struct Geometry {
  const unsigned char *bins;
  size_t pitch;
  int bin_bytes;
  int F;
  int TW, NT, BINS;
  int hist_size;  // bins a split may use (config value); id hist_size = missing
  // optional feature-major copy bins_cm[f * cm_rows + row] (nullptr: absent): the row
  // partition reads one feature of many rows, which is sequential in this layout
  const unsigned char *bins_cm = nullptr;
  size_t cm_rows = 0;
};

struct HistLaunch {
  Geometry geo;
  const unsigned *rowid;  // nullptr: positions are row ids (root level)
  const void *grad;       // quantised gradients: int2[N] (pair) or int[N]
  bool pair;
  const WorkItem *items;  // every item has at most 2^(31 - quant_bits) rows
  const int *n_items;
  int max_items;
  int *partials;  // [item][tile][2][kHistWords] int32 planes, written here
};
void launch_hist(const HistLaunch &a, cudaStream_t s);
int hist_grid_x(int max_items, int NT);

// planes of the items of every built node -> the level's int64 histogram
struct ReduceLaunch {
  const int *partials;
  const int *item_first;  // n_build + 1: items of built node b are [first[b], first[b+1])
  const int *build_node;  // node index (inside the level) of built node b
  int n_build;
  int NT;
  long long *level_hist;
  const long long *parent_hist;  // level above, for the subtraction
  bool subtract;      // also write sibling = parent - built
  bool zero_sibling;  // (no subtract) clear the sibling so the buffer can be all-reduced
  int level_nodes;    // nodes of the level (size of level_hist)
  const int *built_child;  // per parent: which child was built (for the subtraction)
  bool accumulate = false;  // add into level_hist (cleared by the caller): row chunks of one level
};
void launch_reduce(const ReduceLaunch &a, cudaStream_t s);

// sibling = parent - built child, for every parent of the level above
void launch_subtract(long long *level_hist, const long long *parent_hist, const int *built_child,
                     int n_parents, int NT, cudaStream_t s);

struct SplitLaunch {
  Geometry geo;
  const long long *hist;       // level buffer
  const unsigned *node_begin;  // L+1 prefix counts of this level
  const unsigned char *feature_active;  // F flags: evaluated at this level
  const int *feature_size;     // bins in use per feature
  unsigned long long *keys;    // max_nodes packed (gain, feature, bin) maxima followed by
                               // max_nodes u32 arrival counters; zeroed here
  int max_nodes;
  NodeRec *rec;                // L records out
  const NodeRec *parent_rec;   // level above (nullptr at the root)
  const QuantScale *qs;
  GainParams gp;
  bool pair;
  int L;
};
void launch_split(const SplitLaunch &a, cudaStream_t s);

// --- row partition ----------------------------------------------------------
struct PlanBuffers {
  WorkItem *part_items;
  int *n_part_items;
  int *part_item_first;  // per node of the level: first item, L+1 entries
  WorkItem *hist_items;
  int *n_hist_items;
  int *hist_item_first;  // scratch, max_nodes + 1
  int *built_child;  // per parent: 0 = left child built, 1 = right child
  unsigned *scratch_begin, *scratch_len;  // scratch, max_nodes each
  int *scratch_node;
};
// items of the partition pass over the nodes of `level`
void launch_plan_partition(const unsigned *node_begin, int L, PlanBuffers pb, int max_items,
                           cudaStream_t s);
// choose which child of every parent to build and cut those children into items
void launch_plan_hist(const unsigned *node_begin, const NodeRec *parent_rec, int L, int item_rows,
                      bool use_trick, bool by_hessian, PlanBuffers pb, int max_items,
                      cudaStream_t s);

struct PartitionLaunch {
  Geometry geo;
  const unsigned *rowid_src;  // nullptr: identity (root)
  unsigned *rowid_dst;
  unsigned *cursors;          // 2 per node: rows placed so far in the left / right child
  const unsigned *node_begin; // level L prefix counts
  unsigned *node_begin_next;  // 2L+1 prefix counts out
  NodeRec *rec;               // split records of the level (left_count filled)
  PlanBuffers pb;
  int L;
  int max_items;
  unsigned n_rows;
  const unsigned *go_right = nullptr;  // bit per row from launch_descend (nullptr: the kernel
                                       // reads the split feature's bin itself)
};
void launch_partition(const PartitionLaunch &a, cudaStream_t s);

// One step of every row down the tree, in row order (see descend_kernel).
struct DescendLaunch {
  Geometry geo;
  const NodeRec *rec;        // split records of the level the rows stand on
  int L;                     // nodes of that level
  unsigned short *node_of;   // per row: its node inside the level; becomes the child's (L == 1:
                             // not read, every row stands on the root)
  unsigned *go_right;        // bit per row, written here; nullptr = the final step, which adds
  const float *leaf_w;       //   leaf_w[child] to
  float *yhat;               //   yhat[row] instead
  size_t n;
};
void launch_descend(const DescendLaunch &a, cudaStream_t s);
// next level's prefix counts and the split records' left row counts from the cursors
void launch_partition_finish(const unsigned *cursors, const unsigned *node_begin,
                             unsigned *node_begin_next, NodeRec *rec, int L, cudaStream_t s);

// --- fused level step (one-tile uint8 data): partition of level l-1 + histogram of level l
// items are pieces of the parents' row lists; the built child of every parent is
// chosen from the parent's split record (smaller hessian sum, ties left)
void launch_plan_fused(const unsigned *parent_begin, const NodeRec *parent_rec, int n_parents,
                       int item_rows, PlanBuffers pb, int max_items, cudaStream_t s);
struct FusedLaunch {
  Geometry geo;
  const unsigned *rowid_src;  // nullptr: identity (parents are the root)
  unsigned *rowid_dst;
  const void *grad;
  bool pair;
  const WorkItem *items;
  const int *n_items;
  int max_items;
  const NodeRec *parent_rec;
  const int *built_child;
  const unsigned *parent_begin;
  unsigned *cursors;  // 2 per parent, zeroed by the launcher
  int n_parents;
  int *partials;
};
void launch_fused(const FusedLaunch &a, cudaStream_t s);

// --- objective, leaves, prediction ----------------------------------------------
// grad from (y, yhat); also tracks max|g|, max h in qs
void launch_gradients(int objective, int K, size_t n, const float *y, const unsigned char *label,
                      const float *yhat, void *grad, QuantScale *qs, cudaStream_t s);
void launch_finish_scales(QuantScale *qs, int K, int quant_bits, bool pair, cudaStream_t s);
// float gradients -> fixed-point integers, in place (g_q = rint(g * sg), h_q = max(1, rint(h * sh)))
void launch_quantize_grads(void *grad, size_t n, bool pair, const QuantScale *qs, cudaStream_t s);

struct LeafLaunch {
  const NodeRec *last_rec;
  int L;  // nodes of the last level
  float *leaf_w;  // 2L
  const QuantScale *qs;
  float mcw;
  unsigned mls;
  float lambda, alpha, mlw, eta;
  bool pair;
};
void launch_leaf_weights(const LeafLaunch &a, cudaStream_t s);

// yhat[row] += leaf weight of the tree just grown, walking the tree over bins
void launch_update_yhat(const Geometry &geo, const NodeRec *rec /*[levels][max_nodes]*/,
                        int levels, int max_nodes, const float *leaf_w, float *yhat, size_t n,
                        cudaStream_t s);

// inference over raw fp32 rows (RegTree::Predict of the reference, on the device)
struct PackedTree {  // device arrays of one forest
  const int *fid;        // [trees][nodes]
  const float *thr;      // [trees][nodes]
  const float *weights;  // [trees][leaves]
  const int *label;      // [trees]
};
void launch_predict(const float *X, size_t n, int F, PackedTree t, int first_tree, int n_trees,
                    int depth, float *out /*[K][n]*/, cudaStream_t s);
void launch_fill(float *dst, size_t n, float value, cudaStream_t s);
void launch_link(int objective, int K, size_t n, const float *internal /*[K][n]*/,
                 float *out /*[n][K]*/, cudaStream_t s);

// --- quantizer ---------------------------------------------------------------------
// thresholds of one sorted column (device) -> thr[hist_size]
void launch_thresholds(const float *sorted, size_t n, int hist_size, float *thr, unsigned *scratch,
                       cudaStream_t s);
size_t thresholds_scratch_words(size_t n);
// bin every (row, feature) of a row-major fp32 matrix
void launch_binning(const float *X, size_t n, int F, const float *thr /*[F][hist_size]*/,
                    const int *fsize, int hist_size, bool missing_bin, unsigned char *bins,
                    size_t pitch, int bin_bytes, cudaStream_t s);
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
// sorts n fp32 keys (radix order); tmp sizes itself on first use
void sort_floats(const float *in, float *out, size_t n, DevBuf &tmp, cudaStream_t s);

}  // namespace arb
