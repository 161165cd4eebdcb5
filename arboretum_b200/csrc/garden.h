// Host-side objects behind the C ABI: DataMatrix (src/io/io.h:15-83 of the
// reference) and Garden (src/core/garden.h:141-160), rebuilt around a device
// resident, row-major bin matrix and a level loop that never returns to the host
// inside a tree.
#pragma once
#include <cstdint>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "common.cuh"
#include "config.h"
#include "kernels.cuh"

namespace arb {

// Row shards (one process per GPU): what InitHist needs to find the thresholds of the WHOLE
// data set.  allgather(ctx, send, recv, bytes, stream): every rank contributes `bytes`
// bytes from device memory; recv (device) receives world x bytes in rank order.
typedef int (*AllgatherFn)(void *ctx, const void *send, void *recv, size_t bytes, cudaStream_t stream);
struct ShardInfo {
  int rank = 0, world = 1;
  AllgatherFn allgather = nullptr;
  void *ctx = nullptr;
};

class DataMatrix {
 public:
  DataMatrix(int64_t rows, int cols_dense, int cols_cat)
      : rows(rows), cols_dense(cols_dense), cols_cat(cols_cat) {}

  int64_t rows;
  int cols_dense;
  int cols_cat;
  std::vector<float> x;  // dense features, row-major copy of the caller's matrix (only when
                         // the device copy below could not be made)
  DevBuf d_x;            // the same matrix in HBM, uploaded at construction
  int device = -1;       // device that holds d_x
  std::vector<float> y;  // targets on the host (only when the matrix is not in HBM)
  std::vector<unsigned char> labels;
  DevBuf d_y, d_labels;  // targets in HBM, uploaded by ASetY / ASetLabel beside the matrix
  bool has_y() const { return d_y.p || y.size() == size_t(rows); }
  bool has_labels() const { return d_labels.p || labels.size() == size_t(rows); }
  std::vector<float> weights;
  // categorical columns (arboretum_wrapper.cu:30-33): category codes, row-major [rows][cols_cat],
  // on the host (for the quantiser) and on the device (for inference).  Feature ids
  // cols_dense .. cols_dense + cols_cat - 1 denote them, as in the reference (garden.h:79-84).
  std::vector<unsigned> cat;
  DevBuf d_cat;
  int cols() const { return cols_dense + cols_cat; }
  // Quantised categorical column c: the categories that got a bin of their own, most
  // frequent first (ties: smaller code first), bin id = position; when a column has more
  // categories than bins, the rest share the bin after them, which no split can single out.
  std::vector<std::vector<unsigned>> cat_codes;
  std::vector<int> cat_candidates;  // per feature (dense and categorical): bins a one-vs-rest
                                    // split may name; 0 for dense features
  void BinCategories(cudaStream_t s);

  // quantised form (built by the first AGrowTree, like DataMatrix::InitHist)
  bool binned = false;
  bool prebinned = false;
  bool thresholds_given = false;
  int hist_size = 0;
  int bin_bytes = 1;
  size_t pitch = 0;
  DevBuf d_bins;
  DevBuf d_bins_cm;  // feature-major copy for the descend step (in-core only)
  // out-of-core: the row-major bin matrix in pinned host memory, rows of host_pitch bytes.  The
  // device wants rows padded to 32 bytes; where that padding is an eighth of a row or more
  // (100 features: 128 against 100 bytes) the host rows go without it, so that it does not
  // cross the host link once per level, and a kernel pads every chunk on arrival.
  PinnedBuf h_bins;
  size_t host_pitch = 0;
  static size_t HostPitchFor(int F, int bin_bytes) {
    const size_t padded = PitchFor(F, bin_bytes), tight = (size_t(F) * bin_bytes + 3) / 4 * 4;
    return padded - tight >= padded / 8 ? tight : padded;
  }
  bool out_of_core = false;
  std::vector<float> thr;  // [F][hist_size] data_reduced_mapping
  std::vector<int> fsize;  // bins in use per feature
  int max_reduced_bits = 0;
  std::vector<unsigned char> host_bins;  // caller's pre-binned rows (row-major), if they were not
                                         // uploaded at construction
  DevBuf d_raw;  // caller's pre-binned rows in HBM, unpadded [rows][cols]

  // predictions accumulated by AAppendLastTree, internal scale, [K][rows]
  DevBuf d_yhat;
  int yhat_planes = 0;

  void InitHist(int hist_size, bool missing_bin, bool verbose, cudaStream_t s, long long chunk_rows = 0,
                const ShardInfo *shards = nullptr);
  void ShardedThresholds(const float *d_x_local, int hs, const ShardInfo &sh, cudaStream_t s);
  static size_t PitchFor(int F, int bin_bytes) {
    return (size_t(F) * bin_bytes + 31) / 32 * 32;
  }
};

struct TreeNode {  // reg_tree.h:16-38
  int fid = 0;
  float threshold = 0.0f;
  unsigned quantized = 0;
  bool categorical = false;  // the test is `value == category` (garden.h:79-84)
  unsigned category = unsigned(-1);
};
struct Tree {  // reg_tree.h:40-45 + RegTree::label
  int depth = 0;
  int label = 0;
  std::vector<TreeNode> nodes;  // heap order, (1 << depth) - 1
  std::vector<float> weights;   // 1 << (depth - 1), already multiplied by eta
};

// Optional exchange step of multi-GPU training: sums `count` int64 values in
// place across all ranks, ordered on `stream`.  Returns 0 on success.
typedef int (*AllreduceFn)(void *ctx, long long *device_buf, size_t count, cudaStream_t stream);
// The other exchange: element-wise maximum of `count` uint32 values over all ranks (the
// bit patterns of the round's largest |gradient| and hessian, which fix the fixed-point
// scale: every rank must quantise with the same one).
typedef int (*AllreduceMaxFn)(void *ctx, unsigned *device_buf, size_t count, cudaStream_t stream);

// Health of the communicator behind `allreduce`, asked by the host while it waits for a tree:
// 0 = fine; otherwise `msg` says what the library reported and the communicator has been
// aborted (so that the kernels waiting in it end and the stream can be synchronised).
// `give_up` != 0: abort it in any case (the host's time limit ran out).
typedef int (*CommCheckFn)(void *ctx, int give_up, char *msg, size_t msg_len);

struct PhaseTimes {  // CUDA-event time per kernel class, milliseconds
  // (partition = the descend steps, plan = plan kernel + row lists, update = the final descend)
  double grad = 0, hist = 0, subtract = 0, split = 0, partition = 0, plan = 0, update = 0, allreduce = 0;
  double hist_kernel = 0;  // of `hist`: the histogram kernel's launches alone (the rest is the
                           // reduction of their planes)
  long long hist_launches = 0;
  double hist_rows = 0;      // rows scanned by histogram launches
  double hist_features = 0;  // features per scanned row (summed per launch)
  double hist_bytes = 0;     // algorithmic bytes of those launches
  long long trees = 0;
  double tree = 0;       // whole GrowTree calls, device time
  double enqueue = 0;    // host wall time of GrowTree up to the wait for the tree: launching the kernels
  double host_wait = 0;  // host wall time of that wait (the device is behind the host for this long)
  long long host_trees = 0;
  double h2d_bytes = 0;  // bins streamed from pinned host memory (out-of-core)
};

class Builder;
class Garden;

// Read-only window on the builder's state of the last grown tree, for the
// read-back entry points of the C ABI.
struct BuilderView {
  // records of tree `tree_in_round` (0 .. labels_count - 1; -1 = the last one) of the last round
  static const NodeRec *host_rec(const Garden *g, int tree_in_round, int *max_nodes, int *levels);
  static const unsigned *host_node_begin(const Garden *g, int tree_in_round, int *stride);
  static void scales(Garden *g, QuantScale *out);
  static void train_yhat(Garden *g, float *out);
  // device time of the peer-memory exchanges so far (see PeerExchange::Clock); false: none in use
  static bool exchange_clock(Garden *g, double ms[3], long long *exchanges, bool reset);
};

class Garden {
 public:
  explicit Garden(const Configuration &cfg);
  ~Garden();
  Configuration cfg;
  void GrowTree(DataMatrix *data, const float *grad);
  void Predict(DataMatrix *data, std::vector<float> &out, int n_rounds);
  void UpdateByLastTree(DataMatrix *data);
  void GetY(DataMatrix *data, std::vector<float> &out);
  std::string GetModel() const;
  void Restore(const char *json_model);
  float InternalInitialY() const;

  std::vector<Tree> trees;
  int max_fid = -1;  // largest feature id any tree tests: a matrix given to Predict must have it
  AllreduceFn allreduce = nullptr;
  AllreduceMaxFn allreduce_max = nullptr;
  ShardInfo shards;  // rank, world and the all-gather of the sharded quantizer
  void *allreduce_ctx = nullptr;
  CommCheckFn comm_check = nullptr;
  bool profile = false;
  bool peer_exchange = false;  // the level exchange of the row shards runs over peer memory
  PhaseTimes times;
  // device copies of the forest for inference
  void SyncForest();
  void EnsureStream();
  void ReleaseBuilder();
  DevBuf d_fid, d_thr, d_w, d_label, d_category;
  size_t forest_trees_on_device = 0;
  cudaStream_t stream = nullptr;
  Builder *builder = nullptr;
};

}  // namespace arb
