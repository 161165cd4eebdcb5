// Row partition / node assignment (row P of the hot path; replaces set_segment,
// CreatePartitioningIndexes + scatter_kernel and apply_split of the reference:
// src/core/garden.cu:32-43,255-294, src/core/partition.cuh:20-206,
// src/core/builder.h:51-59,107-123,287-300).
//
// The binned matrix never moves.  Each level keeps a list of row ids grouped by
// node (`node_begin` are the prefix counts, like parent_node_count in the
// reference) and a level step splits every node's piece of the list into its two
// children: rows whose bin of the split feature is <= the split bin go left
// (builder.h:113-120); inside every 2048-row piece both sides keep their order,
// so row ids stay ascending in long runs and gathers stay local.  The
// observable contract of the reference -- per-level node row counts and the leaf
// every row ends in -- is the same; its physical order (rights reversed) is not
// observable and is not reproduced.
#include <algorithm>

#include "kernels.cuh"

namespace arb {

namespace {

constexpr int kRowsPerThread = kPartRows / kPartThreads;  // 8

// first[n] = first item of node n, items of `rows_per_item` rows; one CTA.
__device__ void make_items(const unsigned *begin, const unsigned *len, const int *node_id,
                           int n_nodes, int rows_per_item, int *first, WorkItem *items,
                           int *n_items, int max_items) {
  __shared__ int total;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < n_nodes; ++i) {
      first[i] = run;
      run += int((len[i] + rows_per_item - 1) / rows_per_item);
    }
    first[n_nodes] = run;
    total = run < max_items ? run : max_items;
    *n_items = total;
  }
  __syncthreads();
  for (int it = threadIdx.x; it < total; it += blockDim.x) {
    int lo = 0, hi = n_nodes;  // last node with first[node] <= it
    while (hi - lo > 1) {
      const int mid = (lo + hi) / 2;
      if (first[mid] <= it) lo = mid; else hi = mid;
    }
    const unsigned off = unsigned(it - first[lo]) * rows_per_item;
    WorkItem w;
    w.begin = begin[lo] + off;
    w.len = min(unsigned(rows_per_item), len[lo] - off);
    w.node = node_id ? node_id[lo] : lo;
    w.pad = 0;
    items[it] = w;
  }
}

__global__ void plan_partition_kernel(const unsigned *__restrict__ node_begin, int L, PlanBuffers pb,
                                      unsigned *sb, unsigned *sl, int *sn, int max_items) {
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    sb[i] = node_begin[i];
    sl[i] = node_begin[i + 1] - node_begin[i];
    sn[i] = i;
  }
  __syncthreads();
  make_items(sb, sl, sn, L, kPartRows, pb.part_item_first, pb.part_items, pb.n_part_items,
             max_items);
}

__global__ void plan_hist_kernel(const unsigned *__restrict__ node_begin,
                                 const NodeRec *__restrict__ parent_rec, int L, int item_rows,
                                 bool use_trick, bool by_hessian, PlanBuffers pb, unsigned *sb,
                                 unsigned *sl, int *sn, int *first, int max_items) {
  int n_build;
  if (use_trick && L > 1) {
    n_build = L / 2;
    for (int p = threadIdx.x; p < n_build; p += blockDim.x) {
      const unsigned ls = node_begin[2 * p + 1] - node_begin[2 * p];
      const unsigned rs = node_begin[2 * p + 2] - node_begin[2 * p + 1];
      int built;
      if (by_hessian) {  // identical on every rank: decided from the global sums
        const long long lh = parent_rec[p].lh, rh = parent_rec[p].th - parent_rec[p].lh;
        built = lh <= rh ? 0 : 1;
      } else {  // smaller child, ties build the left one (hist_grad_sum.cu:288-290)
        built = ls <= rs ? 0 : 1;
      }
      pb.built_child[p] = built;
      const int node = 2 * p + built;
      sb[p] = node_begin[node];
      sl[p] = built ? rs : ls;
      sn[p] = node;
    }
  } else {
    n_build = L;
    for (int i = threadIdx.x; i < L; i += blockDim.x) {
      sb[i] = node_begin[i];
      sl[i] = node_begin[i + 1] - node_begin[i];
      sn[i] = i;
    }
  }
  __syncthreads();
  make_items(sb, sl, sn, n_build, item_rows, first, pb.hist_items, pb.n_hist_items, max_items);
}

// items over the parents of a fused level step; built child = smaller hessian sum
__global__ void plan_fused_kernel(const unsigned *__restrict__ parent_begin,
                                  const NodeRec *__restrict__ parent_rec, int n_parents, int item_rows,
                                  PlanBuffers pb, unsigned *sb, unsigned *sl, int *build_node,
                                  int *first, int max_items) {
  for (int p = threadIdx.x; p < n_parents; p += blockDim.x) {
    const long long lh = parent_rec[p].lh, rh = parent_rec[p].th - parent_rec[p].lh;
    const int built = lh <= rh ? 0 : 1;
    pb.built_child[p] = built;
    build_node[p] = 2 * p + built;
    sb[p] = parent_begin[p];
    sl[p] = parent_begin[p + 1] - parent_begin[p];
  }
  __syncthreads();
  make_items(sb, sl, nullptr, n_parents, item_rows, first, pb.hist_items, pb.n_hist_items, max_items);
}

// One pass per level: every CTA takes one item (a piece of one node's row list),
// decides left / right for its rows (left <=> bin of the split feature <= split
// bin, builder.h:113-120), orders them in shared memory (lefts first, both sides
// in list order) and reserves room in the two children with one atomicAdd per
// side: lefts grow upwards from the node's begin, rights downwards from its end,
// so both children are contiguous without knowing their sizes in advance.  The
// order of the items inside a child depends on scheduling; nothing observable
// does, because every sum over rows is an exact integer sum.
template <typename BIN_T>
__global__ void __launch_bounds__(kPartThreads)
partition_kernel(const unsigned char *__restrict__ bins, const size_t pitch,
                 const unsigned char *__restrict__ bins_cm, const size_t cm_rows,
                 const unsigned *__restrict__ rowid_src, unsigned *__restrict__ rowid_dst,
                 const NodeRec *__restrict__ rec, const unsigned *__restrict__ node_begin,
                 unsigned *__restrict__ cursors, const WorkItem *__restrict__ items,
                 const int *__restrict__ n_items, const unsigned *__restrict__ go_right) {
  constexpr int kWarps = kPartThreads / 32;
  __shared__ unsigned buf[kPartRows];
  __shared__ int cnt[kRowsPerThread * kWarps];
  __shared__ int pre[kRowsPerThread * kWarps + 1];
  __shared__ unsigned base_l, base_r;
  if (int(blockIdx.x) >= *n_items) return;
  const WorkItem item = items[blockIdx.x];
  const int fid = rec[item.node].fid;
  const int split_bin = rec[item.node].bin;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned rid[kRowsPerThread];
  int before[kRowsPerThread];  // lefts before this element inside its warp round
  unsigned left_bits = 0;
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const unsigned off = k * kPartThreads + threadIdx.x;
    const bool valid = off < item.len;
    rid[k] = 0;
    bool left = false;
    if (valid) {
      rid[k] = rowid_src ? rowid_src[item.begin + off] : item.begin + off;
      left = true;
      if (go_right) {  // decided by the descend step; the bit array stays in L2
        left = ((go_right[rid[k] >> 5] >> (rid[k] & 31)) & 1u) == 0;
      } else if (fid >= 0) {
        const int b = bins_cm ? int(reinterpret_cast<const BIN_T *>(bins_cm)[size_t(fid) * cm_rows + rid[k]])
                              : int(reinterpret_cast<const BIN_T *>(bins + size_t(rid[k]) * pitch)[fid]);
        left = b <= split_bin;
      }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, left);
    before[k] = __popc(bal & ((1u << lane) - 1));
    if (lane == 0) cnt[k * kWarps + warp] = __popc(bal);
    left_bits |= unsigned(left) << k;
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the 64 (round, warp) counts
    constexpr int kN = kRowsPerThread * kWarps;
    const int a = cnt[2 * lane], b = cnt[2 * lane + 1];
    int incl = a + b;
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    static_assert(kN == 64, "two counts per lane");
    pre[2 * lane] = incl - a - b;
    pre[2 * lane + 1] = incl - b;
    if (lane == 31) pre[kN] = incl;
  }
  __syncthreads();
  const int nl = pre[kRowsPerThread * kWarps];
  const int nr = int(item.len) - nl;
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const unsigned off = k * kPartThreads + threadIdx.x;
    if (off < item.len) {
      const int lefts_before = pre[k * kWarps + warp] + before[k];
      if ((left_bits >> k) & 1u)
        buf[lefts_before] = rid[k];
      else
        buf[nl + int(off) - lefts_before] = rid[k];
    }
  }
  if (threadIdx.x == 0) {
    base_l = atomicAdd(&cursors[2 * item.node], unsigned(nl));
    base_r = atomicAdd(&cursors[2 * item.node + 1], unsigned(nr));
  }
  __syncthreads();
  const unsigned ldst = node_begin[item.node] + base_l;
  const unsigned rdst = node_begin[item.node + 1] - base_r - unsigned(nr);
  for (unsigned i = threadIdx.x; i < item.len; i += kPartThreads)
    rowid_dst[int(i) < nl ? ldst + i : rdst + (i - unsigned(nl))] = buf[i];
}

// Every row takes one step down the tree, in row order: its node's split decides left or
// right (left <=> bin of the split feature <= split bin, builder.h:113-120; a node without
// a split keeps its rows on the left).  The step reads each row's node number and one bin
// of the feature-major matrix, both in row order, so DRAM lines are used whole however
// deep the tree is; the row lists are then partitioned from the bit array written here,
// which is small enough to stay in L2.  A warp takes 256 consecutive rows per turn, row
// base + 32 k + lane in pass k, so that every access is coalesced and a lane has eight
// independent loads in flight.
// FINAL: the step below the last level; instead of storing the child, the row's
// prediction receives the child's leaf weight (garden.cu:45-76 of the reference).
constexpr int kDescendPasses = 8;
constexpr int kDescendTable = 2048;

template <typename BIN_T, bool FINAL>
__global__ void __launch_bounds__(256)
descend_kernel(const unsigned char *__restrict__ bins, const size_t pitch,
               const unsigned char *__restrict__ bins_cm, const size_t cm_rows,
               const NodeRec *__restrict__ rec, const int L, unsigned short *__restrict__ node_of,
               unsigned *__restrict__ go_right, const float *__restrict__ leaf_w,
               float *__restrict__ yhat, const size_t n) {
  __shared__ int2 table[kDescendTable];  // (fid, bin) of the level's nodes
  const bool cached = L <= kDescendTable;
  if (cached) {
    for (int i = threadIdx.x; i < L; i += blockDim.x) table[i] = make_int2(rec[i].fid, rec[i].bin);
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const size_t warps = size_t(gridDim.x) * (blockDim.x >> 5);
  const size_t span = size_t(32) * kDescendPasses;
  for (size_t base = (size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * span; base < n;
       base += warps * span) {
    int node[kDescendPasses];
#pragma unroll
    for (int k = 0; k < kDescendPasses; ++k) {
      const size_t r = base + size_t(k) * 32 + lane;
      node[k] = (L > 1 && r < n) ? int(node_of[r]) : 0;
    }
    int binv[kDescendPasses], split_bin[kDescendPasses];
#pragma unroll
    for (int k = 0; k < kDescendPasses; ++k) {
      const size_t r = base + size_t(k) * 32 + lane;
      const int2 fb = cached ? table[node[k]] : make_int2(rec[node[k]].fid, rec[node[k]].bin);
      split_bin[k] = fb.y;
      binv[k] = -1;  // no split, or past the end: left
      if (fb.x >= 0 && r < n)
        binv[k] = bins_cm ? int(reinterpret_cast<const BIN_T *>(bins_cm)[size_t(fb.x) * cm_rows + r])
                          : int(reinterpret_cast<const BIN_T *>(bins + r * pitch)[fb.x]);
    }
    unsigned mine = 0;
#pragma unroll
    for (int k = 0; k < kDescendPasses; ++k) {
      const size_t r = base + size_t(k) * 32 + lane;
      const int right = binv[k] > split_bin[k];
      const int child = 2 * node[k] + right;
      if (FINAL) {
        if (r < n) yhat[r] += leaf_w[child];
      } else {
        if (r < n) node_of[r] = (unsigned short)child;
        const unsigned word = __ballot_sync(0xffffffffu, right);
        if (lane == k) mine = word;
      }
    }
    if (!FINAL && lane < kDescendPasses && base + size_t(lane) * 32 < n) go_right[base / 32 + lane] = mine;
  }
}

// next level's prefix counts (count_next[2n+1] = left end, [2n+2] = node end:
// hist_tree_grower.cu:80-83) and the left row count of every split record
__global__ void partition_finish_kernel(const unsigned *__restrict__ cursors,
                                        const unsigned *__restrict__ node_begin,
                                        unsigned *__restrict__ node_begin_next,
                                        NodeRec *__restrict__ rec, int L) {
  const int node = blockIdx.x * blockDim.x + threadIdx.x;
  if (node >= L) return;
  const unsigned nl = cursors[2 * node];
  node_begin_next[2 * node] = node_begin[node];
  node_begin_next[2 * node + 1] = node_begin[node] + nl;
  if (node == L - 1) node_begin_next[2 * L] = node_begin[L];
  rec[node].left_count += nl;  // cleared by the split search; row chunks add up
}

}  // namespace

void launch_plan_partition(const unsigned *node_begin, int L, PlanBuffers pb, int max_items,
                           cudaStream_t s) {
  plan_partition_kernel<<<1, 256, 0, s>>>(node_begin, L, pb, pb.scratch_begin, pb.scratch_len,
                                          pb.scratch_node, max_items);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_plan_hist(const unsigned *node_begin, const NodeRec *parent_rec, int L, int item_rows,
                      bool use_trick, bool by_hessian, PlanBuffers pb, int max_items,
                      cudaStream_t s) {
  plan_hist_kernel<<<1, 256, 0, s>>>(node_begin, parent_rec, L, item_rows, use_trick, by_hessian,
                                     pb, pb.scratch_begin, pb.scratch_len, pb.scratch_node,
                                     pb.hist_item_first, max_items);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_plan_fused(const unsigned *parent_begin, const NodeRec *parent_rec, int n_parents,
                       int item_rows, PlanBuffers pb, int max_items, cudaStream_t s) {
  plan_fused_kernel<<<1, 256, 0, s>>>(parent_begin, parent_rec, n_parents, item_rows, pb,
                                      pb.scratch_begin, pb.scratch_len, pb.scratch_node,
                                      pb.hist_item_first, max_items);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_descend(const DescendLaunch &a, cudaStream_t s) {
  if (a.n == 0) return;
  const size_t span = size_t(32) * kDescendPasses * (256 / 32);  // rows of one CTA turn
  const int grid = int(std::min<size_t>((a.n + span - 1) / span, size_t(148) * 8));
  const Geometry &g = a.geo;
  const bool fin = a.go_right == nullptr;
#define ARB_LAUNCH(T, FIN)                                                                        \
  descend_kernel<T, FIN><<<grid, 256, 0, s>>>(g.bins, g.pitch, g.bins_cm, g.cm_rows, a.rec, a.L, \
                                              a.node_of, a.go_right, a.leaf_w, a.yhat, a.n)
  if (g.bin_bytes == 1) {
    if (fin) ARB_LAUNCH(unsigned char, true); else ARB_LAUNCH(unsigned char, false);
  } else {
    if (fin) ARB_LAUNCH(unsigned short, true); else ARB_LAUNCH(unsigned short, false);
  }
#undef ARB_LAUNCH
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_partition_finish(const unsigned *cursors, const unsigned *node_begin,
                             unsigned *node_begin_next, NodeRec *rec, int L, cudaStream_t s) {
  partition_finish_kernel<<<ceil_div(L, 128), 128, 0, s>>>(cursors, node_begin, node_begin_next, rec, L);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_partition(const PartitionLaunch &a, cudaStream_t s) {
  launch_plan_partition(a.node_begin, a.L, a.pb, a.max_items, s);
  ARB_CUDA(cudaMemsetAsync(a.cursors, 0, 2 * sizeof(unsigned) * a.L, s));
  if (a.geo.bin_bytes == 1)
    partition_kernel<unsigned char><<<a.max_items, kPartThreads, 0, s>>>(
      a.geo.bins, a.geo.pitch, a.geo.bins_cm, a.geo.cm_rows, a.rowid_src, a.rowid_dst, a.rec,
      a.node_begin, a.cursors,
      a.pb.part_items, a.pb.n_part_items, a.go_right);
  else
    partition_kernel<unsigned short><<<a.max_items, kPartThreads, 0, s>>>(
      a.geo.bins, a.geo.pitch, a.geo.bins_cm, a.geo.cm_rows, a.rowid_src, a.rowid_dst, a.rec,
      a.node_begin, a.cursors,
      a.pb.part_items, a.pb.n_part_items, a.go_right);
  ARB_CUDA(cudaGetLastError());
  count_launch();
  launch_partition_finish(a.cursors, a.node_begin, a.node_begin_next, a.rec, a.L, s);
}

}  // namespace arb
