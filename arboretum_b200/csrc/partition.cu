// Row partition / node assignment (row P of the hot path; replaces set_segment,
// CreatePartitioningIndexes + scatter_kernel and apply_split of the reference:
// src/core/garden.cu:32-43,255-294, src/core/partition.cuh:20-206,
// src/core/builder.h:51-59,107-123,287-300).
//
// The binned matrix never moves.  Each level keeps a list of row ids grouped by
// node (`node_begin` are the prefix counts, like parent_node_count in the
// reference) and a level step splits every node's piece of the list into its two
// children with a stable partition: rows whose bin of the split feature is
// <= the split bin go left (builder.h:113-120), both sides keep their order, so
// row ids stay ascending inside every node and gathers stay local.  The
// observable contract of the reference -- per-level node row counts and the leaf
// every row ends in -- is the same; its physical order (rights reversed) is not
// observable and is not reproduced.
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
    w.node = node_id[lo];
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

__device__ __forceinline__ int block_exclusive_scan(int v, int *warp_sums, int &total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  int off = 0, tot = 0;
  for (int w = 0; w < kPartThreads / 32; ++w) {
    const int s = warp_sums[w];
    if (w < warp) off += s;
    tot += s;
  }
  total = tot;
  __syncthreads();
  return off + incl - v;
}

// pass 1: decision flag of every row and the number of lefts of every item
template <typename BIN_T>
__global__ void __launch_bounds__(kPartThreads)
partition_count_kernel(const unsigned char *__restrict__ bins, const size_t pitch,
                       const unsigned *__restrict__ rowid, unsigned char *__restrict__ flags,
                       unsigned *__restrict__ item_left, const NodeRec *__restrict__ rec,
                       const WorkItem *__restrict__ items, const int *__restrict__ n_items) {
  __shared__ int warp_sums[kPartThreads / 32];
  if (int(blockIdx.x) >= *n_items) return;
  const WorkItem item = items[blockIdx.x];
  const int fid = rec[item.node].fid;
  const int split_bin = rec[item.node].bin;
  int lefts = 0;
  const unsigned t0 = threadIdx.x * kRowsPerThread;
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const unsigned off = t0 + k;
    if (off < item.len) {
      const unsigned pos = item.begin + off;
      unsigned char right = 0;
      if (fid >= 0) {
        const unsigned rid = rowid ? rowid[pos] : pos;
        const int b = reinterpret_cast<const BIN_T *>(bins + size_t(rid) * pitch)[fid];
        right = b > split_bin;
      }
      flags[pos] = right;
      lefts += !right;
    }
  }
  for (int o = 16; o > 0; o >>= 1) lefts += __shfl_down_sync(0xffffffffu, lefts, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = lefts;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < kPartThreads / 32; ++w) s += warp_sums[w];
    item_left[blockIdx.x] = s;
  }
}

// pass 2: one warp per node turns item counts into offsets and writes the next
// level's prefix counts (count_next[2n+1] = left end, [2n+2] = node end:
// hist_tree_grower.cu:80-83)
__global__ void partition_scan_kernel(unsigned *__restrict__ item_left,
                                      const int *__restrict__ item_first,
                                      const unsigned *__restrict__ node_begin,
                                      unsigned *__restrict__ node_begin_next,
                                      NodeRec *__restrict__ rec, int L) {
  const int node = blockIdx.x;
  const int lane = threadIdx.x;
  unsigned carry = 0;
  const int first = item_first[node], last = item_first[node + 1];
  for (int base = first; base < last; base += 32) {
    const int i = base + lane;
    const unsigned v = i < last ? item_left[i] : 0u;
    unsigned incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (i < last) item_left[i] = carry + incl - v;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) {
    node_begin_next[2 * node] = node_begin[node];
    node_begin_next[2 * node + 1] = node_begin[node] + carry;
    if (node == L - 1) node_begin_next[2 * L] = node_begin[L];
    rec[node].left_count = carry;
  }
}

// pass 3: stable scatter of the row ids into the two children
__global__ void __launch_bounds__(kPartThreads)
partition_scatter_kernel(const unsigned *__restrict__ rowid_src, unsigned *__restrict__ rowid_dst,
                         const unsigned char *__restrict__ flags,
                         const unsigned *__restrict__ item_left_excl,
                         const unsigned *__restrict__ node_begin,
                         const unsigned *__restrict__ node_begin_next,
                         const WorkItem *__restrict__ items, const int *__restrict__ n_items) {
  __shared__ int warp_sums[kPartThreads / 32];
  if (int(blockIdx.x) >= *n_items) return;
  const WorkItem item = items[blockIdx.x];
  const unsigned t0 = threadIdx.x * kRowsPerThread;
  unsigned rid[kRowsPerThread];
  unsigned char fl[kRowsPerThread];
  int lefts = 0, valid = 0;
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    const unsigned off = t0 + k;
    fl[k] = 0;
    rid[k] = 0;
    if (off < item.len) {
      const unsigned pos = item.begin + off;
      rid[k] = rowid_src ? rowid_src[pos] : pos;
      fl[k] = flags[pos];
      lefts += !fl[k];
      ++valid;
    }
  }
  int total;
  const int lo = block_exclusive_scan(lefts, warp_sums, total);
  const int ro = int(min(t0, item.len)) - lo;
  const unsigned nb = node_begin[item.node];
  const unsigned left_excl = item_left_excl[blockIdx.x];
  const unsigned right_begin = node_begin_next[2 * item.node + 1];
  unsigned ldst = nb + left_excl + lo;
  unsigned rdst = right_begin + (item.begin - nb - left_excl) + ro;
#pragma unroll
  for (int k = 0; k < kRowsPerThread; ++k) {
    if (k < valid) {
      if (fl[k]) rowid_dst[rdst++] = rid[k]; else rowid_dst[ldst++] = rid[k];
    }
  }
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

void launch_partition(const PartitionLaunch &a, cudaStream_t s) {
  launch_plan_partition(a.node_begin, a.L, a.pb, a.max_items, s);
  if (a.geo.bin_bytes == 1)
    partition_count_kernel<unsigned char><<<a.max_items, kPartThreads, 0, s>>>(
      a.geo.bins, a.geo.pitch, a.rowid_src, a.flags, a.item_left, a.rec, a.pb.part_items,
      a.pb.n_part_items);
  else
    partition_count_kernel<unsigned short><<<a.max_items, kPartThreads, 0, s>>>(
      a.geo.bins, a.geo.pitch, a.rowid_src, a.flags, a.item_left, a.rec, a.pb.part_items,
      a.pb.n_part_items);
  ARB_CUDA(cudaGetLastError());
  count_launch();
  partition_scan_kernel<<<a.L, 32, 0, s>>>(a.item_left, a.pb.part_item_first, a.node_begin,
                                           a.node_begin_next, a.rec, a.L);
  ARB_CUDA(cudaGetLastError());
  count_launch();
  partition_scatter_kernel<<<a.max_items, kPartThreads, 0, s>>>(
    a.rowid_src, a.rowid_dst, a.flags, a.item_left, a.node_begin, a.node_begin_next,
    a.pb.part_items, a.pb.n_part_items);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

}  // namespace arb
