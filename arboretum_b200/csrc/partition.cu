// Node assignment and row lists (row P of the hot path; replaces set_segment,
// CreatePartitioningIndexes + scatter_kernel and apply_split of the reference:
// src/core/garden.cu:32-43,255-294, src/core/partition.cuh:20-206,
// src/core/builder.h:51-59,107-123,287-300).
//
// The binned matrix never moves and no list is carried from level to level.  Every
// row keeps the number of the node it stands on (`node_of`), and a level step is three
// passes in row order, each of them a stream over whole DRAM lines whatever the depth:
//   1. descend: every row steps to a child of its node (left <=> bin of the split
//      feature <= split bin, builder.h:113-120) and the children are counted;
//   2. plan (one CTA): prefix counts of the level (`node_begin`, like parent_node_count
//      in the reference), which child of every parent gets a histogram of its own (the
//      other is parent - built), where the row list of every built node starts, and the
//      work items of the histogram pass;
//   3. lists: the rows of the built nodes -- the only ones a histogram pass reads --
//      are written to their node's list; a CTA reserves room for its rows with one
//      atomicAdd per node it meets.
// The order of the rows inside a list depends on scheduling; nothing observable does,
// because every sum over rows is an exact integer sum.  The observable contract of the
// reference -- per-level node row counts and the leaf every row ends in -- is the same;
// its physical row order is not observable and is not reproduced.
#include <algorithm>

#include "kernels.cuh"

namespace arb {

namespace {

constexpr unsigned kNoList = 0xffffffffu;
constexpr unsigned kCatFlag = 0x8000u;  // in a packed split: the feature is categorical
constexpr int kDescendPasses = 8;   // a warp takes 32 * 8 consecutive rows per turn
constexpr int kSmemNodes = 2048;    // nodes of a level whose tables fit in shared memory
constexpr int kListRows = 2048;     // rows of one CTA of the list pass
constexpr int kListThreads = 256;
constexpr int kPlanThreads = 1024;  // one CTA: its loops over nodes and work items are latency-bound
// Counters that many CTAs add to (children counts, list cursors) sit one per 128-byte line:
// atomics on one line are served one after the other by a single L2 slice, so packed
// counters would serialise every CTA's updates of a whole level.
constexpr int kPad = kCounterStride;
constexpr int kFewNodes = 2;        // descend: up to here a level's right-goers are counted from ballots
constexpr int kFewLists = 4;        // lists: up to here lanes are grouped by node before they take ranks

// out[i] = sum of in[0..i) for i <= n (n + 1 values); one CTA; in place allowed
__device__ void block_exclusive_scan(const unsigned *in, unsigned *out, int n) {
  __shared__ unsigned warp_sums[32];
  const int per = (n + int(blockDim.x) - 1) / int(blockDim.x);
  const int lo = min(n, int(threadIdx.x) * per), hi = min(n, lo + per);
  unsigned sum = 0;
  for (int i = lo; i < hi; ++i) sum += in[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned incl = sum;
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  unsigned run = incl - sum;
  for (int w = 0; w < warp; ++w) run += warp_sums[w];
  for (int i = lo; i < hi; ++i) {  // a thread reads its own elements before it overwrites them
    const unsigned v = in[i];
    out[i] = run;
    run += v;
  }
  if (hi == n) out[n] = run;  // every thread at or past the end holds the total
  __syncthreads();
}

// first[b] = first item of list b, items of `rows_per_item` rows; one CTA.
// Runs: the histogram launch gives each of its `grid_x` CTAs (per feature tile) a contiguous
// share of ceil(items / grid_x) items; inside a share, neighbouring items of one list are
// one run while their rows fit an int32 plane together (`items_per_run` of them).  slot[it] =
// the run of item it (runs numbered in item order), slot_first[b] = first run of list b:
// the reduction adds up the planes of the runs [slot_first[b], slot_first[b + 1]).
__device__ void make_items(const unsigned *begin, const unsigned *len, const int *node_id,
                           int n_lists, int rows_per_item, int *first, WorkItem *items,
                           int *n_items, int max_items, int grid_x, int items_per_run, int *slot,
                           int *slot_first) {
  __shared__ int total;
  unsigned *ufirst = reinterpret_cast<unsigned *>(first);
  for (int i = threadIdx.x; i < n_lists; i += blockDim.x)
    ufirst[i] = (len[i] + unsigned(rows_per_item) - 1) / unsigned(rows_per_item);
  __syncthreads();
  block_exclusive_scan(ufirst, ufirst, n_lists);
  if (threadIdx.x == 0) {
    total = first[n_lists] < max_items ? first[n_lists] : max_items;
    *n_items = total;
  }
  __syncthreads();
  const int per = (total + grid_x - 1) / max(1, grid_x);
  unsigned *starts = reinterpret_cast<unsigned *>(slot) + max_items;  // scratch: max_items + 1 words
  for (int it = threadIdx.x; it < total; it += blockDim.x) {
    int lo = 0, hi = n_lists;  // last list with first[list] <= it
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
    // a run starts where a CTA's share or a list starts, and every items_per_run items from there
    const int seg = max(first[lo], per > 0 ? (it / per) * per : 0);
    starts[it] = ((it - seg) % items_per_run == 0) ? 1u : 0u;
  }
  __syncthreads();
  block_exclusive_scan(starts, starts, total);  // starts[it] = runs that begin before item it
  for (int it = threadIdx.x; it < total; it += blockDim.x)
    slot[it] = int(starts[it + 1]) - 1;  // the last run that begins at or before item it
  for (int b = threadIdx.x; b <= n_lists; b += blockDim.x)
    slot_first[b] = int(starts[b < n_lists ? min(first[b], total) : total]);
  __syncthreads();
}

// One CTA per level: prefix counts, the children that get a histogram of their own, their
// row lists and the work items of the histogram pass.
//   child_count : per parent, the rows that stepped to its right child (nullptr at the
//                 root, whose prefix counts {0, rows} are already in node_begin)
//   parent_begin: prefix counts of the level above
//   parent_rec  : split records of the level above; left_count += rows that went left
//                 (cleared by the split search; row chunks add up)
__global__ void plan_level_kernel(const unsigned *__restrict__ child_count,
                                  const unsigned *__restrict__ parent_begin,
                                  unsigned *__restrict__ node_begin, NodeRec *__restrict__ parent_rec,
                                  int L, int item_rows, bool use_trick, bool by_hessian,
                                  PlanBuffers pb, int max_items, int hist_grid, int items_per_run) {
  overlap_release();
  overlap_wait();
  unsigned *sb = pb.scratch_begin, *sl = pb.scratch_len;
  int *sn = pb.scratch_node;
  if (child_count) {  // rows that went right, per parent; the others of the parent went left
    for (int p = threadIdx.x; p < L / 2; p += blockDim.x) {
      const unsigned size = parent_begin[p + 1] - parent_begin[p], rights = child_count[size_t(p) * kPad];
      sl[2 * p] = size - rights;
      sl[2 * p + 1] = rights;
    }
    __syncthreads();
    block_exclusive_scan(sl, node_begin, L);
    for (int p = threadIdx.x; p < L / 2; p += blockDim.x) parent_rec[p].left_count += sl[2 * p];
  }
  // the next descend step counts into L counters at most; the level's split search starts
  // from cleared keys
  for (int i = threadIdx.x; i < L; i += blockDim.x) pb.right_count[size_t(i) * kPad] = 0;
  for (int i = threadIdx.x; i < pb.split_scratch_words; i += blockDim.x) pb.split_scratch[i] = 0;
  __syncthreads();
  int n_build;
  if (use_trick && L > 1) {
    n_build = L / 2;
    for (int p = threadIdx.x; p < n_build; p += blockDim.x) {
      const unsigned ls = node_begin[2 * p + 1] - node_begin[2 * p];
      const unsigned rs = node_begin[2 * p + 2] - node_begin[2 * p + 1];
      int built;
      if (by_hessian) {  // identical on every rank and for every row chunk: from the global sums
        const long long lh = parent_rec[p].lh, rh = parent_rec[p].th - parent_rec[p].lh;
        built = lh <= rh ? 0 : 1;
      } else {  // smaller child, ties build the left one (hist_grad_sum.cu:288-290)
        built = ls <= rs ? 0 : 1;
      }
      pb.built_child[p] = built;
      sl[p] = built ? rs : ls;
      sn[p] = 2 * p + built;
      pb.list_base[2 * p + 1 - built] = kNoList;
    }
  } else {
    n_build = L;
    for (int i = threadIdx.x; i < L; i += blockDim.x) {
      sl[i] = node_begin[i + 1] - node_begin[i];
      sn[i] = i;
    }
  }
  __syncthreads();
  // a node's list lies on the node's own range of the level's prefix counts
  for (int b = threadIdx.x; b < n_build; b += blockDim.x) {
    sb[b] = node_begin[sn[b]];
    pb.list_base[sn[b]] = sb[b];
    pb.cursor[size_t(sn[b]) * kPad] = 0;
  }
  __syncthreads();
  make_items(sb, sl, sn, n_build, item_rows, pb.hist_item_first, pb.hist_items, pb.n_hist_items,
             max_items, hist_grid, items_per_run, pb.item_slot, pb.slot_first);
}

__device__ __forceinline__ void red_shared_u32(unsigned *p, unsigned v) {
  const unsigned a = unsigned(__cvta_generic_to_shared(p));
  asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

// Every row takes one step down the tree, in row order.  A warp takes 256 consecutive rows
// per turn, row base + 32 k + lane in pass k, so that every access is coalesced and a lane
// has eight independent loads in flight; the bin comes from the feature-major copy when
// there is one (neighbouring rows share its lines whatever their nodes are).  The rows that
// go right are counted per node: in registers (lane c counts for node c, from ballots) while
// the level has at most kFewNodes nodes, with shared-memory atomics beyond that, where lanes
// rarely meet on a node.
// FINAL: the step below the last level; instead of storing and counting the child, the
// row's prediction receives the child's leaf weight (garden.cu:45-76 of the reference).
template <typename BIN_T, bool FINAL>
__global__ void __launch_bounds__(256)
descend_kernel(const unsigned char *__restrict__ bins, const size_t pitch,
               const unsigned char *__restrict__ bins_cm, const size_t cm_rows,
               const NodeRec *__restrict__ rec, const int L, unsigned short *__restrict__ node_of,
               unsigned *__restrict__ right_count, const float *__restrict__ leaf_w,
               float *__restrict__ yhat, const size_t n, const int n_dense) {
  overlap_release();
  overlap_wait();
  // feature << 16 | split bin, bit 15 set for a categorical feature (left <=> bin == split
  // bin; a dense feature goes left with bin <= split bin); feature 0xffff: no split
  __shared__ unsigned table[kSmemNodes];
  __shared__ unsigned cnt[kSmemNodes];    // rows of this CTA that went right, per node
  const bool cached = L <= kSmemNodes;
  auto packed = [&](int i) {
    const int fid = rec[i].fid;
    return fid < 0 ? 0xffff0000u
                   : (unsigned(fid) << 16) | unsigned(rec[i].bin) | (fid >= n_dense ? kCatFlag : 0u);
  };
  if (cached) {
    for (int i = threadIdx.x; i < L; i += blockDim.x) {
      table[i] = packed(i);
      cnt[i] = 0;
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const bool few = L <= kFewNodes;
  unsigned mine = 0;  // few nodes: lane c < L counts the right-goers of node c
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
      const unsigned e = cached ? table[node[k]] : packed(node[k]);
      const int fid = int(e >> 16);
      split_bin[k] = int(e & 0xffffu);  // with the categorical flag
      binv[k] = -1;  // no split, or past the end: left
      if (fid != 0xffff && r < n)
        binv[k] = bins_cm ? int(reinterpret_cast<const BIN_T *>(bins_cm)[size_t(fid) * cm_rows + r])
                          : int(reinterpret_cast<const BIN_T *>(bins + r * pitch)[fid]);
    }
#pragma unroll
    for (int k = 0; k < kDescendPasses; ++k) {
      const size_t r = base + size_t(k) * 32 + lane;
      const bool right = (split_bin[k] & int(kCatFlag)) ? (binv[k] >= 0 && binv[k] != (split_bin[k] & 0x7fff))
                                                       : binv[k] > split_bin[k];
      const int child = 2 * node[k] + (right ? 1 : 0);
      if (FINAL) {
        if (r < n) yhat[r] += leaf_w[child];
      } else {
        if (r < n) node_of[r] = (unsigned short)child;
        if (!cached) {
          if (right) atomicAdd(&right_count[size_t(node[k]) * kPad], 1u);
        } else if (few) {
          for (int c = 0; c < L; ++c) {
            const unsigned m = __ballot_sync(0xffffffffu, right && node[k] == c);
            if (lane == c) mine += unsigned(__popc(m));
          }
        } else if (right) {
          red_shared_u32(&cnt[node[k]], 1u);
        }
      }
    }
  }
  if (!FINAL && cached) {
    if (few && lane < L && mine) red_shared_u32(&cnt[lane], mine);
    __syncthreads();
    for (int i = threadIdx.x; i < L; i += blockDim.x)
      if (cnt[i]) atomicAdd(&right_count[size_t(i) * kPad], cnt[i]);
  }
}

// The same step for the common case (the level's table fits shared memory, a feature-major
// copy of the bins exists, node_of and yhat start on 16-byte boundaries), laid out for more
// rows in flight per register: a lane takes kWideRows consecutive rows, reads their eight
// nodes with one 16-byte load (and, FINAL, their predictions with two, before anything
// depends on them), keeps nodes and split bins packed two to a word beside the eight bins in
// flight, and writes the children (FINAL: the predictions) with 16-byte stores.  A warp
// still covers 256 consecutive rows per turn, so the bin reads of rows on one feature share
// sectors.  The counts of the first two nodes are kept per lane while the level has at most
// kFewNodes nodes.
constexpr int kWideRows = 8;
constexpr int kWideCtasPerSm = 6;  // 40 registers: no spills

template <typename BIN_T, bool FINAL>
__global__ void __launch_bounds__(256, FINAL ? 5 : kWideCtasPerSm)
descend_wide_kernel(const unsigned char *__restrict__ bins_cm, const size_t cm_rows,
                    const NodeRec *__restrict__ rec, const int L, unsigned short *__restrict__ node_of,
                    unsigned *__restrict__ right_count, const float *__restrict__ leaf_w,
                    float *__restrict__ yhat, const size_t n, const int n_dense) {
  overlap_release();
  overlap_wait();
  __shared__ unsigned table[kSmemNodes];             // packed splits, as in descend_kernel
  __shared__ unsigned cnt[FINAL ? 1 : kSmemNodes];   // rows of this CTA that went right, per node
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    const int fid = rec[i].fid;
    table[i] = fid < 0 ? 0xffff0000u
                       : (unsigned(fid) << 16) | unsigned(rec[i].bin) | (fid >= n_dense ? kCatFlag : 0u);
    if (!FINAL) cnt[i] = 0;
  }
  __syncthreads();
  const bool few = L <= kFewNodes;
  unsigned mine0 = 0, mine1 = 0;  // few nodes: this lane's right-goers of nodes 0 and 1
  const BIN_T *__restrict__ cm = reinterpret_cast<const BIN_T *>(bins_cm);
  const size_t threads = size_t(gridDim.x) * blockDim.x;
  for (size_t r0 = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * kWideRows; r0 < n;
       r0 += threads * kWideRows) {
    const bool whole = r0 + kWideRows <= n;
    uint4 nodes = make_uint4(0u, 0u, 0u, 0u);  // eight nodes, two to a word (low half first)
    if (L > 1) nodes = *reinterpret_cast<const uint4 *>(node_of + r0);
    float y[kWideRows];
    if (FINAL) {
      if (whole) {
        const float4 a = *reinterpret_cast<const float4 *>(yhat + r0);
        const float4 b = *reinterpret_cast<const float4 *>(yhat + r0 + 4);
        y[0] = a.x, y[1] = a.y, y[2] = a.z, y[3] = a.w, y[4] = b.x, y[5] = b.y, y[6] = b.z, y[7] = b.w;
      } else {
#pragma unroll
        for (int k = 0; k < kWideRows; ++k) y[k] = r0 + k < n ? yhat[r0 + k] : 0.0f;
      }
    }
    unsigned nw[4] = {nodes.x, nodes.y, nodes.z, nodes.w};
    if (!whole) {  // what lies past the last row is not a node number
#pragma unroll
      for (int k = 0; k < kWideRows; ++k)
        if (r0 + k >= n) nw[k >> 1] &= ~(0xffffu << (16 * (k & 1)));
    }
    unsigned sb[4] = {0u, 0u, 0u, 0u};  // the eight split bins, packed the same way
    int binv[kWideRows];
#pragma unroll
    for (int k = 0; k < kWideRows; ++k) {
      const unsigned node = (nw[k >> 1] >> (16 * (k & 1))) & 0xffffu;
      const unsigned e = table[node];
      const unsigned fid = e >> 16;
      sb[k >> 1] |= (e & 0xffffu) << (16 * (k & 1));
      binv[k] = -1;  // no split, or past the end: left
      if (fid != 0xffffu && r0 + k < n) binv[k] = int(cm[size_t(fid) * cm_rows + r0 + k]);
    }
    unsigned out[4];
#pragma unroll
    for (int k = 0; k < kWideRows; ++k) {
      const unsigned node = (nw[k >> 1] >> (16 * (k & 1))) & 0xffffu;
      const int sbin = int((sb[k >> 1] >> (16 * (k & 1))) & 0xffffu);
      const bool right = (sbin & int(kCatFlag)) ? (binv[k] >= 0 && binv[k] != (sbin & 0x7fff)) : binv[k] > sbin;
      const unsigned child = 2u * node + (right ? 1u : 0u);
      if (FINAL) {
        y[k] += leaf_w[child];
      } else {
        if (k & 1) out[k >> 1] |= child << 16; else out[k >> 1] = child;
        if (few) {
          mine0 += (right && node == 0u) ? 1u : 0u;
          mine1 += (right && node == 1u) ? 1u : 0u;
        } else if (right) {
          red_shared_u32(&cnt[node], 1u);
        }
      }
    }
    if (FINAL) {
      if (whole) {
        *reinterpret_cast<float4 *>(yhat + r0) = make_float4(y[0], y[1], y[2], y[3]);
        *reinterpret_cast<float4 *>(yhat + r0 + 4) = make_float4(y[4], y[5], y[6], y[7]);
      } else {
#pragma unroll
        for (int k = 0; k < kWideRows; ++k)
          if (r0 + k < n) yhat[r0 + k] = y[k];
      }
    } else if (whole) {
      *reinterpret_cast<uint4 *>(node_of + r0) = make_uint4(out[0], out[1], out[2], out[3]);
    } else {
      for (int k = 0; r0 + k < n; ++k)
        node_of[r0 + k] = (unsigned short)((out[k >> 1] >> (16 * (k & 1))) & 0xffffu);
    }
  }
  if (FINAL) return;
  if (few) {
    mine0 = __reduce_add_sync(0xffffffffu, mine0);
    mine1 = __reduce_add_sync(0xffffffffu, mine1);
    if ((threadIdx.x & 31) == 0) {
      if (mine0) red_shared_u32(&cnt[0], mine0);
      if (mine1 && L > 1) red_shared_u32(&cnt[1], mine1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < L; i += blockDim.x)
    if (cnt[i]) atomicAdd(&right_count[size_t(i) * kPad], cnt[i]);
}

// The rows of the built nodes go to their node's list.  A CTA takes kListRows consecutive
// rows: every row gets a rank among the CTA's rows of its node from a shared-memory counter
// (one atomic per group of lanes with the same node while the level has at most kFewLists
// nodes: there the lanes of a warp would all meet on the same few counters), the CTA
// reserves room in every list it has rows for with one global atomicAdd, and the rows are
// written at list start + CTA base + rank.
template <typename GRAD_T>  // int2 / int: the gradient record copied along; char: none
__global__ void __launch_bounds__(kListThreads)
gather_lists_kernel(const unsigned short *__restrict__ node_of, const size_t n, const int L,
                    const unsigned *__restrict__ list_base, unsigned *__restrict__ cursor,
                    unsigned *__restrict__ list, const GRAD_T *__restrict__ grad,
                    GRAD_T *__restrict__ list_grad) {
  overlap_release();
  overlap_wait();
  // per node: first the CTA's row count, then where the CTA's rows of the node go (kNoList:
  // the node has no list)
  __shared__ unsigned s_at[kSmemNodes];
  constexpr int kPer = kListRows / kListThreads;
  const bool cached = L <= kSmemNodes;
  const bool few = L <= kFewLists;
  const size_t base = size_t(blockIdx.x) * kListRows;
  const int lane = threadIdx.x & 31;
  // bit i: node i has a list; the rows of the other nodes (about half of all rows under the
  // subtraction trick) then take no rank
  __shared__ unsigned s_has_list[kSmemNodes / 32];
  int node[kPer];
  unsigned rank[kPer];
  GRAD_T gv[kPer];  // the gradient records of the rows that go to a list
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const size_t r = base + size_t(k) * kListThreads + threadIdx.x;
    node[k] = r < n ? int(node_of[r]) : -1;
  }
  if (cached) {
    for (int i0 = 0; i0 < L; i0 += kListThreads) {  // a warp's 32 nodes make one word of the mask
      const int i = i0 + threadIdx.x;
      const unsigned m = __ballot_sync(0xffffffffu, i < L && list_base[i] != kNoList);
      if (i < L) s_at[i] = 0;
      if (lane == 0 && i < L) s_has_list[i >> 5] = m;
    }
    __syncthreads();
    const unsigned first_word = s_has_list[0];
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      if (node[k] < 0) continue;
      const unsigned word = L <= 32 ? first_word : s_has_list[node[k] >> 5];
      if (!((word >> (node[k] & 31)) & 1u)) node[k] = -1;
    }
  }
  if (sizeof(GRAD_T) > 1) {  // in flight while the ranks are taken
#pragma unroll
    for (int k = 0; k < kPer; ++k)
      if (node[k] >= 0) gv[k] = grad[base + size_t(k) * kListThreads + threadIdx.x];
  }
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    rank[k] = 0;
    if (!cached) {  // too many nodes for the table: row by row, straight to the list position
      if (node[k] >= 0) {
        const unsigned lb = list_base[node[k]];
        if (lb == kNoList) node[k] = -1;
        else rank[k] = lb + atomicAdd(&cursor[size_t(node[k]) * kPad], 1u);
      }
    } else if (few) {  // the lanes that hold the same node take their ranks from one atomic
      const unsigned peers = __match_any_sync(0xffffffffu, node[k]);
      if (node[k] >= 0) {
        const int leader = __ffs(peers) - 1;
        unsigned first = 0;
        if (lane == leader) first = atomicAdd(&s_at[node[k]], unsigned(__popc(peers)));
        first = __shfl_sync(peers, first, leader);
        rank[k] = first + unsigned(__popc(peers & ((1u << lane) - 1)));
      }
    } else if (node[k] >= 0) {
      rank[k] = atomicAdd(&s_at[node[k]], 1u);
    }
  }
  if (cached) {
    __syncthreads();
    for (int i = threadIdx.x; i < L; i += kListThreads) {
      const unsigned c = s_at[i], lb = list_base[i];
      s_at[i] = lb == kNoList ? kNoList : (c ? lb + atomicAdd(&cursor[size_t(i) * kPad], c) : lb);
    }
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    if (node[k] < 0) continue;
    const size_t r = base + size_t(k) * kListThreads + threadIdx.x;
    const unsigned at = cached ? s_at[node[k]] : 0u;
    if (at != kNoList) {
      list[at + rank[k]] = unsigned(r);
      if (sizeof(GRAD_T) > 1) list_grad[at + rank[k]] = gv[k];
    }
  }
}


}  // namespace

void launch_plan_level(const LevelPlanLaunch &a, cudaStream_t s) {
  launch_overlapped(plan_level_kernel, 1, kPlanThreads, 0, s, a.child_count, a.parent_begin, a.node_begin, a.parent_rec,
                    a.L, a.item_rows, a.use_trick, a.by_hessian, a.pb, a.max_items, a.hist_grid_x,
                    std::max(1, a.items_per_run));
  count_launch();
}

namespace {

// CTAs of `kernel` that are resident on the current device at once
template <typename K>
int resident_ctas(K kernel, int threads) {
  int per_sm = 0;
  ARB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
  return std::max(1, per_sm * device_sm_count());
}
// the same, asked once per kernel and device (a process may drive several devices)
template <typename K>
int resident_ctas_cached(K kernel, int threads) {
  static int cached[kMaxDevices] = {};
  const int dev = current_device();
  if (!cached[dev]) cached[dev] = resident_ctas(kernel, threads);
  return cached[dev];
}

}  // namespace

void launch_descend(const DescendLaunch &a, cudaStream_t s) {
  if (a.n == 0) return;
  const bool fin = a.child_count == nullptr;
  const Geometry &g = a.geo;
  // exactly as many CTAs as are resident at once: a second, partly filled wave would cost
  // as much as a full one
  const bool wide = g.bins_cm && a.L <= kSmemNodes && reinterpret_cast<uintptr_t>(a.node_of) % 16 == 0 &&
                    (!fin || reinterpret_cast<uintptr_t>(a.yhat) % 16 == 0);
  if (wide) {
    const size_t span = size_t(256) * kWideRows;  // rows of one CTA turn
#define ARB_LAUNCH(T, FIN)                                                                          \
  do {                                                                                              \
    const int resident = resident_ctas_cached(descend_wide_kernel<T, FIN>, 256);                    \
    const int grid = int(std::min<size_t>((a.n + span - 1) / span, size_t(resident)));              \
    launch_overlapped(descend_wide_kernel<T, FIN>, grid, 256, 0, s, g.bins_cm, g.cm_rows, a.rec,    \
                      a.L, a.node_of, a.child_count, a.leaf_w, a.yhat, a.n, g.n_dense);             \
  } while (0)
    if (g.bin_bytes == 1) {
      if (fin) ARB_LAUNCH(unsigned char, true); else ARB_LAUNCH(unsigned char, false);
    } else {
      if (fin) ARB_LAUNCH(unsigned short, true); else ARB_LAUNCH(unsigned short, false);
    }
#undef ARB_LAUNCH
    ARB_CUDA(cudaGetLastError());
    count_launch();
    return;
  }
  const size_t span = size_t(32) * kDescendPasses * (256 / 32);  // rows of one CTA turn
#define ARB_LAUNCH(T, FIN)                                                                          \
  do {                                                                                              \
    const int resident = resident_ctas_cached(descend_kernel<T, FIN>, 256);                         \
    const int grid = int(std::min<size_t>((a.n + span - 1) / span, size_t(resident)));              \
    launch_overlapped(descend_kernel<T, FIN>, grid, 256, 0, s, g.bins, g.pitch, g.bins_cm,          \
                      g.cm_rows, a.rec, a.L, a.node_of, a.child_count, a.leaf_w, a.yhat, a.n,       \
                      g.n_dense);                                                                   \
  } while (0)
  if (g.bin_bytes == 1) {
    if (fin) ARB_LAUNCH(unsigned char, true); else ARB_LAUNCH(unsigned char, false);
  } else {
    if (fin) ARB_LAUNCH(unsigned short, true); else ARB_LAUNCH(unsigned short, false);
  }
#undef ARB_LAUNCH
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_gather_lists(const unsigned short *node_of, size_t n, int L, const PlanBuffers &pb,
                         unsigned *list, const void *grad, void *list_grad, bool pair,
                         cudaStream_t s) {
  if (n == 0) return;
  const unsigned grid = unsigned((n + kListRows - 1) / kListRows);
  if (!list_grad)
    launch_overlapped(gather_lists_kernel<char>, grid, kListThreads, 0, s, node_of, n, L, pb.list_base, pb.cursor,
                      list, nullptr, nullptr);
  else if (pair)
    launch_overlapped(gather_lists_kernel<int2>, grid, kListThreads, 0, s, node_of, n, L, pb.list_base, pb.cursor,
                      list, static_cast<const int2 *>(grad), static_cast<int2 *>(list_grad));
  else
    launch_overlapped(gather_lists_kernel<int>, grid, kListThreads, 0, s, node_of, n, L, pb.list_base, pb.cursor,
                      list, static_cast<const int *>(grad), static_cast<int *>(list_grad));
  count_launch();
}

}  // namespace arb
