// Per-level gradient histograms (row H of the hot path; replaces the reference's
// sort-based hist_sum_node / hist_sum_multi_node, src/core/hist_grad_sum.cu:109-406,
// and update_multi_node, :6-33).
//
// Design for sm_100a:
//  * Gradients are fixed-point integers (g_q, h_q) for the whole round, so a
//    histogram is an exact integer sum: any CTA order, any number of GPUs and the
//    sibling subtraction all give bit-identical results.
//  * A CTA owns (work item = piece of one node's row list) x (tile of TW features)
//    and keeps a private sub-histogram in shared memory as two int32 planes
//    G[bin][feature], H[bin][feature] (64 KB).  A work item has at most
//    2^(31 - quant_bits) rows, so a plane cannot overflow.
//  * uint8 fast path (TW = 32): rows are fetched by row id, one 32-byte sector per
//    row, with cp.async straight into a per-warp ring of shared-memory stages
//    (the next batches are in flight while the current one is consumed).  A warp
//    consumes 4 rows per step: lane (q, m) reads one 32-bit word = features
//    4m..4m+3 of row 4s+q, and in pass k updates feature 4m + ((k + q) & 3).  The
//    32 lanes of every red.shared instruction therefore hit 32 different banks
//    whatever the bin values are -- no bank conflicts, also for skewed or sorted
//    columns -- at 2.5 shared-memory wavefronts per row.  The two red.shared per 32
//    (row, feature) pairs are what bounds the kernel on consecutive rows:
//    measure_shared_atomic_peak() times them alone.
//  * Below the root a row list (row ids, and the gradient records in the same order)
//    says which rows a node has: ids and gradients are read in list order, the bins
//    are gathered with the 64-byte L2 fetch qualifier, since a plain copy would pull
//    the whole 128-byte line (four rows) for the one row the node wants.
//    With ARBORETUM_TMA_GATHER in the environment (and the matrix resident in HBM) the gather
//    is done by the TMA unit instead: cp.async.bulk.tensor.2d ... tile::gather4 names four
//    rows per instruction, eight lanes fetch a warp's batch of 32 rows, the tensor map asks
//    L2 for 64-byte fetches, and completion is counted on a per-warp mbarrier.  The address
//    work of the gather then no longer goes through the load/store pipe that the
//    red.shared instructions need; measured, the pass is 6 % slower this way (both gathers
//    reach the same rate alone, and the reductions bound the pass), so it is not the default.
//  * The CTA stores its planes with plain coalesced stores; reduce_kernel then
//    sums the planes of every built node into the level's int64 histogram and, in
//    the same pass, derives the sibling as parent - built (the subtraction trick).
#include <cuda.h>

#include <cstring>

#include "kernels.cuh"

namespace arb {

namespace {

constexpr int kStages = 2;
constexpr int kStageBytes = 1024 + 256;  // 32 rows x 32 B of bins, 32 x (g_q, h_q)

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
  const unsigned d = unsigned(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}
// The same copy for rows fetched by row id.  A miss of the plain copy brings the whole
// 128-byte line into L2, four bin rows of which a gathered node wants one; with this
// qualifier L2 fetches the 64-byte half only (measured on a bare gather of every fourth
// row: 128 -> 64 B of DRAM reads per 32-byte row, 1.7x the rows per second).
__device__ __forceinline__ void cp_async16_gather(void *dst, const void *src) {
  const unsigned d = unsigned(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global.L2::64B [%0], [%1], 16;" ::"r"(d), "l"(src));
}
// copies `bytes` (0 or SIZE) and zero-fills the rest of the SIZE-byte destination
template <int SIZE>
__device__ __forceinline__ void cp_async_zfill(void *dst, const void *src, int bytes) {
  const unsigned d = unsigned(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(d), "l"(src), "n"(SIZE), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void red_shared(int *p, int v) {
  const unsigned a = unsigned(__cvta_generic_to_shared(p));
  asm volatile("red.shared.add.s32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

// ---- TMA row gather ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(unsigned long long *bar, int count) {
  const unsigned a = unsigned(__cvta_generic_to_shared(bar));
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
  const unsigned a = unsigned(__cvta_generic_to_shared(bar));
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
  const unsigned a = unsigned(__cvta_generic_to_shared(bar));
  unsigned ok;
  asm volatile(
    "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
    : "=r"(ok)
    : "r"(a), "r"(parity)
    : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// four rows y0..y3 of the 2-D tensor (bytes of a row, rows), `x` bytes into each, to 4 x 32
// consecutive bytes of shared memory; x must be a multiple of 16
__device__ __forceinline__ void tma_gather4(void *dst, const CUtensorMap *map, int x, int y0, int y1, int y2,
                                            int y3, unsigned long long *bar) {
  const unsigned d = unsigned(__cvta_generic_to_shared(dst));
  const unsigned a = unsigned(__cvta_generic_to_shared(bar));
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
    "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(d),
    "l"(map), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(a)
    : "memory");
}
// A wait on the gather's barrier gives up after this long and reports it (the data of a
// copy that never arrives cannot be had any other way; the host then refuses the tree).
constexpr unsigned long long kGatherWaitNs = 2000000000ull;

// the CTA's two int32 planes -> partials[(item * NT + tile)][2][kHistWords]
__device__ __forceinline__ void store_planes(const int *smem, int *dst) {
  const int4 *src4 = reinterpret_cast<const int4 *>(smem);
  int4 *dst4 = reinterpret_cast<int4 *>(dst);
  for (int w = threadIdx.x; w < 2 * kHistWords / 4; w += blockDim.x) dst4[w] = src4[w];
}

// uint8 bins, 32 features per tile, 256 bins.
// TMA: rows are gathered through `row_map` (never with IDENT); `status` takes a 1 when a wait
// on a gather ran into its time limit.
template <bool PAIR, bool IDENT, bool TMA>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
hist_u8_kernel(const unsigned char *__restrict__ bins, const size_t pitch, const size_t tile_stride, const int NT,
               const unsigned *__restrict__ rowid, const void *__restrict__ grad,
               const WorkItem *__restrict__ items, const int *__restrict__ n_items,
               const int *__restrict__ item_slot, int *__restrict__ partials,
               const void *__restrict__ list_grad, const __grid_constant__ CUtensorMap row_map,
               int *__restrict__ status) {
  static_assert(!(TMA && IDENT), "consecutive rows are copied, not gathered");
  extern __shared__ __align__(128) int smem[];
  constexpr int kWarps = kHistThreads / 32;
  unsigned char *stage0 = reinterpret_cast<unsigned char *>(smem + 2 * kHistWords);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char *my = stage0 + warp * kStages * kStageBytes;
  // one barrier per warp and stage, behind the stages
  unsigned long long *bars =
    reinterpret_cast<unsigned long long *>(stage0 + kWarps * kStages * kStageBytes) + warp * kStages;
  unsigned phases = 0;   // bit s: the parity the next wait on stage s looks for
  bool gave_up = false;  // a wait ran out: no more gathers are issued or waited for
  // the histogram of the CTA's first item is cleared while the kernel before this one drains
  overlap_release();
  for (int w = threadIdx.x; w < 2 * kHistWords; w += kHistThreads) smem[w] = 0;
  overlap_wait();
  if (TMA) {
    // after the wait, not in the preamble: with the barriers initialised before it, a kernel
    // launched as a programmatic dependent built wrong histograms for the last nodes of a level
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < kStages; ++st) mbar_init(bars + st, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
  }
  bool cleared = true;
  int *G = smem;
  // grid = (tiles, shares): the CTAs that take the same rows in neighbouring tiles are launched
  // side by side, so a row's line is fetched from DRAM once for the tiles that share it
  const int tile = blockIdx.x;
  // row-major: the tile's 32 bytes inside every row; tile by tile: the tile's own block of rows
  const unsigned char *tile_base = bins + size_t(tile) * (tile_stride ? tile_stride : size_t(32));
  const int q = lane >> 3, m = lane & 7;
  int foff[4], sh[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = (k + q) & 3;
    foff[k] = 4 * m + r;
    sh[k] = 8 * r;
  }
  constexpr int GSZ = PAIR ? 8 : 4;  // bytes of one quantised gradient record
  const int total_items = *n_items;
  // A CTA takes a contiguous share of the items.  Neighbouring items of one node are one run
  // (the plan kernel gave them the same slot: together they stay within what an int32 plane
  // holds): their rows lie back to back in the node's list and go through the pipeline as one
  // piece, and the planes are stored once per run.
  const int per = (total_items + int(gridDim.y) - 1) / int(gridDim.y);
  const int it_end = min(total_items, (int(blockIdx.y) + 1) * per);
  for (int it = int(blockIdx.y) * per; it < it_end;) {
    WorkItem item = items[it];
    const int slot = item_slot ? item_slot[it] : it;
    for (++it; it < it_end && item_slot && item_slot[it] == slot; ++it) item.len += items[it].len;
    if (!cleared)
      for (int w = threadIdx.x; w < 2 * kHistWords; w += kHistThreads) smem[w] = 0;
    cleared = false;
    __syncthreads();
    const unsigned len = item.len;
    const int nb = int((len + 31) / 32);  // batches of 32 rows, dealt round-robin to warps

    auto rid_of = [&](int b) -> unsigned {
      const unsigned pos = min(unsigned(b * 32 + lane), len - 1);
      return IDENT ? item.begin + pos : __ldg(rowid + item.begin + pos);
    };
    auto issue = [&](int b, int stage, unsigned rid_lane) {
      unsigned char *sb = my + stage * kStageBytes;
      if (TMA) {
        // lane j < 8 names rows 4j..4j+3 of the batch; the barrier expects the batch's 1024 bytes
        const int src = (lane & 7) * 4;
        const int y0 = int(__shfl_sync(0xffffffffu, rid_lane, src));
        const int y1 = int(__shfl_sync(0xffffffffu, rid_lane, src + 1));
        const int y2 = int(__shfl_sync(0xffffffffu, rid_lane, src + 2));
        const int y3 = int(__shfl_sync(0xffffffffu, rid_lane, src + 3));
        if (!gave_up) {
          if (lane == 0) mbar_expect_tx(bars + stage, 1024);
          __syncwarp();
          if (lane < 8) tma_gather4(sb + lane * 128, &row_map, tile * 32, y0, y1, y2, y3, bars + stage);
        }
      } else {
        // bins: lane handles half (lane & 1) of rows (lane >> 1) and 16 + (lane >> 1)
        const unsigned r0 = __shfl_sync(0xffffffffu, rid_lane, lane >> 1);
        const unsigned r1 = __shfl_sync(0xffffffffu, rid_lane, 16 + (lane >> 1));
        if (IDENT) {  // consecutive rows: whole lines are wanted
          cp_async16(sb + (lane >> 1) * 32 + (lane & 1) * 16,
                     tile_base + size_t(r0) * pitch + (lane & 1) * 16);
          cp_async16(sb + (16 + (lane >> 1)) * 32 + (lane & 1) * 16,
                     tile_base + size_t(r1) * pitch + (lane & 1) * 16);
        } else {
          cp_async16_gather(sb + (lane >> 1) * 32 + (lane & 1) * 16,
                            tile_base + size_t(r0) * pitch + (lane & 1) * 16);
          cp_async16_gather(sb + (16 + (lane >> 1)) * 32 + (lane & 1) * 16,
                            tile_base + size_t(r1) * pitch + (lane & 1) * 16);
        }
      }
      // rows past the end of the item get a zero gradient record: they add nothing
      const bool valid = unsigned(b * 32 + lane) < len;
      // the gradient records lie in list order beside the row ids when the list pass copied
      // them (a sequential read); otherwise they are gathered by row id like the bins
      const char *gsrc = list_grad
                           ? static_cast<const char *>(list_grad) +
                               size_t(item.begin + min(unsigned(b * 32 + lane), len - 1)) * GSZ
                           : static_cast<const char *>(grad) + size_t(rid_lane) * GSZ;
      cp_async_zfill<GSZ>(sb + 1024 + lane * GSZ, gsrc, valid ? GSZ : 0);
      cp_async_commit();
    };

    int b_issue = warp;
    unsigned rid_next = 0;
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      if (b_issue < nb) issue(b_issue, s, rid_of(b_issue)); else cp_async_commit();
      b_issue += kWarps;
    }
    if (b_issue < nb) rid_next = rid_of(b_issue);
    int stage = 0;
    for (int b = warp; b < nb; b += kWarps) {
      cp_async_wait<kStages - 1>();
      if (TMA && !gave_up) {
        // lane 0 watches the barrier for the warp; the __syncwarp below hands what it saw
        // (the gathered rows in shared memory) on to the other lanes
        bool timed_out = false;
        if (lane == 0) {
          const unsigned parity = (phases >> stage) & 1u;
          if (!mbar_try_wait(bars + stage, parity)) {
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(bars + stage, parity)) {
              if (global_timer_ns() - t0 > kGatherWaitNs) {
                timed_out = true;
                break;
              }
            }
          }
          if (timed_out) atomicExch(status, 1);
        }
        gave_up = __shfl_sync(0xffffffffu, int(timed_out), 0) != 0;
        phases ^= 1u << stage;
      }
      __syncwarp();
      const unsigned char *sb = my + stage * kStageBytes;
      const int nvalid = int(min(32u, len - unsigned(b) * 32));
#pragma unroll 2
      for (int s = 0; s < 8; ++s) {
        const int row = 4 * s + q;
        const unsigned wv = *reinterpret_cast<const unsigned *>(sb + row * 32 + 4 * m);
        int gq, hq;
        if (PAIR) {
          const int2 gh = *reinterpret_cast<const int2 *>(sb + 1024 + row * 8);
          gq = gh.x;
          hq = gh.y;
        } else {
          gq = *reinterpret_cast<const int *>(sb + 1024 + row * 4);
          hq = row < nvalid;  // hessian == 1: the plane counts rows
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int bin = (wv >> sh[k]) & 255;
          int *p = G + bin * 32 + foff[k];
          red_shared(p, gq);
          red_shared(p + kHistWords, hq);
        }
      }
      __syncwarp();
      if (b_issue < nb) {
        const unsigned rid_c = rid_next;
        const int bn = b_issue + kWarps;
        if (bn < nb) rid_next = rid_of(bn);
        issue(b_issue, stage, rid_c);
      } else {
        cp_async_commit();
      }
      b_issue += kWarps;
      stage = (stage + 1 == kStages) ? 0 : stage + 1;
    }
    cp_async_wait<0>();
    __syncthreads();
    store_planes(smem, partials + (size_t(slot) * NT + tile) * 2 * kHistWords);
    __syncthreads();
  }
  if (TMA && gave_up) {
    // gathers issued before the wait ran out may still be on their way into this CTA's shared
    // memory: give them one more time limit before the CTA ends
    const unsigned long long t0 = global_timer_ns();
#pragma unroll
    for (int st = 0; st < kStages; ++st)
      while (!mbar_try_wait(bars + st, (phases >> st) & 1u) && global_timer_ns() - t0 < kGatherWaitNs) {
      }
  }
}

// Any bin width / tile width: thread = (row in group, feature in tile).
template <bool PAIR, bool IDENT, typename BIN_T>
__global__ void __launch_bounds__(kHistThreads, kHistCtasPerSm)
hist_generic_kernel(const unsigned char *__restrict__ bins, const size_t pitch, const int NT,
                    const int TW, const int F, const unsigned *__restrict__ rowid,
                    const void *__restrict__ grad, const WorkItem *__restrict__ items,
                    const int *__restrict__ n_items, const int *__restrict__ item_slot,
                    int *__restrict__ partials) {
  extern __shared__ __align__(128) int smem[];
  int *G = smem;
  int *H = smem + kHistWords;
  const int tile = blockIdx.x;  // grid = (tiles, shares), see hist_u8_kernel
  const int rows_per_pass = kHistThreads / TW;
  const int f_in_tile = threadIdx.x % TW;
  const int rsub = threadIdx.x / TW;
  const int f = tile * TW + f_in_tile;
  const int total_items = *n_items;
  const int per = (total_items + int(gridDim.y) - 1) / int(gridDim.y);  // runs of items: see hist_u8_kernel
  const int it_end = min(total_items, (int(blockIdx.y) + 1) * per);
  for (int it = int(blockIdx.y) * per; it < it_end;) {
    WorkItem item = items[it];
    const int slot = item_slot ? item_slot[it] : it;
    for (++it; it < it_end && item_slot && item_slot[it] == slot; ++it) item.len += items[it].len;
    for (int w = threadIdx.x; w < 2 * kHistWords; w += kHistThreads) smem[w] = 0;
    __syncthreads();
    if (f < F) {
      for (unsigned pos = rsub; pos < item.len; pos += rows_per_pass) {
        const unsigned rid = IDENT ? item.begin + pos : rowid[item.begin + pos];
        const BIN_T bin = reinterpret_cast<const BIN_T *>(bins + size_t(rid) * pitch)[f];
        int gq, hq;
        if (PAIR) {
          const int2 g = __ldg(reinterpret_cast<const int2 *>(grad) + rid);
          gq = g.x;
          hq = g.y;
        } else {
          gq = __ldg(reinterpret_cast<const int *>(grad) + rid);
          hq = 1;
        }
        red_shared(&G[int(bin) * TW + f_in_tile], gq);
        red_shared(&H[int(bin) * TW + f_in_tile], hq);
      }
    }
    __syncthreads();
    store_planes(smem, partials + (size_t(slot) * NT + tile) * 2 * kHistWords);
    __syncthreads();
  }
}

// One thread per (built node, slice, tile, word): sums the planes of its share of
// the node's items.  With one slice per node the sum goes straight into the
// level's int64 histogram and, with SUBTRACT, the other child of the same parent
// is written as parent - built (update_multi_node of the reference); with more
// slices (few, large nodes) the sums meet in red.global.add.u64 on a cleared
// buffer and the subtraction runs as its own pass.
template <bool SUBTRACT>
__global__ void reduce_kernel(const int *__restrict__ partials, const int *__restrict__ item_first,
                              const int *__restrict__ build_node, long long *__restrict__ level_hist,
                              const long long *__restrict__ parent_hist, const int NT,
                              const int slices, const bool atomic) {
  overlap_release();
  overlap_wait();
  const int b = blockIdx.z / slices, slice = blockIdx.z - b * slices, tile = blockIdx.y;
  const int w = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = item_first[b], last = item_first[b + 1];
  long long g = 0, h = 0;
#pragma unroll 4
  for (int it = first + slice; it < last; it += slices) {
    const int *p = partials + (size_t(it) * NT + tile) * 2 * kHistWords;
    g += p[w];
    h += p[kHistWords + w];
  }
  const int node = build_node ? build_node[b] : b;  // no map: the output holds the built nodes only
  const size_t off = (size_t(node) * NT + tile) * kHistWords + w;
  if (slices > 1 || atomic) {
    if (g) atomicAdd(reinterpret_cast<unsigned long long *>(level_hist) + 2 * off, (unsigned long long)g);
    if (h) atomicAdd(reinterpret_cast<unsigned long long *>(level_hist) + 2 * off + 1, (unsigned long long)h);
    return;
  }
  reinterpret_cast<longlong2 *>(level_hist)[off] = make_longlong2(g, h);
  if (SUBTRACT) {
    const size_t poff = (size_t(node >> 1) * NT + tile) * kHistWords + w;
    const longlong2 pv = reinterpret_cast<const longlong2 *>(parent_hist)[poff];
    const size_t soff = (size_t(node ^ 1) * NT + tile) * kHistWords + w;
    reinterpret_cast<longlong2 *>(level_hist)[soff] = make_longlong2(pv.x - g, pv.y - h);
  }
}

__global__ void subtract_kernel(long long *__restrict__ level_hist,
                                const long long *__restrict__ parent_hist,
                                const int *__restrict__ built_child, const size_t words_per_node,
                                const size_t total) {
  overlap_release();
  overlap_wait();
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t p = i / words_per_node;
    const size_t w = i - p * words_per_node;
    const int built = built_child[p];
    const size_t src = (2 * p + built) * words_per_node + w;
    const size_t dst = (2 * p + (1 - built)) * words_per_node + w;
    level_hist[dst] = parent_hist[i] - level_hist[src];
  }
}

// built nodes only (in build order) -> both children of every parent:
// built child = compact, sibling = parent - compact
__global__ void expand_kernel(const long long *__restrict__ compact,
                              const long long *__restrict__ parent_hist,
                              long long *__restrict__ level_hist,
                              const int *__restrict__ built_child, const size_t words_per_node,
                              const size_t total) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t p = i / words_per_node;
    const size_t w = i - p * words_per_node;
    const int built = built_child[p];
    const long long v = compact[i];
    level_hist[(2 * p + built) * words_per_node + w] = v;
    level_hist[(2 * p + (1 - built)) * words_per_node + w] = parent_hist[i] - v;
  }
}

// opt in to more than 48 KB of dynamic shared memory, once per call site and device (the
// attribute belongs to the kernel's image on the current device)
#define ARB_SET_SMEM(kernel, bytes)                                                        \
  do {                                                                                     \
    static bool done__[kMaxDevices] = {};                                                  \
    const int dev__ = current_device();                                                    \
    if (!done__[dev__]) {                                                                  \
      ARB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                    int(bytes)));                                          \
      done__[dev__] = true;                                                                \
    }                                                                                      \
  } while (0)

}  // namespace

void launch_expand(const long long *compact, const long long *parent_hist, long long *level_hist,
                   const int *built_child, int n_parents, int NT, cudaStream_t s) {
  const size_t words_per_node = size_t(NT) * kHistWords * 2;
  const size_t total = size_t(n_parents) * words_per_node;
  const int threads = 256;
  const int blocks = int(std::min<size_t>((total + threads - 1) / threads, size_t(device_sm_count()) * 16));
  expand_kernel<<<blocks, threads, 0, s>>>(compact, parent_hist, level_hist, built_child, words_per_node,
                                           total);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_subtract(long long *level_hist, const long long *parent_hist, const int *built_child,
                     int n_parents, int NT, cudaStream_t s);

int hist_grid_x(int max_items, int NT) {
  // persistent CTAs: kHistCtasPerSm per SM over all tiles, and never more than are resident at
  // once -- a few CTAs left over for a second wave would double the pass (10 shares of 32 tiles
  // are 320 CTAs for 296 places)
  const int per_tile = std::max(1, kHistCtasPerSm * device_sm_count() / NT);
  return std::max(1, std::min(max_items, per_tile));
}

static_assert(sizeof(RowGatherMap) == sizeof(CUtensorMap) && alignof(RowGatherMap) >= alignof(CUtensorMap),
              "RowGatherMap is the driver's tensor map, kept opaque in the headers");

bool make_row_gather_map(RowGatherMap *out, const unsigned char *bins, size_t pitch, size_t rows) {
  // Opt-in: on a B200 the 10 M x 28 workload's histogram pass takes 0.735 ms per round with
  // this gather against 0.692 ms with cp.async (the bare gather rates are equal, 72 G rows/s,
  // and the pass is bound by its shared-memory reductions either way; the barrier round trip
  // per batch costs more than the freed load/store slots give back).
  const bool on = std::getenv("ARBORETUM_TMA_GATHER") != nullptr;  // read once per matrix
  if (!on || rows == 0 || rows >= (size_t(1) << 31) || pitch % 16 != 0 || pitch >= (size_t(1) << 32) ||
      reinterpret_cast<uintptr_t>(bins) % 16 != 0)
    return false;
  // the encoder is a driver function: ask the runtime for it instead of linking the driver
  using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                CUtensorMapFloatOOBfill);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult found;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess ||
      found != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return false;
  }
  // bytes of a padded row x rows; a box is the 32 bytes of one feature tile of one row (gather4
  // fetches four such boxes); L2 fetches 64 bytes for a miss, not the whole 128-byte line
  const cuuint64_t dims[2] = {cuuint64_t(pitch), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch)};
  const cuuint32_t box[2] = {32, 1};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult r = reinterpret_cast<EncodeFn>(fn)(
    &map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<unsigned char *>(bins), dims, strides, box, elem,
    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_64B,
    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::memcpy(out, &map, sizeof map);
  return true;
}

void launch_hist(const HistLaunch &a, cudaStream_t s) {
  const Geometry &g = a.geo;
  const dim3 grid(g.NT, a.grid_x > 0 ? a.grid_x : hist_grid_x(a.max_items, g.NT));
  const bool ident = a.rowid == nullptr;
  if (g.bin_bytes == 1 && g.TW == 32) {
    constexpr int kWarps = kHistThreads / 32;
    const size_t smem = 2 * kHistWords * 4 + kWarps * kStages * kStageBytes + kWarps * kStages * 8;
    const bool tma = a.row_map != nullptr && a.status != nullptr && !ident;
    CUtensorMap map;
    if (tma)
      std::memcpy(&map, a.row_map, sizeof map);
    else
      std::memset(&map, 0, sizeof map);
#define ARB_LAUNCH(P, I, T)                                                                      \
  do {                                                                                           \
    ARB_SET_SMEM((hist_u8_kernel<P, I, T>), smem);                                               \
    launch_overlapped(hist_u8_kernel<P, I, T>, grid, kHistThreads, smem, s, g.bins, g.pitch,     \
                      g.tile_stride, g.NT, a.rowid, a.grad, a.items, a.n_items, a.item_slot, a.partials,        \
                      a.list_grad, map, a.status);                                               \
  } while (0)
    if (a.pair) {
      if (ident) ARB_LAUNCH(true, true, false);
      else if (tma) ARB_LAUNCH(true, false, true);
      else ARB_LAUNCH(true, false, false);
    } else {
      if (ident) ARB_LAUNCH(false, true, false);
      else if (tma) ARB_LAUNCH(false, false, true);
      else ARB_LAUNCH(false, false, false);
    }
#undef ARB_LAUNCH
  } else {
    const size_t smem = 2 * kHistWords * 4;
#define ARB_LAUNCH(P, I, T)                                                                   \
  do {                                                                                        \
    ARB_SET_SMEM((hist_generic_kernel<P, I, T>), smem);                                       \
    hist_generic_kernel<P, I, T><<<grid, kHistThreads, smem, s>>>(                            \
      g.bins, g.pitch, g.NT, g.TW, g.F, a.rowid, a.grad, a.items, a.n_items, a.item_slot,     \
      a.partials);                                                                            \
  } while (0)
#define ARB_LAUNCH_T(T)                                                        \
  do {                                                                         \
    if (a.pair) {                                                              \
      if (ident) ARB_LAUNCH(true, true, T); else ARB_LAUNCH(true, false, T);   \
    } else {                                                                   \
      if (ident) ARB_LAUNCH(false, true, T); else ARB_LAUNCH(false, false, T); \
    }                                                                          \
  } while (0)
    if (g.bin_bytes == 1) ARB_LAUNCH_T(unsigned char); else ARB_LAUNCH_T(unsigned short);
#undef ARB_LAUNCH_T
#undef ARB_LAUNCH
  }
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

namespace {
// Ceiling of the histogram kernels' inner loop: every lane adds one (g, h) pair per step to
// its own column of the two int32 planes at a pseudo-random bin -- the same two conflict-free
// red.shared instructions per 32 (row, feature) pairs, with no loads, no staging and no
// stores around them, and with all 64 warps an SM can hold (the rate grows with the warps
// in flight: 2.6 T pairs/s with 32 warps, 2.9 T with 64).
constexpr int kPeakThreads = 1024;
__global__ void __launch_bounds__(kPeakThreads, 2) shared_atomic_peak_kernel(int steps, int *sink) {
  extern __shared__ __align__(128) int smem[];
  for (int w = threadIdx.x; w < 2 * kHistWords; w += kPeakThreads) smem[w] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  unsigned state = threadIdx.x * 2654435761u + blockIdx.x * 97u + 1u;
  for (int i = 0; i < steps; ++i) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      state = state * 1664525u + 1013904223u;
      const int bin = int(state >> 24);
      red_shared(smem + bin * 32 + lane, int(state & 0xffffu) - 32768);
      red_shared(smem + kHistWords + bin * 32 + lane, 1 + int(state & 0xffu));
    }
  }
  __syncthreads();
  int acc = 0;
  for (int w = threadIdx.x; w < 2 * kHistWords; w += kPeakThreads) acc ^= smem[w];
  if (acc == 0x7fffffff) sink[0] = acc;  // keeps the adds alive
}
}  // namespace

double measure_shared_atomic_peak(int steps, cudaStream_t s) {
  const size_t smem = 2 * kHistWords * 4;
  ARB_SET_SMEM(shared_atomic_peak_kernel, smem);
  DevBuf sink;
  sink.alloc(sizeof(int));
  const int grid = 2 * device_sm_count();
  cudaEvent_t e0, e1;
  ARB_CUDA(cudaEventCreate(&e0));
  ARB_CUDA(cudaEventCreate(&e1));
  float best = 0.0f;
  for (int rep = 0; rep < 4; ++rep) {  // the first launch warms up
    ARB_CUDA(cudaEventRecord(e0, s));
    shared_atomic_peak_kernel<<<grid, kPeakThreads, smem, s>>>(steps, sink.as<int>());
    ARB_CUDA(cudaEventRecord(e1, s));
    ARB_CUDA(cudaEventSynchronize(e1));
    float ms = 0.0f;
    ARB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (rep > 0 && (best == 0.0f || ms < best)) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  count_launch(4);
  return double(grid) * kPeakThreads * double(steps) * 8.0 / (double(best) * 1e-3);
}

void launch_reduce(const ReduceLaunch &a, cudaStream_t s) {
  const int threads = 256;
  // few built nodes: cut every node's item list into slices so the GPU is filled
  int slices = 1;
  while (slices < 64 && a.n_build * a.NT * slices < 64) slices <<= 1;
  const dim3 grid(kHistWords / threads, a.NT, a.n_build * slices);
  if (slices > 1 || a.accumulate) {
    const size_t bytes = size_t(a.level_nodes) * a.NT * kHistWords * 2 * sizeof(long long);
    if (!a.accumulate) ARB_CUDA(cudaMemsetAsync(a.level_hist, 0, bytes, s));
    launch_overlapped(reduce_kernel<false>, grid, threads, 0, s, a.partials, a.item_first, a.build_node,
                      a.level_hist, nullptr, a.NT, slices, true);
    count_launch();
    if (a.subtract) launch_subtract(a.level_hist, a.parent_hist, a.built_child, a.level_nodes / 2, a.NT, s);
    return;
  }
  if (a.subtract)
    launch_overlapped(reduce_kernel<true>, grid, threads, 0, s, a.partials, a.item_first, a.build_node,
                      a.level_hist, a.parent_hist, a.NT, 1, false);
  else
    launch_overlapped(reduce_kernel<false>, grid, threads, 0, s, a.partials, a.item_first, a.build_node,
                      a.level_hist, nullptr, a.NT, 1, false);
  count_launch();
}

void launch_subtract(long long *level_hist, const long long *parent_hist, const int *built_child,
                     int n_parents, int NT, cudaStream_t s) {
  const size_t words_per_node = size_t(NT) * kHistWords * 2;
  const size_t total = words_per_node * n_parents;
  const int threads = 256;
  const int blocks = int(std::min<size_t>((total + threads - 1) / threads, size_t(device_sm_count()) * 16));
  launch_overlapped(subtract_kernel, blocks, threads, 0, s, level_hist, parent_hist, built_child, words_per_node,
                    total);
  count_launch();
}

}  // namespace arb
