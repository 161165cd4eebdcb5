// Per-level gradient histograms (row H of the hot path; replaces the reference's
// sort-based hist_sum_node / hist_sum_multi_node, src/core/hist_grad_sum.cu:109-406,
// and update_multi_node, :6-33).
//
// Design for sm_100a:
//  * Gradients are turned into fixed-point integers per round (g_q, h_q), so a
//    histogram is an exact integer sum: any CTA order, any number of GPUs and
//    the sibling subtraction all give bit-identical results.
//  * One CTA owns (work item = piece of one node's row list) x (tile of TW
//    features).  Its private sub-histogram lives in shared memory as two int32
//    planes G[bin][lane], H[bin][lane] with lane = feature inside the tile: a
//    warp updates one row at a time, every lane a different feature, so the 32
//    shared-memory atomics of a warp instruction always hit 32 different banks
//    whatever the bin values are (no bank conflicts, no same-address conflicts,
//    also for skewed or sorted columns).
//  * Rows are fetched by row id, one 32-byte sector per row and tile (uint8 bins,
//    TW = 32), staged per warp in shared memory and read back transposed.
//  * A work item has at most 2^(31 - quant_bits) rows, so an int32 plane cannot
//    overflow; the CTA then adds its plane to the level's int64 histogram in
//    global memory with one red.global.add.u64 per non-zero word.
#include "kernels.cuh"

namespace arb {

namespace {

__device__ __forceinline__ void quantize(float g, float h, const float sg, const float sh, bool pair,
                                         int &gq, int &hq) {
  gq = __float2int_rn(g * sg);
  hq = pair ? max(1, __float2int_rn(h * sh)) : 1;
}

__device__ __forceinline__ void flush_planes(const int *G, const int *H, long long *dst) {
  for (int w = threadIdx.x; w < kHistWords; w += blockDim.x) {
    const int g = G[w];
    const int h = H[w];
    if (g != 0) atomicAdd(reinterpret_cast<unsigned long long *>(dst + 2 * w), (unsigned long long)(long long)g);
    if (h != 0) atomicAdd(reinterpret_cast<unsigned long long *>(dst + 2 * w + 1), (unsigned long long)(long long)h);
  }
}

// uint8 bins, 32 features per tile, 256 bins.
template <bool PAIR, bool IDENT>
__global__ void __launch_bounds__(kHistThreads, 3)
hist_u8_kernel(const unsigned char *__restrict__ bins, const size_t pitch, const int NT,
               const unsigned *__restrict__ rowid, const void *__restrict__ grad,
               const WorkItem *__restrict__ items, const int *__restrict__ n_items,
               long long *__restrict__ hist, const QuantScale *__restrict__ qs) {
  extern __shared__ __align__(16) int smem[];
  int *G = smem;
  int *H = smem + kHistWords;
  constexpr int kWarps = kHistThreads / 32;
  // per warp: 32 rows x 32 bytes of bins, then 32 x (g_q, h_q)
  unsigned char *stage_bins = reinterpret_cast<unsigned char *>(smem + 2 * kHistWords);
  int2 *stage_gh = reinterpret_cast<int2 *>(stage_bins + kWarps * 1024);

  if (int(blockIdx.x) >= *n_items) return;
  const WorkItem item = items[blockIdx.x];
  const int tile = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  for (int w = threadIdx.x; w < 2 * kHistWords; w += kHistThreads) smem[w] = 0;
  __syncthreads();

  const float sg = qs->sg, sh = qs->sh;
  unsigned char *my_bins = stage_bins + warp * 1024;
  int2 *my_gh = stage_gh + warp * 32;
  const unsigned char *tile_base = bins + size_t(tile) * 32;

  for (unsigned base = warp * 32; base < item.len; base += kWarps * 32) {
    const unsigned pos = base + lane;
    const bool valid = pos < item.len;
    uint4 a = make_uint4(0, 0, 0, 0), b = a;
    int gq = 0, hq = 0;
    if (valid) {
      const unsigned rid = IDENT ? item.begin + pos : rowid[item.begin + pos];
      const uint4 *src = reinterpret_cast<const uint4 *>(tile_base + size_t(rid) * pitch);
      a = __ldg(src);
      b = __ldg(src + 1);
      if (PAIR) {
        const float2 g = __ldg(reinterpret_cast<const float2 *>(grad) + rid);
        quantize(g.x, g.y, sg, sh, true, gq, hq);
      } else {
        const float g = __ldg(reinterpret_cast<const float *>(grad) + rid);
        quantize(g, 1.0f, sg, sh, false, gq, hq);
      }
    }
    uint4 *dst = reinterpret_cast<uint4 *>(my_bins + lane * 32);
    dst[0] = a;
    dst[1] = b;
    my_gh[lane] = make_int2(gq, hq);
    __syncwarp();
    const int nvalid = min(32u, item.len - base);
#pragma unroll 4
    for (int j = 0; j < nvalid; ++j) {
      const int bin = my_bins[j * 32 + lane];
      const int2 gh = my_gh[j];
      atomicAdd(&G[bin * 32 + lane], gh.x);
      atomicAdd(&H[bin * 32 + lane], gh.y);
    }
    __syncwarp();
  }
  __syncthreads();
  flush_planes(G, H, hist + (size_t(item.node) * NT + tile) * kHistWords * 2);
}

// Any bin width / tile width: lane = (row in group, feature in tile).
template <bool PAIR, bool IDENT, typename BIN_T>
__global__ void __launch_bounds__(kHistThreads, 3)
hist_generic_kernel(const unsigned char *__restrict__ bins, const size_t pitch, const int NT,
                    const int TW, const int F, const unsigned *__restrict__ rowid,
                    const void *__restrict__ grad, const WorkItem *__restrict__ items,
                    const int *__restrict__ n_items, long long *__restrict__ hist,
                    const QuantScale *__restrict__ qs) {
  extern __shared__ __align__(16) int smem[];
  int *G = smem;
  int *H = smem + kHistWords;
  if (int(blockIdx.x) >= *n_items) return;
  const WorkItem item = items[blockIdx.x];
  const int tile = blockIdx.y;
  for (int w = threadIdx.x; w < 2 * kHistWords; w += kHistThreads) smem[w] = 0;
  __syncthreads();
  const float sg = qs->sg, sh = qs->sh;
  const int rows_per_pass = kHistThreads / TW;
  const int f_in_tile = threadIdx.x % TW;
  const int rsub = threadIdx.x / TW;
  const int f = tile * TW + f_in_tile;
  if (f < F) {
    for (unsigned pos = rsub; pos < item.len; pos += rows_per_pass) {
      const unsigned rid = IDENT ? item.begin + pos : rowid[item.begin + pos];
      const BIN_T bin = reinterpret_cast<const BIN_T *>(bins + size_t(rid) * pitch)[f];
      int gq, hq;
      if (PAIR) {
        const float2 g = __ldg(reinterpret_cast<const float2 *>(grad) + rid);
        quantize(g.x, g.y, sg, sh, true, gq, hq);
      } else {
        const float g = __ldg(reinterpret_cast<const float *>(grad) + rid);
        quantize(g, 1.0f, sg, sh, false, gq, hq);
      }
      atomicAdd(&G[int(bin) * TW + f_in_tile], gq);
      atomicAdd(&H[int(bin) * TW + f_in_tile], hq);
    }
  }
  __syncthreads();
  flush_planes(G, H, hist + (size_t(item.node) * NT + tile) * kHistWords * 2);
}

__global__ void subtract_kernel(long long *__restrict__ level_hist,
                                const long long *__restrict__ parent_hist,
                                const int *__restrict__ built_child, const size_t words_per_node,
                                const size_t total) {
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

// opt in to more than 48 KB of dynamic shared memory, once per call site
#define ARB_SET_SMEM(kernel, bytes)                                                        \
  do {                                                                                     \
    static bool done__ = false;                                                            \
    if (!done__) {                                                                         \
      ARB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                    int(bytes)));                                          \
      done__ = true;                                                                       \
    }                                                                                      \
  } while (0)

}  // namespace

void launch_hist(const HistLaunch &a, cudaStream_t s) {
  const Geometry &g = a.geo;
  const dim3 grid(a.max_items, g.NT);
  const bool ident = a.rowid == nullptr;
  if (g.bin_bytes == 1 && g.TW == 32) {
    const size_t smem = 2 * kHistWords * 4 + (kHistThreads / 32) * (1024 + 256);
#define ARB_LAUNCH(P, I)                                                                       \
  do {                                                                                         \
    ARB_SET_SMEM((hist_u8_kernel<P, I>), smem);                                                    \
    hist_u8_kernel<P, I><<<grid, kHistThreads, smem, s>>>(g.bins, g.pitch, g.NT, a.rowid,      \
                                                          a.grad, a.items, a.n_items, a.hist,  \
                                                          a.qs);                               \
  } while (0)
    if (a.pair) {
      if (ident) ARB_LAUNCH(true, true); else ARB_LAUNCH(true, false);
    } else {
      if (ident) ARB_LAUNCH(false, true); else ARB_LAUNCH(false, false);
    }
#undef ARB_LAUNCH
  } else {
    const size_t smem = 2 * kHistWords * 4;
#define ARB_LAUNCH(P, I, T)                                                                    \
  do {                                                                                         \
    ARB_SET_SMEM((hist_generic_kernel<P, I, T>), smem);                                            \
    hist_generic_kernel<P, I, T><<<grid, kHistThreads, smem, s>>>(                             \
      g.bins, g.pitch, g.NT, g.TW, g.F, a.rowid, a.grad, a.items, a.n_items, a.hist, a.qs);    \
  } while (0)
#define ARB_LAUNCH_T(T)                                                    \
  do {                                                                     \
    if (a.pair) {                                                          \
      if (ident) ARB_LAUNCH(true, true, T); else ARB_LAUNCH(true, false, T);   \
    } else {                                                               \
      if (ident) ARB_LAUNCH(false, true, T); else ARB_LAUNCH(false, false, T); \
    }                                                                      \
  } while (0)
    if (g.bin_bytes == 1) ARB_LAUNCH_T(unsigned char); else ARB_LAUNCH_T(unsigned short);
#undef ARB_LAUNCH_T
#undef ARB_LAUNCH
  }
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_subtract(long long *level_hist, const long long *parent_hist, const int *built_child,
                     int n_parents, int NT, cudaStream_t s) {
  const size_t words_per_node = size_t(NT) * kHistWords * 2;
  const size_t total = words_per_node * n_parents;
  const int threads = 256;
  const int blocks = int(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
  subtract_kernel<<<blocks, threads, 0, s>>>(level_hist, parent_hist, built_child, words_per_node,
                                             total);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

}  // namespace arb
