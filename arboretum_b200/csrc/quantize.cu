// Feature quantizer (row Q of the hot path; reference: DataMatrix::InitHistInternal,
// src/io/io.cu:349-435, with ValueSegmentIterator :27-142, SegmentLength :144-153,
// ThresholdOutputIterator :255-271 and build_histogram :293-312).
//
// Thresholds must be bit-identical to the reference's, so the column is sorted in
// fp32 radix order (the toolkit's cub::DeviceRadixSort, the same primitive the
// reference calls) and the border scan is restated as three small kernels:
//   count borders per block -> scan the block counts -> for every border i with
//   inclusive border count c, slot k = min(c + 1, i / seg + 1) - 2 receives
//   min(thr[k], float((s[i] + s[i-1]) * 0.5)).
// Binning then maps all features of all rows in one pass over the row-major fp32
// matrix and writes the row-major bin matrix the histogram kernels read.
#include <atomic>

#include <cub/device/device_radix_sort.cuh>

#include "kernels.cuh"

namespace arb {

namespace {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

__device__ __forceinline__ bool is_border(const float *s, size_t i) { return i > 0 && s[i] != s[i - 1]; }

// The three border kernels take several columns of n sorted values at once (grid.y = column):
// column c lies at s + c * n, its block counts at block_count + c * gridDim.x, its
// thresholds at thr + c * hist_size.
__global__ void border_count_kernel(const float *__restrict__ s, size_t n, unsigned *block_count) {
  __shared__ unsigned warp_sums[kScanThreads / 32];
  s += size_t(blockIdx.y) * n;
  block_count += size_t(blockIdx.y) * gridDim.x;
  const size_t base = size_t(blockIdx.x) * kScanTile;
  unsigned c = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {  // any order will do for a count: coalesced
    const size_t i = base + size_t(k) * kScanThreads + threadIdx.x;
    if (i < n) c += is_border(s, i);
  }
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned t = 0;
    for (int w = 0; w < kScanThreads / 32; ++w) t += warp_sums[w];
    block_count[blockIdx.x] = t;
  }
}

// exclusive scan of the block counts, one CTA (the array has n / 2048 entries)
__global__ void border_scan_kernel(unsigned *block_count, int nblocks) {
  __shared__ unsigned warp_sums[32];
  __shared__ unsigned carry_s;
  block_count += size_t(blockIdx.y) * nblocks;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < nblocks; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const unsigned v = i < nblocks ? block_count[i] : 0u;
    unsigned incl = v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    unsigned off = 0;
    for (int w = 0; w < warp; ++w) off += warp_sums[w];
    const unsigned carry = carry_s;
    if (i < nblocks) block_count[i] = carry + off + incl - v;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = carry + off + incl;
    __syncthreads();
  }
}

__device__ __forceinline__ void atomic_min_float(float *addr, float v) {  // io.cu:258-269
  int *a = reinterpret_cast<int *>(addr);
  int old = *a;
  while (v < __int_as_float(old)) {
    const int seen = atomicCAS(a, old, __float_as_int(v));
    if (seen == old) break;
    old = seen;
  }
}

__global__ void border_apply_kernel(const float *__restrict__ s, size_t n, size_t seg, int hist_size,
                                    const unsigned *__restrict__ block_off, float *thr) {
  __shared__ unsigned warp_sums[kScanThreads / 32];
  // the tile and the value before it, read coalesced; a thread then walks 8 consecutive
  // values, so slot p is kept at p + p / 32: the 32 lanes' strides of 8 fall on 32 banks
  __shared__ float tile[kScanTile + 1 + (kScanTile + 1) / 32 + 1];
  s += size_t(blockIdx.y) * n;
  block_off += size_t(blockIdx.y) * gridDim.x;
  thr += size_t(blockIdx.y) * hist_size;
  const size_t tile_base = size_t(blockIdx.x) * kScanTile;
  for (int p = threadIdx.x; p < kScanTile + 1; p += kScanThreads) {
    const size_t i = tile_base + size_t(p);  // tile[p] = s[i - 1]
    tile[p + (p >> 5)] = (i >= 1 && i - 1 < n) ? s[i - 1] : 0.0f;
  }
  __syncthreads();
  auto at = [&](int p) { return tile[p + (p >> 5)]; };
  const int first = threadIdx.x * kScanItems;
  const size_t base = tile_base + size_t(first);
  bool flag[kScanItems];
  unsigned c = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    const size_t i = base + k;
    flag[k] = i > 0 && i < n && at(first + k + 1) != at(first + k);
    c += flag[k];
  }
  unsigned incl = c;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  unsigned run = block_off[blockIdx.x] + incl - c;
  for (int w = 0; w < warp; ++w) run += warp_sums[w];
  // Midpoints grow with the position, so a slot keeps the midpoint of its first border.
  // Only that one is sent to the atomic minimum: a thread drops a border that falls in
  // the slot of its previous one, and among the lanes of a warp that hold the same slot
  // in the same step the lowest lane (the smallest position) speaks for all.
  long long last_slot = -1;
  // base / seg once per thread; the quotient of the following positions by counting up
  unsigned long long quot = base / seg, rem = base - quot * seg;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    long long slot = -1;
    float mid = 0.0f;
    if (flag[k]) {
      ++run;  // inclusive border count of position i (io.cu:144-153)
      mid = float((at(first + k + 1) + at(first + k)) * 0.5);  // io.cu:72-79
      const long long a = (long long)run + 1, b = (long long)quot + 1;  // quot = i / seg
      slot = (a < b ? a : b) - 2;  // io.cu:257
      // slots past the table are a defect of the reference (out-of-range write); skipped
      if (slot >= hist_size || slot == last_slot) slot = -1;
      if (slot >= 0) last_slot = slot;
    }
    if (++rem == seg) {
      rem = 0;
      ++quot;
    }
    // most steps have no candidate in the whole warp (a thread's later borders fall in the
    // slot of its first): the vote is cheap, the match is not
    if (__any_sync(0xffffffffu, slot >= 0)) {
      const unsigned peers = __match_any_sync(0xffffffffu, slot);
      if (slot >= 0 && (peers & ((1u << lane) - 1)) == 0) atomic_min_float(thr + slot, mid);
    }
  }
}

// Several short columns sorted in one go: a key is (column, value in radix order), 64 bits.
// A 1 M-row column alone is six small launches of the library's sort; thirty-two of them as
// one array of keys are the same six launches over thirty-two times the data.  The value
// half is the float's bit pattern turned the way the library's own float sort turns it
// (negative values inverted, the sign bit of the others set), so the order is the same.
__device__ __forceinline__ unsigned radix_order(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float radix_order_back(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__global__ void pack_sort_keys_kernel(const float *__restrict__ cols, size_t n, size_t total,
                                      unsigned long long *__restrict__ keys) {
  for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += size_t(gridDim.x) * blockDim.x)
    keys[e] = ((unsigned long long)(e / n) << 32) | radix_order(cols[e]);
}
__global__ void unpack_sort_keys_kernel(const unsigned long long *__restrict__ keys, size_t total,
                                        float *__restrict__ cols) {
  for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += size_t(gridDim.x) * blockDim.x)
    cols[e] = radix_order_back(unsigned(keys[e]));
}

__global__ void fill_inf_kernel(float *thr, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) thr[i] = INFINITY;
}

// columns [f0, f0 + nf) of the row-major matrix -> column-major out[(f - f0) * n + row];
// 32 x 32 tiles through shared memory, every NaN becomes the positive quiet NaN, which sorts last as in the reference's sort
__global__ void transpose_f32_kernel(const float *__restrict__ X, size_t n, int F, int f0, int nf,
                                     float *__restrict__ out) {
  __shared__ float tile[32][33];
  const size_t r0 = size_t(blockIdx.x) * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
  for (int j = ty; j < 32; j += 8) {
    const size_t r = r0 + j;
    const int c = c0 + tx;
    float v = (r < n && c < nf) ? X[r * F + f0 + c] : 0.0f;
    if (v != v) v = __int_as_float(0x7fc00000);
    tile[j][tx] = v;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int c = c0 + j;
    const size_t r = r0 + tx;
    if (c < nf && r < n) out[size_t(c) * n + r] = tile[tx][j];
  }
}

// cuda_helpers.h:207-222 over v[0..size-2] = thr, v[size-1] = +INF (io.cu:297-310)
__device__ __forceinline__ unsigned lower_bound_thr(const float *thr, int size, float x) {
  unsigned l = 0, h = unsigned(size);
  while (l < h) {
    const unsigned mid = (l + h) / 2;
    const float v = int(mid) < size - 1 ? __ldg(thr + mid) : INFINITY;
    if (x <= v) h = mid; else l = mid + 1;
  }
  return l;
}

// 32 rows x 32 features per CTA through shared memory: coalesced on both sides
template <typename BIN_T>
__global__ void transpose_bins_kernel(const unsigned char *__restrict__ bins, size_t pitch, size_t n,
                                      int F, BIN_T *__restrict__ out) {
  __shared__ BIN_T tile[32][33];
  const size_t r0 = size_t(blockIdx.x) * 32;
  const int f0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
  for (int j = ty; j < 32; j += 8) {
    const size_t r = r0 + j;
    const int f = f0 + tx;
    tile[j][tx] = (r < n && f < F) ? reinterpret_cast<const BIN_T *>(bins + r * pitch)[f] : BIN_T(0);
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int f = f0 + j;
    const size_t r = r0 + tx;
    if (f < F && r < n) out[size_t(f) * n + r] = tile[tx][j];
  }
}

// The same for uint8 bins whose row count is a multiple of 16: a CTA takes 256 rows of one
// tile of 32 features, reads whole 32-byte row chunks with 16-byte loads (two lanes per row),
// turns them in shared memory and writes 256 consecutive bytes per feature with 16-byte stores.
constexpr int kTurnRows = 256;
constexpr int kTurnStride = kTurnRows + 16;
__global__ void __launch_bounds__(256)
transpose_bins_u8_kernel(const unsigned char *__restrict__ bins, size_t pitch, size_t n, int F,
                         unsigned char *__restrict__ out) {
  __shared__ __align__(16) unsigned char tile[32 * kTurnStride];
  const size_t r0 = size_t(blockIdx.x) * kTurnRows;
  const int f0 = blockIdx.y * 32;
  const int half = threadIdx.x & 1;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int row = p * 128 + (threadIdx.x >> 1);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r0 + row < n) v = __ldg(reinterpret_cast<const uint4 *>(bins + (r0 + row) * pitch + f0 + half * 16));
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 16; ++j)
      tile[(half * 16 + j) * kTurnStride + row] = (unsigned char)(w[j >> 2] >> (8 * (j & 3)));
  }
  __syncthreads();
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int e = p * 256 + threadIdx.x;  // 32 features x 16 chunks of 16 rows
    const int f = e >> 4, c = e & 15;
    const size_t r = r0 + size_t(c) * 16;
    if (f0 + f < F && r < n)  // n is a multiple of 16: a chunk is inside or outside as a whole
      *reinterpret_cast<uint4 *>(out + size_t(f0 + f) * n + r) =
        *reinterpret_cast<const uint4 *>(tile + f * kTurnStride + c * 16);
  }
}

// unpadded uint8 rows [n][F] -> padded rows [n][pitch] (padding bytes zero), one
// 32-bit word of the padded row per thread
__global__ void pad_rows_kernel(const unsigned char *__restrict__ raw, int F, size_t n,
                                unsigned *__restrict__ out, int words_per_row) {
  const size_t total = n * size_t(words_per_row);
  for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += size_t(gridDim.x) * blockDim.x) {
    const size_t r = e / words_per_row;
    const int f0 = int(e - r * words_per_row) * 4;
    const unsigned char *src = raw + r * F;
    unsigned w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (f0 + k < F) w |= unsigned(src[f0 + k]) << (8 * k);
    out[e] = w;
  }
}

template <typename BIN_T>
__global__ void place_columns_kernel(const BIN_T *__restrict__ src, size_t n, int ccol, int f0,
                                     unsigned char *__restrict__ bins, size_t pitch, bool by_column) {
  const size_t total = n * size_t(ccol);
  for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += size_t(gridDim.x) * blockDim.x) {
    // by_column: src[c * n + r] (consecutive threads take consecutive rows of a column)
    const size_t r = by_column ? e % n : e / ccol;
    const int c = by_column ? int(e / n) : int(e - r * ccol);
    reinterpret_cast<BIN_T *>(bins + r * pitch)[f0 + c] = src[e];
  }
}

// the columns map[0..n_cols) of every row, side by side: one 32-bit word of the output row per
// thread (4 uint8 or 2 uint16 bins), padding words zero
template <typename BIN_T>
__global__ void compact_columns_kernel(const unsigned char *__restrict__ bins, size_t pitch, size_t n,
                                       const int *__restrict__ map, int n_cols,
                                       unsigned *__restrict__ out, int out_words) {
  constexpr int kPer = 4 / int(sizeof(BIN_T));
  const size_t total = n * size_t(out_words);
  for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += size_t(gridDim.x) * blockDim.x) {
    const size_t r = e / out_words;
    const int j0 = int(e - r * out_words) * kPer;
    const BIN_T *src = reinterpret_cast<const BIN_T *>(bins + r * pitch);
    unsigned w = 0;
#pragma unroll
    for (int k = 0; k < kPer; ++k)
      if (j0 + k < n_cols) w |= unsigned(src[__ldg(map + j0 + k)]) << (8 * int(sizeof(BIN_T)) * k);
    out[e] = w;
  }
}

// The same from the feature-major copy (uint8, row count a multiple of 16): only the wanted
// columns are read, 256 consecutive rows of a column at a time with 16-byte loads; a CTA turns
// 32 columns x 256 rows in shared memory and writes 32-byte row chunks of the output.
__global__ void __launch_bounds__(256)
compact_columns_cm_u8_kernel(const unsigned char *__restrict__ bins_cm, size_t n,
                             const int *__restrict__ map, int n_cols, unsigned char *__restrict__ out,
                             size_t out_pitch, bool tile_major) {
  __shared__ __align__(16) unsigned char tile[32 * kTurnStride];
  const size_t r0 = size_t(blockIdx.x) * kTurnRows;
  const int j0 = blockIdx.y * 32;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int e = p * 256 + threadIdx.x;  // 32 columns x 16 chunks of 16 rows
    const int j = e >> 4, c = e & 15;
    const size_t r = r0 + size_t(c) * 16;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (j0 + j < n_cols && r < n)
      v = __ldg(reinterpret_cast<const uint4 *>(bins_cm + size_t(__ldg(map + j0 + j)) * n + r));
    *reinterpret_cast<uint4 *>(tile + j * kTurnStride + c * 16) = v;
  }
  __syncthreads();
  const int half = threadIdx.x & 1;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int row = p * 128 + (threadIdx.x >> 1);
    if (r0 + row >= n) continue;
    unsigned w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j)
      w[j >> 2] |= unsigned(tile[(half * 16 + j) * kTurnStride + row]) << (8 * (j & 3));
    unsigned char *dst = tile_major ? out + (size_t(blockIdx.y) * n + r0 + row) * 32 + half * 16
                                    : out + (r0 + row) * out_pitch + j0 + half * 16;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__global__ void u8_to_f32_kernel(const unsigned char *__restrict__ src, float *__restrict__ dst,
                                 size_t count) {
  for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < count;
       e += size_t(gridDim.x) * blockDim.x)
    dst[e] = float(src[e]);
}

template <typename BIN_T>
__global__ void binning_kernel(const float *__restrict__ X, size_t n, int F,
                               const float *__restrict__ thr, const int *__restrict__ fsize,
                               int hist_size, bool missing_bin, unsigned char *__restrict__ bins,
                               size_t pitch) {
  const size_t total = n * size_t(F);
  // (row, feature) of the element are carried along instead of divided out every time
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  const size_t stride_rows = stride / F;
  const int stride_f = int(stride - stride_rows * F);
  size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  size_t r = e / F;
  int f = int(e - r * F);
  for (; e < total; e += stride, r += stride_rows, f += stride_f) {
    if (f >= F) {
      f -= F;
      ++r;
    }
    const float x = X[e];
    unsigned b;
    if (missing_bin && x != x)
      b = unsigned(hist_size);
    else
      b = lower_bound_thr(thr + size_t(f) * hist_size, fsize[f], x);
    reinterpret_cast<BIN_T *>(bins + r * pitch)[f] = BIN_T(b);
  }
}


// uint8 bins with at most 255 thresholds per feature: a CTA keeps the tables of a tile of 32
// features in shared memory, entry i of the tile's feature l at i * 32 + l.  A warp bins one
// row of the tile at a time, lane l its feature l, with a fixed 8-step search: lane l only ever
// touches bank l, so no step has a bank conflict whatever the values are.  Same result as
// lower_bound_thr: entries from size - 1 on read +INF, so a value that is not NaN stops at
// size - 1 at the latest, and NaN (which compares false everywhere) gets `size` like there.
constexpr int kBinRowsPerStep = 4;  // rows a warp has in flight
__global__ void __launch_bounds__(256)
binning_tile_kernel(const float *__restrict__ X, size_t n, int F, const float *__restrict__ thr,
                    const int *__restrict__ fsize, int hist_size, bool missing_bin,
                    unsigned char *__restrict__ bins, size_t pitch) {
  __shared__ float tbl[255 * 32];
  const int f_tile = blockIdx.y * 32;
  for (int e = threadIdx.x; e < 255 * 32; e += 256) {
    const int f = f_tile + (e & 31), i = e >> 5;
    float v = INFINITY;
    if (f < F && i < hist_size && i < fsize[f] - 1) v = thr[size_t(f) * hist_size + i];
    tbl[e] = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = f_tile + lane;
  if (f >= F) return;
  const unsigned nan_bin = missing_bin ? unsigned(hist_size) : unsigned(fsize[f]);
  const float *t = tbl + lane;
  const size_t step_rows = size_t(gridDim.x) * 8;
  for (size_t r = size_t(blockIdx.x) * 8 + warp; r < n; r += step_rows * kBinRowsPerStep) {
    float v[kBinRowsPerStep];
#pragma unroll
    for (int k = 0; k < kBinRowsPerStep; ++k) {
      const size_t rk = r + size_t(k) * step_rows;
      v[k] = rk < n ? X[rk * F + f] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < kBinRowsPerStep; ++k) {
      const size_t rk = r + size_t(k) * step_rows;
      if (rk >= n) break;
      unsigned b = nan_bin;
      if (v[k] == v[k]) {
        int pos = 0;
#pragma unroll
        for (int step = 128; step >= 1; step >>= 1)
          if (!(v[k] <= t[(pos + step - 1) * 32])) pos += step;
        b = unsigned(pos);
      }
      bins[rk * pitch + f] = (unsigned char)b;
    }
  }
}

}  // namespace

size_t thresholds_scratch_words(size_t n) { return (n + kScanTile - 1) / kScanTile + 1; }

void launch_thresholds_columns(const float *sorted_cols, size_t n, int nf, int hist_size, float *thr,
                               unsigned *scratch, cudaStream_t s) {
  if (nf <= 0) return;
  fill_inf_kernel<<<ceil_div(size_t(hist_size) * nf, 256), 256, 0, s>>>(thr, hist_size * nf);  // io.cu:387
  ARB_CUDA(cudaGetLastError());
  count_launch();
  if (n < 2) return;
  const int nblocks = int((n + kScanTile - 1) / kScanTile);
  const size_t seg = std::max<size_t>(1, n / size_t(hist_size));  // io.cu:376-377
  border_count_kernel<<<dim3(nblocks, nf), kScanThreads, 0, s>>>(sorted_cols, n, scratch);
  border_scan_kernel<<<dim3(1, nf), 1024, 0, s>>>(scratch, nblocks);
  border_apply_kernel<<<dim3(nblocks, nf), kScanThreads, 0, s>>>(sorted_cols, n, seg, hist_size, scratch, thr);
  ARB_CUDA(cudaGetLastError());
  count_launch(3);
}

void launch_thresholds(const float *sorted, size_t n, int hist_size, float *thr, unsigned *scratch,
                       cudaStream_t s) {
  launch_thresholds_columns(sorted, n, 1, hist_size, thr, scratch, s);
}

void launch_transpose_bins(const unsigned char *bins, size_t pitch, int bin_bytes, size_t n, int F,
                           unsigned char *bins_cm, cudaStream_t s) {
  if (bin_bytes == 1 && n % 16 == 0 && pitch % 32 == 0 && reinterpret_cast<uintptr_t>(bins) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(bins_cm) % 16 == 0) {
    const dim3 grid_fast(unsigned((n + kTurnRows - 1) / kTurnRows), unsigned((F + 31) / 32));
    transpose_bins_u8_kernel<<<grid_fast, 256, 0, s>>>(bins, pitch, n, F, bins_cm);
    ARB_CUDA(cudaGetLastError());
    count_launch();
    return;
  }
  const dim3 grid(unsigned((n + 31) / 32), unsigned((F + 31) / 32));
  if (bin_bytes == 1)
    transpose_bins_kernel<unsigned char><<<grid, 256, 0, s>>>(bins, pitch, n, F, bins_cm);
  else
    transpose_bins_kernel<unsigned short><<<grid, 256, 0, s>>>(bins, pitch, n, F,
                                                               reinterpret_cast<unsigned short *>(bins_cm));
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_pad_rows(const unsigned char *raw, int F, size_t n, unsigned char *bins, size_t pitch,
                     cudaStream_t s) {
  if (n == 0) return;
  const int words = int(pitch / 4);
  const size_t total = n * size_t(words);
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(device_sm_count()) * 32));
  pad_rows_kernel<<<grid, 256, 0, s>>>(raw, F, n, reinterpret_cast<unsigned *>(bins), words);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

bool compact_columns_tile_major_ok(int bin_bytes, size_t n, const unsigned char *bins_cm) {
  return bins_cm && bin_bytes == 1 && n % 16 == 0 && reinterpret_cast<uintptr_t>(bins_cm) % 16 == 0;
}

void launch_compact_columns(const unsigned char *bins, size_t pitch, int bin_bytes, size_t n, const int *map,
                            int n_cols, unsigned char *out, size_t out_pitch, cudaStream_t s,
                            const unsigned char *bins_cm, bool tile_major) {
  if (n == 0 || n_cols == 0) return;
  if (compact_columns_tile_major_ok(bin_bytes, n, bins_cm) && out_pitch % 32 == 0 &&
      reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const dim3 grid_cm(unsigned((n + kTurnRows - 1) / kTurnRows), unsigned(out_pitch / 32));
    compact_columns_cm_u8_kernel<<<grid_cm, 256, 0, s>>>(bins_cm, n, map, n_cols, out, out_pitch, tile_major);
    ARB_CUDA(cudaGetLastError());
    count_launch();
    return;
  }
  ARB_CHECK(!tile_major, "the tile-by-tile copy needs the feature-major matrix");
  const int words = int(out_pitch / 4);
  const size_t total = n * size_t(words);
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(device_sm_count()) * 32));
  if (bin_bytes == 1)
    compact_columns_kernel<unsigned char><<<grid, 256, 0, s>>>(bins, pitch, n, map, n_cols,
                                                               reinterpret_cast<unsigned *>(out), words);
  else
    compact_columns_kernel<unsigned short><<<grid, 256, 0, s>>>(bins, pitch, n, map, n_cols,
                                                                reinterpret_cast<unsigned *>(out), words);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_place_columns(const void *src, size_t n, int ccol, int f0, unsigned char *bins, size_t pitch,
                          int bin_bytes, cudaStream_t s, bool by_column) {
  if (n == 0 || ccol == 0) return;
  const size_t total = n * size_t(ccol);
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(device_sm_count()) * 32));
  if (bin_bytes == 1)
    place_columns_kernel<unsigned char><<<grid, 256, 0, s>>>(static_cast<const unsigned char *>(src), n, ccol, f0,
                                                            bins, pitch, by_column);
  else
    place_columns_kernel<unsigned short><<<grid, 256, 0, s>>>(static_cast<const unsigned short *>(src), n, ccol,
                                                             f0, bins, pitch, by_column);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_u8_to_f32(const unsigned char *src, float *dst, size_t count, cudaStream_t s) {
  if (count == 0) return;
  const int grid = int(std::min<size_t>((count + 255) / 256, size_t(device_sm_count()) * 32));
  u8_to_f32_kernel<<<grid, 256, 0, s>>>(src, dst, count);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_transpose_columns(const float *X, size_t n, int F, int f0, int nf, float *out,
                              cudaStream_t s) {
  const dim3 grid(unsigned((n + 31) / 32), unsigned((nf + 31) / 32));
  transpose_f32_kernel<<<grid, 256, 0, s>>>(X, n, F, f0, nf, out);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

size_t sort_floats_temp_bytes(size_t n) {
  size_t bytes = 0;
  ARB_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, bytes, static_cast<const float *>(nullptr),
                                          static_cast<float *>(nullptr), n, 0, 32, nullptr));
  return bytes;
}

void sort_floats(const float *in, float *out, size_t n, DevBuf &tmp, cudaStream_t s) {
  size_t bytes = 0;
  ARB_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, bytes, in, out, n, 0, 32, s));
  if (tmp.bytes < bytes) tmp.alloc(bytes);
  ARB_CUDA(cub::DeviceRadixSort::SortKeys(tmp.p, bytes, in, out, n, 0, 32, s));
}

namespace {
int column_key_bits(int nf) {
  int bits = 0;
  while ((1 << bits) < nf) ++bits;
  return 32 + bits;
}
}  // namespace

size_t sort_columns_temp_bytes(size_t n, int nf) {
  size_t bytes = 0;
  ARB_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, bytes, static_cast<const unsigned long long *>(nullptr),
                                          static_cast<unsigned long long *>(nullptr), n * size_t(nf), 0,
                                          column_key_bits(nf), nullptr));
  return bytes;
}

void sort_columns(float *cols, size_t n, int nf, unsigned long long *keys_a, unsigned long long *keys_b,
                  DevBuf &tmp, cudaStream_t s) {
  const size_t total = n * size_t(nf);
  if (total == 0) return;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(device_sm_count()) * 32));
  pack_sort_keys_kernel<<<grid, 256, 0, s>>>(cols, n, total, keys_a);
  size_t bytes = 0;
  ARB_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, bytes, keys_a, keys_b, total, 0, column_key_bits(nf), s));
  if (tmp.bytes < bytes) tmp.alloc(bytes);
  ARB_CUDA(cub::DeviceRadixSort::SortKeys(tmp.p, bytes, keys_a, keys_b, total, 0, column_key_bits(nf), s));
  unpack_sort_keys_kernel<<<grid, 256, 0, s>>>(keys_b, total, cols);
  ARB_CUDA(cudaGetLastError());
  count_launch(2);
}

void launch_binning(const float *X, size_t n, int F, const float *thr, const int *fsize,
                    int hist_size, bool missing_bin, unsigned char *bins, size_t pitch, int bin_bytes,
                    cudaStream_t s) {
  if (n == 0) return;
  if (bin_bytes == 1 && hist_size <= 255) {
    const int tiles = (F + 31) / 32;
    const size_t row_blocks = (n + 7) / 8;
    // every CTA loads its tile's tables once: enough CTAs to fill the SMs, not more
    const int grid_x = int(std::min<size_t>(row_blocks, size_t(std::max(1, device_sm_count() * 8 / tiles))));
    binning_tile_kernel<<<dim3(grid_x, tiles), 256, 0, s>>>(X, n, F, thr, fsize, hist_size, missing_bin, bins,
                                                           pitch);
    ARB_CUDA(cudaGetLastError());
    count_launch();
    return;
  }
  const int threads = 256;
  const size_t total = n * size_t(F);
  const int grid = int(std::min<size_t>((total + threads - 1) / threads, size_t(device_sm_count()) * 32));
  if (bin_bytes == 1)
    binning_kernel<unsigned char><<<grid, threads, 0, s>>>(X, n, F, thr, fsize, hist_size, missing_bin,
                                                           bins, pitch);
  else
    binning_kernel<unsigned short><<<grid, threads, 0, s>>>(X, n, F, thr, fsize, hist_size,
                                                            missing_bin, bins, pitch);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

// ---------------------------------------------------------------------------
// Threshold search without any allocation.
//
// Some callers may not allocate device memory at all: a host that has handed the
// whole GPU to one arena at start-up and forbids cudaMalloc afterwards, a service
// that runs inside a fixed memory budget, or code that is called while an
// allocation could not be tolerated (latency-critical sections, other libraries'
// callbacks).  The border scan of the threshold search needs one word of scratch
// per 2048 sorted values; here that scratch is a fixed array inside the library
// image, so the call only launches kernels.  The price is a size limit and the
// fact that every call on a device shares the one array.
// ---------------------------------------------------------------------------
namespace {
constexpr long long kStaticThresholdRows = 1ll << 26;  // 67,108,864 values per call
constexpr size_t kStaticScratchWords = size_t(kStaticThresholdRows / kScanTile) + 1;
// 128 KB of device memory per GPU that loads the library, held until exit
static __device__ __align__(256) unsigned g_threshold_scratch[kStaticScratchWords];
// device address of the array, per device; filled on a device's first call (two threads that
// make it together store the same value)
std::atomic<unsigned *> g_scratch_ptr[kMaxDevices];
}  // namespace
}  // namespace arb

extern "C" const char *AThresholdsNoAlloc(const float *sorted_device, long long n, int hist_size,
                                           float *thr_device, void *stream) {
  using namespace arb;
  static thread_local std::string error;
  try {
    ARB_CHECK(sorted_device && thr_device, "NULL argument");
    ARB_CHECK(hist_size > 0 && hist_size < 2048, "hist_size must be in [1, 2047]");
    ARB_CHECK(n >= 0, "negative row count");
    if (n > kStaticThresholdRows)
      throw std::runtime_error("AThresholdsNoAlloc: " + std::to_string(n) + " values exceed the limit of " +
                               std::to_string(kStaticThresholdRows) +
                               " of the built-in scratch array; use AQuantize for larger columns");
    int dev = 0;
    ARB_CUDA(cudaGetDevice(&dev));
    ARB_CHECK(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
    unsigned *scratch = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!scratch) {
      // In host code the array's name is only a handle: the kernels need the address
      // the symbol has on THIS device, which the runtime hands out here.
      void *p = nullptr;
      ARB_CUDA(cudaGetSymbolAddress(&p, g_threshold_scratch));
      scratch = static_cast<unsigned *>(p);
      g_scratch_ptr[dev].store(scratch, std::memory_order_release);
    }
    // block counts are rewritten in full for the blocks of this call, so nothing of an
    // earlier call's contents is read: no clearing is needed
    launch_thresholds(sorted_device, size_t(n), hist_size, thr_device, scratch,
                      static_cast<cudaStream_t>(stream));
    return nullptr;
  } catch (const std::exception &e) {
    error = e.what();
    return error.c_str();
  }
}
