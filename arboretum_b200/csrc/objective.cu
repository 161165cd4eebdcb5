// Objective gradients, leaf weights, prediction update and inference (rows G, W, U
// and Pred of the hot path; reference: src/core/objective.cu:15-56,
// src/core/objective.h:19-113, src/core/garden.cu:45-76,487-503,
// src/core/garden.h:70-90).
#include <cfloat>
#include <cstddef>

#include "kernels.cuh"

namespace arb {

namespace {

// objective.h:66-68: the exponential is evaluated in float, the rest in double.
// (1.0 / d and the correctly rounded reciprocal are the same number)
__device__ __forceinline__ float sigmoid(float x) { return float(__drcp_rn(1.0 + double(expf(-x)))); }
// single-precision stand-in, good to a few units in the last place: only used to bound the
// round's largest |gradient| and hessian, never for a gradient that is summed
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
constexpr float kMaxSlack = 1.0f + 1.0f / 1024.0f;  // the bound errs upwards by far more than that error

// Fixed-point conversion with a dither: floor(v * scale + u), u in [0, 1) a hash of (row of
// the whole data set, round, salt).  Rounding to nearest would give every row with the same
// gradient the same error -- and first rounds are full of equal gradients, so a node's sum
// would be off by rows x error; with the dither the errors of equal values spread evenly
// over one step and cancel like those of unequal ones.  The hash depends on the row's index
// in the whole data set, so shards and row chunks quantise a row like one GPU does.
// no_dither (round == 0xffffffff): plain round-to-nearest.
constexpr unsigned kNoDither = 0xffffffffu;
__device__ __forceinline__ float dither(unsigned long long row, unsigned round, unsigned salt) {
  unsigned x = unsigned(row) ^ (unsigned(row >> 32) * 0x9E3779B1u) ^ (round * 0x85EBCA6Bu) ^ salt;
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return float(x >> 8) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ int to_fixed(float v, float scale, unsigned long long row, unsigned round,
                                        unsigned salt, int lim) {
  const int q = round == kNoDither ? __float2int_rn(v * scale)
                                   : __float2int_rd(v * scale + dither(row, round, salt));
  return max(-lim, min(lim, q));  // |q| < 2^quant_bits, whatever the dither adds at the largest value
}

// The round's largest |gradient| and hessian: one atomicMax per CTA and value, and only
// when the CTA's maximum beats what is already there (the counters share a cache line, so
// thousands of unconditional atomics would queue up behind one another).
__device__ __forceinline__ void block_max_to(QuantScale *qs, float mg, float mh) {
  __shared__ float warp_g[32], warp_h[32];
  for (int o = 16; o > 0; o >>= 1) {
    mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
    mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, o));
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    warp_g[warp] = mg;
    warp_h[warp] = mh;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    mg = lane < nw ? warp_g[lane] : 0.0f;
    mh = lane < nw ? warp_h[lane] : 0.0f;
    for (int o = 16; o > 0; o >>= 1) {
      mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
      mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, o));
    }
    if (lane == 0) {
      const volatile unsigned *seen_g = &qs->max_g_bits, *seen_h = &qs->max_h_bits;
      if (mg > 0.0f && __float_as_uint(mg) > *seen_g) atomicMax(&qs->max_g_bits, __float_as_uint(mg));
      if (mh > 0.0f && __float_as_uint(mh) > *seen_h) atomicMax(&qs->max_h_bits, __float_as_uint(mh));
    }
  }
}

// Sign convention of the reference: grad = negative gradient (objective.cu:31,45).
// Two passes over (y, yhat): EMIT = false finds the maxima that fix the round's fixed-point
// scale, EMIT = true computes the same floats again and stores them as integers
// (g_q = rint(g * sg), h_q = max(1, rint(h * sh))): the float gradients never touch memory.
// n4: the rows taken four at a time with 16-byte loads and stores (a multiple of 4; 0 when
// a pointer is not 16-byte aligned), so that a thread has enough bytes in flight to keep the
// memory busy; the other rows go one at a time.
template <bool EMIT>
__global__ void grad_linear_kernel(const float *__restrict__ y, const float *__restrict__ yhat,
                                   int *__restrict__ grad, QuantScale *qs, size_t n,
                                   unsigned long long row0, unsigned round, int lim, size_t n4) {
  overlap_release();
  overlap_wait();
  float m = 0.0f;
  const float sg = EMIT ? qs->sg : 0.0f;
  const int lim_g = EMIT ? qs->lim_g : lim;  // the scale may have taken extra bits from the tails
  const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, total = size_t(gridDim.x) * blockDim.x;
  auto row = [&](float yi, float yh, size_t i) -> int {
    const float g = yi - yh;
    if (EMIT) return to_fixed(g, sg, row0 + i, round, 0u, lim_g);
    m = fmaxf(m, fabsf(g));
    return 0;
  };
  for (size_t i = tid * 4; i < n4; i += total * 4) {
    const float4 a = *reinterpret_cast<const float4 *>(y + i), b = *reinterpret_cast<const float4 *>(yhat + i);
    const int4 q = make_int4(row(a.x, b.x, i), row(a.y, b.y, i + 1), row(a.z, b.z, i + 2), row(a.w, b.w, i + 3));
    if (EMIT) *reinterpret_cast<int4 *>(grad + i) = q;
  }
  for (size_t i = n4 + tid; i < n; i += total) {
    const int q = row(y[i], yhat[i], i);
    if (EMIT) grad[i] = q;
  }
  if (!EMIT) block_max_to(qs, m, 0.0f);
}

// reg:linear between the two passes: rows with |g| >= max|g| / 2^(j + 1), j = 0 .. 7
__global__ void grad_linear_tail_kernel(const float *__restrict__ y, const float *__restrict__ yhat,
                                        QuantScale *qs, size_t n, size_t n4) {
  overlap_release();
  overlap_wait();
  __shared__ unsigned block_cnt[kTailLevels];
  if (threadIdx.x < kTailLevels) block_cnt[threadIdx.x] = 0;
  __syncthreads();
  const float mx = __uint_as_float(qs->max_g_bits);
  float t[kTailLevels];
  unsigned c[kTailLevels];
#pragma unroll
  for (int j = 0; j < kTailLevels; ++j) {
    t[j] = ldexpf(mx, -(j + 1));
    c[j] = 0;
  }
  auto row = [&](float yi, float yh) {
    const float a = fabsf(yi - yh);
#pragma unroll
    for (int j = 0; j < kTailLevels; ++j) c[j] += a >= t[j] ? 1u : 0u;
  };
  const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, total = size_t(gridDim.x) * blockDim.x;
  for (size_t i = tid * 4; i < n4; i += total * 4) {
    const float4 a = *reinterpret_cast<const float4 *>(y + i), b = *reinterpret_cast<const float4 *>(yhat + i);
    row(a.x, b.x), row(a.y, b.y), row(a.z, b.z), row(a.w, b.w);
  }
  for (size_t i = n4 + tid; i < n; i += total) row(y[i], yhat[i]);
#pragma unroll
  for (int j = 0; j < kTailLevels; ++j) {
    const unsigned w = __reduce_add_sync(0xffffffffu, c[j]);
    if ((threadIdx.x & 31) == 0 && w) atomicAdd(&block_cnt[j], w);
  }
  __syncthreads();
  if (threadIdx.x < kTailLevels && block_cnt[threadIdx.x]) atomicAdd(&qs->tail[threadIdx.x], block_cnt[threadIdx.x]);
}

template <bool EMIT>
__global__ void grad_logistic_kernel(const float *__restrict__ y, const float *__restrict__ yhat,
                                     int2 *__restrict__ grad, QuantScale *qs, size_t n,
                                     unsigned long long row0, unsigned round, int lim, size_t n4) {
  overlap_release();
  overlap_wait();
  float mg = 0.0f, mh = 0.0f;
  const float sg = EMIT ? qs->sg : 0.0f, sh = EMIT ? qs->sh : 0.0f;
  const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, total = size_t(gridDim.x) * blockDim.x;
  auto row = [&](float yi, float yh, size_t i) -> int2 {
    const float s = EMIT ? sigmoid(yh) : sigmoid_fast(yh);
    const float2 g = make_float2(yi - s, s * (1.0f - s));
    if (EMIT)  // h_q >= 1 for every row, so that a zero hessian sum means "no rows"
      return make_int2(to_fixed(g.x, sg, row0 + i, round, 0u, lim),
                       max(1, to_fixed(g.y, sh, row0 + i, round, 0x68E31DA4u, lim)));
    mg = fmaxf(mg, fabsf(g.x));
    mh = fmaxf(mh, g.y);
    return make_int2(0, 0);
  };
  for (size_t i = tid * 4; i < n4; i += total * 4) {
    const float4 a = *reinterpret_cast<const float4 *>(y + i), b = *reinterpret_cast<const float4 *>(yhat + i);
    const int2 q0 = row(a.x, b.x, i), q1 = row(a.y, b.y, i + 1), q2 = row(a.z, b.z, i + 2), q3 = row(a.w, b.w, i + 3);
    if (EMIT) {
      *reinterpret_cast<int4 *>(grad + i) = make_int4(q0.x, q0.y, q1.x, q1.y);
      *reinterpret_cast<int4 *>(grad + i + 2) = make_int4(q2.x, q2.y, q3.x, q3.y);
    }
  }
  for (size_t i = n4 + tid; i < n; i += total) {
    const int2 q = row(y[i], yhat[i], i);
    if (EMIT) grad[i] = q;
  }
  if (!EMIT) block_max_to(qs, mg * kMaxSlack, mh * kMaxSlack);
}

// multi:softmax as the reference intends it (objective.cu:60-89, objective.h:100-112):
// probabilities in double, g_k = 1[k == label] - p_k, h_k = 2 p_k (1 - p_k).
__global__ void grad_softmax_kernel(const unsigned char *__restrict__ label,
                                    const float *__restrict__ yhat, float2 *__restrict__ grad,
                                    QuantScale *qs, size_t n, int K) {
  float mg = 0.0f, mh = 0.0f;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x) {
    double sum = 0.0;
    for (int k = 0; k < K; ++k) sum += exp(double(yhat[size_t(k) * n + i]));
    const int lab = label[i];
    for (int k = 0; k < K; ++k) {
      const double p = exp(double(yhat[size_t(k) * n + i])) / sum;
      const float2 g = make_float2(float((k == lab ? 1.0 : 0.0) - p), float(2.0 * p * (1.0 - p)));
      grad[size_t(k) * n + i] = g;
      mg = fmaxf(mg, fabsf(g.x));
      mh = fmaxf(mh, g.y);
    }
  }
  block_max_to(qs, mg, mh);
}

__global__ void finish_scales_kernel(QuantScale *qs, int quant_bits, bool pair, bool tails, int stage) {
  overlap_release();
  overlap_wait();
  // largest |g| < 2^e  =>  |g * 2^(quant_bits - e)| < 2^quant_bits
  int eg = 0, eh = 0;
  const float mg = __uint_as_float(qs->max_g_bits), mh = __uint_as_float(qs->max_h_bits);
  if (mg > 0.0f && mg <= FLT_MAX) frexpf(mg, &eg);
  if (mh > 0.0f && mh <= FLT_MAX) frexpf(mh, &eh);
  int s = quant_bits - eg;  // sg = 2^s
  if (stage == 2) {
    s = 1024 - int(qs->neg_s);
  } else if (tails && mg > 0.0f && mg <= FLT_MAX) {
    // An int32 sub-histogram takes at most cap = 2^(31 - quant_bits) rows.  Walking the tail
    // counts from the top bounds the sum of the cap largest |g| by B x max|g|; every
    // quantised value exceeds |g| sg by less than 1, so sg (B max|g|) + cap < 2^31 keeps the
    // sums of any such rows inside an int32.  At most 24 - quant_bits bits are added, so that
    // the largest value stays exactly representable in the float arithmetic of to_fixed.
    const double cap = ldexp(1.0, 31 - quant_bits);
    double remaining = cap, B = 0.0, prev = 0.0;
    for (int j = 0; j < kTailLevels; ++j) {
      const double cj = double(qs->tail[j]);
      const double take = fmin(remaining, cj - prev);
      B += take * ldexp(1.0, -j);
      remaining -= take;
      prev = cj;
    }
    B += remaining * ldexp(1.0, -kTailLevels);
    const double room = (ldexp(1.0, 31) - 2.0 * cap) / (B * double(mg));
    int s_tail = 0;
    frexp(room, &s_tail);  // room in [2^(s_tail - 1), 2^s_tail)
    s_tail -= 1;
    const int most = s + max(0, 24 - quant_bits);
    s = min(max(s, s_tail), most);
  }
  qs->neg_s = unsigned(1024 - s);
  if (stage == 1) return;
  qs->sg = ldexpf(1.0f, s);
  qs->inv_sg = ldexp(1.0, -s);
  // |g| sg < 2^(eg + s) <= 2^24
  qs->lim_g = (1 << min(24, max(quant_bits, eg + s))) - 1;
  if (pair) {
    qs->sh = ldexpf(1.0f, quant_bits - eh);
    qs->inv_sh = ldexp(1.0, eh - quant_bits);
  } else {
    qs->sh = 1.0f;
    qs->inv_sh = 1.0;
  }
}

// `rows` rows per plane (several planes: multi:softmax); plane k of row r is element k * rows + r
__global__ void quantize_pair_kernel(float2 *grad, size_t n, size_t rows, const QuantScale *__restrict__ qs,
                                     unsigned long long row0, unsigned round, int lim) {
  const float sg = qs->sg, sh = qs->sh;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x) {
    const float2 g = grad[i];
    const size_t plane = i / rows;
    const unsigned long long row = row0 + (i - plane * rows);
    const unsigned salt = unsigned(plane) * 0x27D4EB2Fu;
    // h_q >= 1 for every row, so that a zero hessian sum means "no rows"
    reinterpret_cast<int2 *>(grad)[i] = make_int2(to_fixed(g.x, sg, row, round, salt, lim),
                                                  max(1, to_fixed(g.y, sh, row, round, salt ^ 0x68E31DA4u, lim)));
  }
}

__global__ void quantize_single_kernel(float *grad, size_t n, const QuantScale *__restrict__ qs, int lim) {
  const float sg = qs->sg;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    reinterpret_cast<int *>(grad)[i] = to_fixed(grad[i], sg, i, kNoDither, 0u, lim);
}

template <bool PAIR, bool COUNTS>
__global__ void leaf_weights_kernel(LeafLaunch a) {
  overlap_release();
  overlap_wait();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= a.L) return;
  const NodeRec r = a.last_rec[n];
  const double isg = a.qs->inv_sg, ish = a.qs->inv_sh;
  const long long rg = r.tg - r.lg, rh = r.th - r.lh;
  // counts only gate `c >= min_leaf_size`; see split.cu for the PAIR stand-in
  const unsigned lc = COUNTS ? r.lcnt : PAIR ? unsigned(r.lh > 0) : unsigned(r.lh);
  const unsigned rc = COUNTS ? r.tcnt - r.lcnt : PAIR ? unsigned(rh > 0) : unsigned(rh);
  // garden.cu:487-503, split.cu:25-35: eta is applied to the float weight
  a.leaf_w[2 * n] = leaf_weight<PAIR>(double(r.lg) * isg, double(r.lh) * ish, lc, a.mcw, a.mls,
                                      a.lambda, a.alpha, a.mlw) * a.eta;
  a.leaf_w[2 * n + 1] = leaf_weight<PAIR>(double(rg) * isg, double(rh) * ish, rc, a.mcw, a.mls,
                                          a.lambda, a.alpha, a.mlw) * a.eta;
}

// RegTree::Predict garden.h:70-90 (dense features): x < threshold goes left, so
// NaN goes right; trees are added in order, in float, like the reference's loop
// in Garden::Predict garden.cu:643-657.
__global__ void predict_kernel(const float *__restrict__ X, size_t n, int F, PackedTree t,
                               int first_tree, int n_trees, int depth, float *__restrict__ out,
                               size_t plane_stride, const unsigned *__restrict__ cat, int ccol) {
  const int nodes = (1 << depth) - 1;
  const int leaves = 1 << (depth - 1);
  const int offset = leaves - 1;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x) {
    const float *row = X + i * F;
    for (int k = first_tree; k < first_tree + n_trees; ++k) {
      const int *fid = t.fid + size_t(k) * nodes;
      const float *thr = t.thr + size_t(k) * nodes;
      int node = 0;
      for (int j = 1; j < depth; ++j) {
        const int f = fid[node];
        // garden.h:79-84: dense features go left below the threshold, categorical ones when
        // the value is the node's category
        const bool left = f < F ? row[f] < thr[node]
                                : (cat != nullptr && f - F < ccol &&
                                   cat[i * size_t(ccol) + (f - F)] == t.category[size_t(k) * nodes + node]);
        node = left ? 2 * node + 1 : 2 * node + 2;
      }
      out[size_t(t.label[k]) * plane_stride + i] += t.weights[size_t(k) * leaves + node - offset];
    }
  }
}

__global__ void link_kernel(int objective, int K, size_t n, const float *__restrict__ in,
                            float *__restrict__ out) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x) {
    if (objective == 1) {  // objective.h:58-64
      out[i] = sigmoid(in[i]);
    } else if (objective == 3) {  // objective.h:80-113
      double sum = 0.0;
      for (int k = 0; k < K; ++k) sum += exp(double(in[size_t(k) * n + i]));
      for (int k = 0; k < K; ++k) out[i * K + k] = float(exp(double(in[size_t(k) * n + i])) / sum);
    } else {
      out[i] = in[i];
    }
  }
}

template <typename T>
__global__ void fill_kernel(T *dst, size_t n, T v) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    dst[i] = v;
}

inline int grid_for(size_t n, int threads) {
  return int(std::min<size_t>((n + threads - 1) / threads, size_t(device_sm_count()) * 16));
}

}  // namespace

void launch_gradients(int objective, int K, size_t n, const float *y, const unsigned char *label,
                      const float *yhat, void *grad, QuantScale *qs, bool emit, cudaStream_t s,
                      unsigned long long row0, unsigned round, int quant_bits) {
  const int lim = (1 << quant_bits) - 1;
  if (!emit)  // the maxima, the scale exponent, the clamp and the tail counts
    ARB_CUDA(cudaMemsetAsync(&qs->max_g_bits, 0, sizeof(QuantScale) - offsetof(QuantScale, max_g_bits), s));
  const int threads = 256;
  const int grid = grid_for(n, threads);
  const bool aligned = (reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(yhat) |
                        reinterpret_cast<uintptr_t>(grad)) % 16 == 0;
  const size_t n4 = aligned ? n / 4 * 4 : 0;
  const int grid4 = grid_for(n4 / 4 + (n - n4), threads);
  if (objective == 0) {
    if (emit) launch_overlapped(grad_linear_kernel<true>, grid4, threads, 0, s, y, yhat, static_cast<int *>(grad), qs, n, row0, round, lim, n4);
    else launch_overlapped(grad_linear_kernel<false>, grid4, threads, 0, s, y, yhat, static_cast<int *>(grad), qs, n, row0, round, lim, n4);
  } else if (objective == 1) {
    if (emit) launch_overlapped(grad_logistic_kernel<true>, grid4, threads, 0, s, y, yhat, static_cast<int2 *>(grad), qs, n, row0, round, lim, n4);
    else launch_overlapped(grad_logistic_kernel<false>, grid4, threads, 0, s, y, yhat, static_cast<int2 *>(grad), qs, n, row0, round, lim, n4);
  } else if (!emit) {  // the K double-precision exponentials per row are not computed twice:
    grad_softmax_kernel<<<grid, threads, 0, s>>>(label, yhat, static_cast<float2 *>(grad), qs, n, K);
  } else {             // the floats are stored by the first pass and turned into integers in place
    quantize_pair_kernel<<<grid_for(n * K, threads), threads, 0, s>>>(static_cast<float2 *>(grad), n * K, n, qs,
                                                                      row0, round, lim);
  }
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_finish_scales(QuantScale *qs, int K, int quant_bits, bool pair, cudaStream_t s, bool tails,
                          int stage) {
  (void)K;
  launch_overlapped(finish_scales_kernel, 1, 1, 0, s, qs, quant_bits, pair, tails, stage);
  count_launch();
}

void launch_gradient_tails(size_t n, const float *y, const float *yhat, QuantScale *qs, cudaStream_t s) {
  const int threads = 256;
  const bool aligned = (reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(yhat)) % 16 == 0;
  const size_t n4 = aligned ? n / 4 * 4 : 0;
  launch_overlapped(grad_linear_tail_kernel, grid_for(n4 / 4 + (n - n4), threads), threads, 0, s, y, yhat, qs, n, n4);
  count_launch();
}

void launch_quantize_grads(void *grad, size_t n, bool pair, const QuantScale *qs, int quant_bits,
                           cudaStream_t s) {
  const int threads = 256;
  const int lim = (1 << quant_bits) - 1;
  if (pair)
    quantize_pair_kernel<<<grid_for(n, threads), threads, 0, s>>>(static_cast<float2 *>(grad), n, n, qs, 0ull,
                                                                  kNoDither, lim);
  else
    quantize_single_kernel<<<grid_for(n, threads), threads, 0, s>>>(static_cast<float *>(grad), n, qs, lim);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_leaf_weights(const LeafLaunch &a, cudaStream_t s) {
  const int threads = 128;
  if (a.pair && a.counts)
    launch_overlapped(leaf_weights_kernel<true, true>, ceil_div(a.L, threads), threads, 0, s, a);
  else if (a.pair)
    launch_overlapped(leaf_weights_kernel<true, false>, ceil_div(a.L, threads), threads, 0, s, a);
  else
    launch_overlapped(leaf_weights_kernel<false, false>, ceil_div(a.L, threads), threads, 0, s, a);
  count_launch();
}

void launch_predict(const float *X, size_t n, int F, PackedTree t, int first_tree, int n_trees,
                    int depth, float *out, cudaStream_t s, size_t plane_stride, const unsigned *cat,
                    int ccol) {
  if (n_trees <= 0 || n == 0) return;
  const int threads = 256;
  predict_kernel<<<grid_for(n, threads), threads, 0, s>>>(X, n, F, t, first_tree, n_trees, depth, out,
                                                          plane_stride ? plane_stride : n, cat, ccol);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_fill(float *dst, size_t n, float value, cudaStream_t s) {
  if (n == 0) return;
  fill_kernel<float><<<grid_for(n, 256), 256, 0, s>>>(dst, n, value);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_fill_u32(unsigned *dst, size_t n, unsigned value, cudaStream_t s) {
  if (n == 0) return;
  fill_kernel<unsigned><<<grid_for(n, 256), 256, 0, s>>>(dst, n, value);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void launch_link(int objective, int K, size_t n, const float *internal, float *out, cudaStream_t s) {
  if (n == 0) return;
  const int threads = 256;
  link_kernel<<<grid_for(n, threads), threads, 0, s>>>(objective, K, n, internal, out);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

}  // namespace arb
