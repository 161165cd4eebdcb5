// Split search over the histograms of one level (rows S and A of the hot path;
// replaces cub::DeviceScan + hist_gain_kernel + hist_apply_candidates of the
// reference, src/core/hist_tree_grower.cu:9-102,393-450).
//
// One CTA per (node, feature tile).  A thread owns one feature of the tile and
// 8 consecutive bins: it sums them, the CTA turns the partial sums into the
// prefix offsets of the segmented scan, and the thread then walks its bins
// again evaluating the reference's gain for "rows with bin <= b go left".  The
// candidates of a node meet in one 64-bit atomicMax whose integer order is the
// reference's tie order: higher gain, then lower feature id
// (hist_tree_grower.cu:59-60), then higher bin (builder.h:45-46).
#include "kernels.cuh"

namespace arb {

namespace {

constexpr int kSplitThreads = 1024;
constexpr int kBinsPerThread = kHistWords / kSplitThreads;  // 8

__device__ __forceinline__ unsigned long long pack_key(float gain, int fid, int bin) {
  return (static_cast<unsigned long long>(__float_as_uint(gain)) << 32) |
         (static_cast<unsigned long long>(0xFFFFFu - unsigned(fid)) << 12) | unsigned(bin);
}

// Decode the winner of a node and sum its left side (one warp).
__device__ void finalize_node(const long long *__restrict__ hist, const long long *__restrict__ count_hist,
                              const int *__restrict__ cat_candidates, const int *__restrict__ fmap,
                              unsigned long long key, NodeRec *__restrict__ rec, int node, int TW, int NT,
                              int lane) {
  NodeRec r = rec[node];
  r.lcnt = r.tcnt = 0;
  if (count_hist) {  // rows of the node: all bins of its first feature
    const long long *cb = count_hist + size_t(node) * NT * kHistWords * 2;
    long long c = 0;
    for (int b = lane; b < kHistWords / TW; b += 32) c += cb[size_t(b) * TW * 2 + 1];
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    r.tcnt = unsigned(c);
  }
  if (key == 0ull) {  // no positive gain: all rows stay left (hist_tree_grower.cu:84-93)
    r.gain = 0.0f;
    r.fid = -1;
    r.bin = -1;
    r.lg = r.tg;
    r.lh = r.th;
    r.lcnt = r.tcnt;
  } else {
    r.gain = __uint_as_float(unsigned(key >> 32));
    // the key names the histogram's column; the record names the feature behind it
    const int col = int(0xFFFFFu - unsigned((key >> 12) & 0xFFFFFu));
    r.fid = fmap ? fmap[col] : col;
    r.bin = int(key & 0xFFFu);
    const int tile = col / TW, fl = col % TW;
    const long long *base = hist + (size_t(node) * NT + tile) * kHistWords * 2;
    // a categorical winner sends one bin left, a dense one every bin up to the winner
    const int first_bin = (cat_candidates && cat_candidates[r.fid] > 0) ? r.bin : 0;
    long long g = 0, h = 0;
#pragma unroll 8  // the loads of eight turns are in flight together: one latency, not eight
    for (int b = first_bin + lane; b <= r.bin; b += 32) {
      g += base[(size_t(b) * TW + fl) * 2];
      h += base[(size_t(b) * TW + fl) * 2 + 1];
    }
    for (int o = 16; o > 0; o >>= 1) {
      g += __shfl_down_sync(0xffffffffu, g, o);
      h += __shfl_down_sync(0xffffffffu, h, o);
    }
    r.lg = g;
    r.lh = h;
    if (count_hist) {
      const long long *cbase = count_hist + (size_t(node) * NT + tile) * kHistWords * 2;
      long long c = 0;
      for (int b = first_bin + lane; b <= r.bin; b += 32) c += cbase[(size_t(b) * TW + fl) * 2 + 1];
      for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
      r.lcnt = unsigned(c);
    }
  }
  r.left_count = 0;
  if (lane == 0) rec[node] = r;
}

template <bool PAIR, bool COUNTS>
__global__ void __launch_bounds__(kSplitThreads)
split_kernel(const long long *__restrict__ hist, const long long *__restrict__ count_hist,
             const unsigned char *__restrict__ feature_active, const int *__restrict__ cat_candidates,
             const int *__restrict__ fmap, unsigned long long *__restrict__ keys, unsigned *__restrict__ done,
             NodeRec *__restrict__ rec, const QuantScale *__restrict__ qs, const GainParams gp,
             const int TW, const int NT, const int F, const int hist_size, const int parts) {
  overlap_release();
  overlap_wait();
  __shared__ long long part_g[kSplitThreads], part_h[kSplitThreads];
  __shared__ float best_gain[kSplitThreads];
  __shared__ int best_bin[kSplitThreads];
  __shared__ bool is_last;
  const int node = blockIdx.x, tile = blockIdx.y;
  const int lane = threadIdx.x % TW;
  const int chunk = threadIdx.x / TW;
  const int nchunks = kSplitThreads / TW;
  const int f = tile * TW + lane;
  const long long *base = hist + (size_t(node) * NT + tile) * kHistWords * 2;
  const int bin0 = chunk * kBinsPerThread;

  longlong2 v[kBinsPerThread];
  long long sg = 0, sh = 0;
#pragma unroll
  for (int k = 0; k < kBinsPerThread; ++k) {
    v[k] = *reinterpret_cast<const longlong2 *>(base + (size_t(bin0 + k) * TW + lane) * 2);
    sg += v[k].x;
    sh += v[k].y;
  }
  // row counts of the thread's bins ((g, h) objectives with min_leaf_size > 1 only)
  long long cv[COUNTS ? kBinsPerThread : 1];
  long long sc = 0;
  if (COUNTS) {
    const long long *cbase = count_hist + (size_t(node) * NT + tile) * kHistWords * 2;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
      cv[k] = cbase[(size_t(bin0 + k) * TW + lane) * 2 + 1];
      sc += cv[k];
    }
  }
  long long og = 0, oh = 0, tg = 0, th = 0, oc = 0, tcn = 0;
  if (TW == 32) {
    // A warp is one chunk of all 32 features.  The sums change places through shared memory
    // (slot feature * 32 + (chunk ^ feature): no bank conflict on the feature-major side), so
    // that warp f holds the 32 chunk sums of feature f and scans them with shuffles; the
    // offsets travel back through the same slots.
    __shared__ long long tot_g[32], tot_h[32];
    const int slot = lane * 32 + (chunk ^ lane);
    part_g[slot] = sg;
    part_h[slot] = sh;
    __syncthreads();
    {
      const int f_w = chunk, c_l = lane;  // this thread now stands for (chunk c_l, feature f_w)
      const int at = f_w * 32 + (c_l ^ f_w);
      const long long vg = part_g[at], vh = part_h[at];
      long long xg = vg, xh = vh;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const long long ug = __shfl_up_sync(0xffffffffu, xg, o), uh = __shfl_up_sync(0xffffffffu, xh, o);
        if (c_l >= o) {
          xg += ug;
          xh += uh;
        }
      }
      part_g[at] = xg - vg;
      part_h[at] = xh - vh;
      if (c_l == 31) {
        tot_g[f_w] = xg;
        tot_h[f_w] = xh;
      }
    }
    __syncthreads();
    og = part_g[slot];
    oh = part_h[slot];
    tg = tot_g[lane];
    th = tot_h[lane];
    if (COUNTS) {  // the same exchange once more for the counts
      __syncthreads();
      part_g[slot] = sc;
      __syncthreads();
      const int f_w = chunk, c_l = lane;
      const int at = f_w * 32 + (c_l ^ f_w);
      const long long vc = part_g[at];
      long long xc = vc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const long long uc = __shfl_up_sync(0xffffffffu, xc, o);
        if (c_l >= o) xc += uc;
      }
      part_g[at] = xc - vc;
      if (c_l == 31) tot_g[f_w] = xc;
      __syncthreads();
      oc = part_g[slot];
      tcn = tot_g[lane];
    }
  } else {
    part_g[threadIdx.x] = sg;
    part_h[threadIdx.x] = sh;
    __syncthreads();
    for (int c = 0; c < nchunks; ++c) {
      const long long g = part_g[c * TW + lane], h = part_h[c * TW + lane];
      if (c < chunk) {
        og += g;
        oh += h;
      }
      tg += g;
      th += h;
    }
    if (COUNTS) {
      __syncthreads();
      part_g[threadIdx.x] = sc;
      __syncthreads();
      for (int c = 0; c < nchunks; ++c) {
        const long long v = part_g[c * TW + lane];
        if (c < chunk) oc += v;
        tcn += v;
      }
    }
  }
  if (tile == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    rec[node].tg = tg;
    rec[node].th = th;
  }
  float bgain = 0.0f;
  int bbin = -1;
  // the gain search of a (node, tile) is dealt to `parts` CTAs (a power of two): bin k of
  // every thread's 8 goes to CTA k % parts; all of them redo the cheap prefix sums above,
  // so the long double-precision chains run side by side instead of one after another
  // f is a column of the histogram; the column order is the feature order (the map ascends),
  // so ties between columns fall like ties between features
  const int feat = (f < F && fmap) ? fmap[f] : f;
  const bool active = f < F && feature_active[feat];
  // > 0: a categorical feature; a candidate sends the rows of ONE bin left (builder.h:75-105)
  const int ncand = (active && cat_candidates) ? cat_candidates[feat] : 0;
  if (active && th != 0) {
    const double isg = qs->inv_sg, ish = qs->inv_sh;
    const double dtg = double(tg) * isg, dth = double(th) * ish;
    long long rg = og, rh = oh, rc = oc;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
      const int bin = bin0 + k;
      rg += v[k].x;
      rh += v[k].y;
      if (COUNTS) rc += cv[k];
      if (bin >= hist_size) continue;  // ids >= hist_size hold missing values: never a threshold
      if ((k & (parts - 1)) != int(blockIdx.z)) continue;  // another CTA's candidate
      if (ncand > 0 && bin >= ncand) continue;  // the shared bin of the rare categories
      const long long lg = ncand > 0 ? v[k].x : rg, lh = ncand > 0 ? v[k].y : rh;
      unsigned long long lc, tc;
      if (COUNTS) {  // true row counts (gain.cu:125-134 gates every candidate on them)
        lc = (unsigned long long)(ncand > 0 ? cv[k] : rc);
        tc = (unsigned long long)tcn;
      } else if (PAIR) {  // h_q >= 1 for every row, so a zero sum means "no rows"
        lc = lh > 0;
        tc = lc + ((th - lh) > 0);
      } else {  // h_q == 1 for every row: the sum is the row count
        lc = (unsigned long long)lh;
        tc = (unsigned long long)th;
      }
      const float gain = split_gain<PAIR>(double(lg) * isg, double(lh) * ish, dtg, dth, lc, tc, gp);
      if (gain > 0.0f && gain >= bgain) {
        bgain = gain;
        bbin = bin;
      }
    }
  }
  best_gain[threadIdx.x] = bgain;
  best_bin[threadIdx.x] = bbin;
  __syncthreads();
  if (chunk == 0 && active) {
    for (int c = 1; c < nchunks; ++c) {
      const float g = best_gain[c * TW + lane];
      if (g > 0.0f && g >= bgain) {
        bgain = g;
        bbin = best_bin[c * TW + lane];
      }
    }
    if (bgain > 0.0f) atomicMax(&keys[node], pack_key(bgain, f, bbin));
  }
  // the last tile of the node to arrive turns the packed winner into the record
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&done[node], 1u) == unsigned(NT * parts - 1);
  __syncthreads();
  if (is_last && threadIdx.x < 32) {
    __threadfence();
    const unsigned long long key = atomicMax(&keys[node], 0ull);
    finalize_node(hist, COUNTS ? count_hist : nullptr, cat_candidates, fmap, key, rec, node, TW, NT, threadIdx.x);
  }
}

}  // namespace

void launch_split(const SplitLaunch &a, cudaStream_t s) {
  // keys (u64 per node) and arrival counters (u32 per node) live in one buffer, cleared by
  // the level's plan kernel
  unsigned *done = reinterpret_cast<unsigned *>(a.keys + a.max_nodes);
  // Small levels: the double-precision gain arithmetic of a (node, tile) is spread over up
  // to 8 CTAs, which all re-read the tile.  A CTA of 1024 threads with 64 registers each
  // has an SM to itself, so more CTAs than SMs would only run as a second wave: the gains
  // they share out would wait in line all the same, after re-reading the tile.
  const int sms = device_sm_count();
  int parts = kBinsPerThread;
  while (parts > 1 && a.L * a.geo.NT * parts > sms) parts >>= 1;
  const dim3 grid(a.L, a.geo.NT, parts);
  if (a.pair && a.count_hist)
    launch_overlapped(split_kernel<true, true>, grid, kSplitThreads, 0, s, a.hist, a.count_hist, a.feature_active,
                      a.cat_candidates, a.feature_map, a.keys, done, a.rec, a.qs, a.gp, a.geo.TW, a.geo.NT, a.geo.F, a.geo.hist_size, parts);
  else if (a.pair)
    launch_overlapped(split_kernel<true, false>, grid, kSplitThreads, 0, s, a.hist, a.count_hist, a.feature_active,
                      a.cat_candidates, a.feature_map, a.keys, done, a.rec, a.qs, a.gp, a.geo.TW, a.geo.NT, a.geo.F, a.geo.hist_size, parts);
  else
    launch_overlapped(split_kernel<false, false>, grid, kSplitThreads, 0, s, a.hist, a.count_hist, a.feature_active,
                      a.cat_candidates, a.feature_map, a.keys, done, a.rec, a.qs, a.gp, a.geo.TW, a.geo.NT, a.geo.F, a.geo.hist_size, parts);
  count_launch();
}

}  // namespace arb
