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
                              const int *__restrict__ cat_candidates, unsigned long long key,
                              NodeRec *__restrict__ rec, int node, int TW, int NT, int lane) {
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
    r.fid = int(0xFFFFFu - unsigned((key >> 12) & 0xFFFFFu));
    r.bin = int(key & 0xFFFu);
    const int tile = r.fid / TW, fl = r.fid % TW;
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
             unsigned long long *__restrict__ keys, unsigned *__restrict__ done,
             NodeRec *__restrict__ rec, const QuantScale *__restrict__ qs, const GainParams gp,
             const int TW, const int NT, const int F, const int hist_size, const int parts) {
  overlap_release();
  overlap_wait();
  __shared__ long long part_g[kSplitThreads], part_h[kSplitThreads];
  __shared__ float best_gain[kSplitThreads];
  __shared__ int best_bin[kSplitThreads];
  __shared__ bool is_last;
  __shared__ unsigned q_count;            // candidates that survived the single-precision look
  __shared__ unsigned long long s_key;    // the CTA's best exact candidate, packed
  __shared__ long long s_tg, s_th, s_tcn; // the node's totals (every feature's bins add up to them)
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
  if (threadIdx.x == 0) {  // lane 0 of a tile is one of its real features
    s_tg = tg;
    s_th = th;
    s_tcn = tcn;
    q_count = 0;
    s_key = 0ull;
  }
  // the gain search of a (node, tile) is dealt to `parts` CTAs (a power of two): bin k of
  // every thread's 8 goes to CTA k % parts; all of them redo the cheap prefix sums above,
  // so the long double-precision chains run side by side instead of one after another
  const bool active = f < F && feature_active[f];
  // > 0: a categorical feature; a candidate sends the rows of ONE bin left (builder.h:75-105)
  const int ncand = (active && cat_candidates) ? cat_candidates[f] : 0;
  // The exact gain is some 150 double-precision operations per candidate, and only the largest
  // matters.  So every candidate is first valued in single precision; the exact arithmetic
  // then runs for those within a slack of the CTA's largest approximate value that is twenty
  // times what single precision can be off by (1e-5 x (2 x parent term + difference), see
  // split_gain_approx).  The winner and the tie order come from exact values only.
  const double isg = qs->inv_sg, ish = qs->inv_sh;
  const double dtg = double(tg) * isg, dth = double(th) * ish;
  float approx[kBinsPerThread];
  float amax = -INFINITY, parent_term = 0.0f;
  auto counts_of = [&](long long lh, long long rc_k, unsigned long long &lc, unsigned long long &tc) {
    if (COUNTS) {  // true row counts (gain.cu:125-134 gates every candidate on them)
      lc = (unsigned long long)rc_k;
      tc = (unsigned long long)tcn;
    } else if (PAIR) {  // h_q >= 1 for every row, so a zero sum means "no rows"
      lc = lh > 0;
      tc = lc + ((th - lh) > 0);
    } else {  // h_q == 1 for every row: the sum is the row count
      lc = (unsigned long long)lh;
      tc = (unsigned long long)th;
    }
  };
  if (active && th != 0) {
    long long rg = og, rh = oh, rc = oc;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
      const int bin = bin0 + k;
      rg += v[k].x;
      rh += v[k].y;
      if (COUNTS) rc += cv[k];
      approx[k] = -INFINITY;
      if (bin >= hist_size) continue;  // ids >= hist_size hold missing values: never a threshold
      if ((k & (parts - 1)) != int(blockIdx.z)) continue;  // another CTA's candidate
      if (ncand > 0 && bin >= ncand) continue;  // the shared bin of the rare categories
      const long long lg = ncand > 0 ? v[k].x : rg, lh = ncand > 0 ? v[k].y : rh;
      unsigned long long lc, tc;
      counts_of(lh, ncand > 0 ? (COUNTS ? cv[k] : 0) : rc, lc, tc);
      approx[k] = split_gain_approx<PAIR>(float(double(lg) * isg), float(double(lh) * ish), float(dtg), float(dth),
                                          lc, tc, gp, &parent_term);
      amax = fmaxf(amax, approx[k]);
    }
  } else {
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) approx[k] = -INFINITY;
  }
  {  // the CTA's largest approximate value and the parent's term (equal for all features)
    __shared__ float warp_max[kSplitThreads / 32], warp_term[kSplitThreads / 32];
    float m = amax, t = parent_term;
    for (int o = 16; o > 0; o >>= 1) {
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    }
    if ((threadIdx.x & 31) == 0) {
      warp_max[threadIdx.x >> 5] = m;
      warp_term[threadIdx.x >> 5] = t;
    }
    __syncthreads();
    m = warp_max[threadIdx.x & 31];
    t = warp_term[threadIdx.x & 31];
    for (int o = 16; o > 0; o >>= 1) {
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    }
    amax = m;
    parent_term = t;
  }
  // The survivors are dealt out again, one to a thread: they sit in neighbouring bins, which
  // belong to the same few threads, and the exact arithmetic is a long dependent chain.
  long long *q_lg = part_g, *q_lh = part_h;  // the scan is done with them
  unsigned *q_lc = reinterpret_cast<unsigned *>(best_gain), *q_id = reinterpret_cast<unsigned *>(best_bin);
  auto exact = [&](long long lg, long long lh, unsigned lcount, int fid, int bin) {
    unsigned long long lc, tc;
    if (COUNTS) {
      lc = lcount;
      tc = (unsigned long long)s_tcn;
    } else if (PAIR) {
      lc = lh > 0;
      tc = lc + ((s_th - lh) > 0);
    } else {
      lc = (unsigned long long)lh;
      tc = (unsigned long long)s_th;
    }
    const float gain = split_gain<PAIR>(double(lg) * isg, double(lh) * ish, double(s_tg) * isg, double(s_th) * ish,
                                        lc, tc, gp);
    if (gain > 0.0f) atomicMax(&s_key, pack_key(gain, fid, bin));
  };
  if (active && th != 0 && amax > -INFINITY) {
    const float floor_value = amax - 1e-5f * (2.0f * fabsf(parent_term) + fabsf(amax)) - 1e-30f;
    long long rg = og, rh = oh, rc = oc;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
      const int bin = bin0 + k;
      rg += v[k].x;
      rh += v[k].y;
      if (COUNTS) rc += cv[k];
      if (!(approx[k] >= floor_value)) continue;
      const long long lg = ncand > 0 ? v[k].x : rg, lh = ncand > 0 ? v[k].y : rh;
      const unsigned lcount = COUNTS ? unsigned(ncand > 0 ? cv[k] : rc) : 0u;
      const unsigned at = atomicAdd(&q_count, 1u);
      if (at < unsigned(kSplitThreads)) {
        q_lg[at] = lg;
        q_lh[at] = lh;
        q_lc[at] = lcount;
        q_id[at] = (unsigned(f) << 12) | unsigned(bin);
      } else {  // more survivors than threads (many equal gains): valued where they are
        exact(lg, lh, lcount, f, bin);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < min(q_count, unsigned(kSplitThreads))) {
    const unsigned id = q_id[threadIdx.x];
    exact(q_lg[threadIdx.x], q_lh[threadIdx.x], q_lc[threadIdx.x], int(id >> 12), int(id & 0xfffu));
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_key != 0ull) atomicMax(&keys[node], s_key);
  // the last tile of the node to arrive turns the packed winner into the record
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&done[node], 1u) == unsigned(NT * parts - 1);
  __syncthreads();
  if (is_last && threadIdx.x < 32) {
    __threadfence();
    const unsigned long long key = atomicMax(&keys[node], 0ull);
    finalize_node(hist, COUNTS ? count_hist : nullptr, cat_candidates, key, rec, node, TW, NT, threadIdx.x);
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
  // (the exact arithmetic of the few candidates that survive the single-precision look is
  // spread over the threads of one CTA, so a tile is no longer dealt to several CTAs)
  (void)sms;
  const int parts = 1;
  const dim3 grid(a.L, a.geo.NT, parts);
  if (a.pair && a.count_hist)
    launch_overlapped(split_kernel<true, true>, grid, kSplitThreads, 0, s, a.hist, a.count_hist, a.feature_active,
                      a.cat_candidates, a.keys, done, a.rec, a.qs, a.gp, a.geo.TW, a.geo.NT, a.geo.F, a.geo.hist_size, parts);
  else if (a.pair)
    launch_overlapped(split_kernel<true, false>, grid, kSplitThreads, 0, s, a.hist, a.count_hist, a.feature_active,
                      a.cat_candidates, a.keys, done, a.rec, a.qs, a.gp, a.geo.TW, a.geo.NT, a.geo.F, a.geo.hist_size, parts);
  else
    launch_overlapped(split_kernel<false, false>, grid, kSplitThreads, 0, s, a.hist, a.count_hist, a.feature_active,
                      a.cat_candidates, a.keys, done, a.rec, a.qs, a.gp, a.geo.TW, a.geo.NT, a.geo.F, a.geo.hist_size, parts);
  count_launch();
}

}  // namespace arb
