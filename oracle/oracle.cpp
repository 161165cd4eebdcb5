// TEST INFRASTRUCTURE ONLY -- never linked into, imported by or called from the
// product library.  CPU restatement of the histogram ("method = hist") training
// path of sh1ng/arboretum, written from the reference's sources as a checker for
// the CUDA implementation.  Every function cites the reference file:line whose
// behaviour it restates.  Parity status: pinned against the reference's own
// known-answer tests (tests/cpp/test_datamatrix.cu, test_hist.cu,
// test_hist_sum.cu) and its iris golden models (tests/py/test_hist_logregression.py)
// for the quantizer, partition index, histogram, split search, leaf weights and
// prediction.  Parity UNPINNED (the reference has no behaviour to compare with)
// for: the missing-value bin, multi:softmax, pre-binned input.
//
// Build: see oracle/Makefile (g++ -O2 -fopenmp -shared).  C ABI at the bottom.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <random>
#include <string>
#include <map>
#include <vector>

namespace orc {

// ---------------------------------------------------------------------------
// small vector types (src/core/cuda_helpers.h:76-143: float2/double2 operators)
// ---------------------------------------------------------------------------
struct f2 {
  float x, y;
};
struct d2 {
  double x, y;
};
static inline f2 operator+(f2 a, f2 b) { return {a.x + b.x, a.y + b.y}; }
static inline f2 operator-(f2 a, f2 b) { return {a.x - b.x, a.y - b.y}; }
static inline d2 operator+(d2 a, d2 b) { return {a.x + b.x, a.y + b.y}; }
static inline d2 operator-(d2 a, d2 b) { return {a.x - b.x, a.y - b.y}; }
static inline d2 operator+(d2 a, f2 b) { return {a.x + b.x, a.y + b.y}; }
static inline void zero(float &v) { v = 0.0f; }
static inline void zero(double &v) { v = 0.0; }
static inline void zero(f2 &v) { v = {0.0f, 0.0f}; }
static inline void zero(d2 &v) { v = {0.0, 0.0}; }

// ---------------------------------------------------------------------------
// Gain and leaf weight (src/core/gain.cu, src/core/gain.cuh)
// ---------------------------------------------------------------------------
struct GainParams {  // gain.cuh:11-30 (GainFunctionParameters)
  unsigned min_leaf_size;
  float hess;  // = tree.min_child_weight (garden.cu:90-92)
  float gamma_absolute;
  float gamma_relative;
  float lambda;
  float alpha;
  float max_leaf_weight;
};

template <typename T>
static inline int sign(T val) {  // gain.cu:8-11
  return (T(0) < val) - (val < T(0));
}

// gain.cu:13-17.  The arithmetic types follow the reference's expression:
// `0.5` is a double literal, so the middle term and the sum are double.
template <typename T1, typename T2>
static inline float gain_term(T1 grad, T2 hess, float w, float lambda,
                              float alpha) {
  return -2 * (grad * (-w) + 0.5 * (hess + lambda) * w * w +
               alpha * std::fabs(w));
}

// gain.cu:19-23.  `max(0.0, x)` is evaluated in double and narrowed to T.
template <typename T>
static inline T grad_regularized(T grad, const float alpha) {
  const T grad_abs = std::fabs(grad);
  return T(sign(grad) * std::max(0.0, double(grad_abs - alpha)));
}

static inline float threshold_weight(float w, float mlw) {  // gain.cu:25-32
  if (mlw != 0.0f) {
    if (w > mlw) return mlw;
    if (w < -mlw) return -mlw;
  }
  return w;
}

// gain.cu:34-76: four overloads, selected by the sum type.
static inline float weight(float s, unsigned c, float mcw, unsigned mls,
                           float lambda, float alpha, float mlw) {
  float w = 0.0;
  if (c >= mls && c >= mcw) w = grad_regularized(s, alpha) / (c + lambda);
  return threshold_weight(w, mlw);
}
static inline float weight(double s, unsigned c, float mcw, unsigned mls,
                           float lambda, float alpha, float mlw) {
  float w = 0.0;
  if (c >= mls && c >= mcw) w = grad_regularized(s, alpha) / (c + lambda);
  return threshold_weight(w, mlw);
}
static inline float weight(f2 s, unsigned c, float mcw, unsigned mls,
                           float lambda, float alpha, float mlw) {
  float w = 0.0;
  if (c >= mls && s.y >= mcw) w = grad_regularized(s.x, alpha) / (s.y + lambda);
  return threshold_weight(w, mlw);
}
static inline float weight(d2 s, unsigned c, float mcw, unsigned mls,
                           float lambda, float alpha, float mlw) {
  float w = 0.0;
  if (c >= mls && s.y >= mcw) w = grad_regularized(s.x, alpha) / (s.y + lambda);
  return threshold_weight(w, mlw);
}
template <typename S>
static inline float weight(S s, unsigned c, const GainParams &p) {  // gain.cu:101-123
  return weight(s, c, p.hess, p.min_leaf_size, p.lambda, p.alpha,
                p.max_leaf_weight);
}

// gain.cu:125-238: gain of splitting `total` into `left` and the rest.
static inline float gain_func(d2 left, d2 total, size_t lc, size_t tc,
                              const GainParams &p) {
  const d2 right = total - left;
  const size_t rc = tc - lc;
  if (lc >= p.min_leaf_size && rc >= p.min_leaf_size &&
      std::fabs(left.y) >= p.hess && std::fabs(right.y) >= p.hess) {
    const float wl = weight(left, unsigned(lc), p);
    const float wr = weight(right, unsigned(rc), p);
    const float wp = weight(total, unsigned(tc), p);
    const float l = gain_term(left.x, left.y, wl, p.lambda, p.alpha);
    const float r = gain_term(right.x, right.y, wr, p.lambda, p.alpha);
    const float q = gain_term(total.x, total.y, wp, p.lambda, p.alpha);
    const float diff = l + r - q;
    return (diff > p.gamma_absolute && diff > p.gamma_relative * q) * diff;
  }
  return 0.0;
}
static inline float gain_func(f2 left, f2 total, size_t lc, size_t tc,
                              const GainParams &p) {
  const f2 right = total - left;
  const size_t rc = tc - lc;
  if (lc >= p.min_leaf_size && rc >= p.min_leaf_size &&
      std::fabs(left.y) >= p.hess && std::fabs(right.y) >= p.hess) {
    const float wl = weight(left, unsigned(lc), p);
    const float wr = weight(right, unsigned(rc), p);
    const float wp = weight(total, unsigned(tc), p);
    const float l = gain_term(left.x, left.y, wl, p.lambda, p.alpha);
    const float r = gain_term(right.x, right.y, wr, p.lambda, p.alpha);
    const float q = gain_term(total.x, total.y, wp, p.lambda, p.alpha);
    const float diff = l + r - q;
    return (diff > p.gamma_absolute && diff > p.gamma_relative * q) * diff;
  }
  return 0.0;
}
static inline float gain_func(float left, float total, size_t lc, size_t tc,
                              const GainParams &p) {
  const size_t rc = tc - lc;
  const float right = total - left;
  if (lc >= p.min_leaf_size && rc >= p.min_leaf_size) {
    const float wl = weight(left, unsigned(lc), p);
    const float wr = weight(right, unsigned(rc), p);
    const float wp = weight(total, unsigned(tc), p);
    const float l = gain_term(left, lc, wl, p.lambda, p.alpha);
    const float r = gain_term(right, rc, wr, p.lambda, p.alpha);
    const float q = gain_term(total, tc, wp, p.lambda, p.alpha);
    const float diff = l + r - q;
    return (diff > p.gamma_absolute && diff > p.gamma_relative * q) * diff;
  }
  return 0.0;
}
static inline float gain_func(double left, double total, size_t lc, size_t tc,
                              const GainParams &p) {
  const size_t rc = tc - lc;
  const double right = total - left;
  if (lc >= p.min_leaf_size && rc >= p.min_leaf_size) {
    const float wl = weight(left, unsigned(lc), p);
    const float wr = weight(right, unsigned(rc), p);
    const float wp = weight(total, unsigned(tc), p);
    const float l = gain_term(left, lc, wl, p.lambda, p.alpha);
    const float r = gain_term(right, rc, wr, p.lambda, p.alpha);
    const float q = gain_term(total, tc, wp, p.lambda, p.alpha);
    const float diff = l + r - q;
    return (diff > p.gamma_absolute && diff > p.gamma_relative * q) * diff;
  }
  return 0.0;
}

// ---------------------------------------------------------------------------
// Quantizer (src/io/io.cu:349-435, :72-79, :144-153, :255-271, :293-312;
// src/core/cuda_helpers.h:207-222)
// ---------------------------------------------------------------------------
// Radix order of fp32 keys as cub::DeviceRadixSort sorts them (io.cu:382-385):
// sign-magnitude order, -0.0 before +0.0, positive NaNs last.
static inline uint32_t radix_key(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// thr: hist_size floats out (data_reduced_mapping[f], io.cu:398-401).
// returns `size` = min(unique, hist_size) (io.cu:403-410).
static int find_thresholds(const float *col, int64_t n, int hist_size,
                           float *thr) {
  std::vector<float> s(col, col + n);
  std::sort(s.begin(), s.end(),
            [](float a, float b) { return radix_key(a) < radix_key(b); });
  const int64_t seg = std::max<int64_t>(1, n / hist_size);  // io.cu:376-377
  for (int i = 0; i < hist_size; ++i) thr[i] = INFINITY;    // io.cu:387
  uint32_t c = 0;
  for (int64_t i = 1; i < n; ++i) {
    if (s[i] != s[i - 1]) {  // border, io.cu:72-79
      ++c;                   // inclusive border count, io.cu:144-153
      const float mid = (s[i] + s[i - 1]) * 0.5;
      const int k = int(std::min<uint32_t>(c + 1, uint32_t(i / seg + 1))) - 2;  // io.cu:257
      // The reference writes thr[k] without a bound; k >= hist_size is a
      // reference defect that the named shapes never reach: refuse it here.
      if (k >= 0 && k < hist_size && mid < thr[k]) thr[k] = mid;  // io.cu:258-269
    }
  }
  int unique = 0;
  while (unique < hist_size && !std::isinf(thr[unique])) ++unique;  // io.cu:403-407
  ++unique;
  return std::min(unique, hist_size);
}

// lower_bound over v[0..size-2]=thr, v[size-1]=+INF (io.cu:297-310,
// cuda_helpers.h:207-222): number of thresholds strictly below x.  NaN compares
// false everywhere and therefore lands on `size` in the reference; with
// `missing_bin` set NaN goes to the dedicated id `hist_size` instead.
static inline unsigned bin_of(const float *thr, int size, float x, int hist_size,
                              bool missing_bin) {
  if (missing_bin && std::isnan(x)) return unsigned(hist_size);
  unsigned l = 0, h = unsigned(size);
  while (l < h) {
    const unsigned mid = (l + h) / 2;
    const float v = (int(mid) < size - 1) ? thr[mid] : INFINITY;
    if (x <= v)
      h = mid;
    else
      l = mid + 1;
  }
  return l;
}

// ---------------------------------------------------------------------------
// Partition index (src/core/partition.cuh:20-34,:76-86; builder.h:287-300):
// inside each parent segment lefts keep their order from the segment start,
// rights are laid out from the segment end in reversed order.
// seg_begin has nseg+1 entries; go_right[i] is the decision of position i.
// ---------------------------------------------------------------------------
static void partition_index(const uint8_t *go_right, const uint32_t *seg_begin,
                            int nseg, uint32_t *index) {
  for (int s = 0; s < nseg; ++s) {
    uint32_t nl = 0;
    for (uint32_t i = seg_begin[s]; i < seg_begin[s + 1]; ++i) {
      if (!go_right[i]) {
        ++nl;
        index[i] = seg_begin[s] + nl - 1;
      } else {
        index[i] = seg_begin[s + 1] - (i - seg_begin[s] - nl + 1);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Configuration (src/core/param.h:20-60, json_conversion.h:108-112)
// ---------------------------------------------------------------------------
struct Config {
  int objective;  // 0 reg:linear, 1 reg:logistic, 3 multi:softmax (extension)
  int depth;      // max_depth + 1
  float min_child_weight;
  unsigned min_leaf_size;
  float colsample_bytree, colsample_bylevel;
  float gamma_absolute, gamma_relative, lambda, alpha;
  float initial_y, eta, max_leaf_weight;
  int labels_count;
  int double_precision;
  unsigned seed;
  int use_trick;
  int hist_size;
  int missing_bin;  // extension: NaN -> dedicated bin id hist_size
};

struct Node {
  int fid;
  unsigned quantized;
  float threshold;
  // extension (the reference's categorical training is a stub, hist_tree_grower.h:55-63):
  // the node sends `value == category` left, like RegTree::Predict garden.h:79-84
  bool categorical = false;
  unsigned category = unsigned(-1);
};
struct Tree {  // reg_tree.h:16-45, garden.h:32-68
  int depth;
  int label;
  std::vector<Node> nodes;     // heap order, (1<<depth)-1
  std::vector<float> weights;  // 1<<(depth-1)
};

struct LevelStat {  // what the parity tests compare level by level
  std::vector<uint32_t> node_begin;  // prefix counts, L+1
  std::vector<float> gain;           // per node best gain
  std::vector<float> gain2;          // per node runner-up gain over (feature)
  std::vector<int> fid;
  std::vector<int> bin;
  std::vector<double> left_g, left_h, tot_g, tot_h;
  std::vector<double> abs_g;  // sum |g| over the node's rows: scale of the tolerance
  std::vector<uint32_t> left_count;
};

static inline double gx(float v) { return v; }
static inline double gx(double v) { return v; }
static inline double gx(f2 v) { return v.x; }
static inline double gx(d2 v) { return v.x; }
static inline double gy(float) { return 0; }
static inline double gy(double) { return 0; }
static inline double gy(f2 v) { return v.y; }
static inline double gy(d2 v) { return v.y; }
static inline void acc(float &s, float g) { s += g; }
static inline void acc(double &s, float g) { s += g; }
static inline void acc(f2 &s, f2 g) { s = s + g; }
static inline void acc(d2 &s, f2 g) { s = s + g; }

static inline float sigmoid(float x) {  // objective.h:66-68
  return 1.0 / (1.0 + std::exp(-x));
}

class TrainerBase {
 public:
  virtual ~TrainerBase() {}
  virtual void grow_round() = 0;
  virtual void get_yhat(float *out) const = 0;  // original row order, internal scale
  std::vector<Tree> trees;
  std::vector<std::vector<LevelStat>> stats;  // per tree, per level
  // dense histogram of the last processed (tree, level, feature) pairs, kept
  // only when `keep_hist` is set: [level][feature] -> L*HW (g,h,count)
  int keep_hist = 0;
  std::vector<std::vector<std::vector<double>>> hist_g, hist_h;
  std::vector<std::vector<std::vector<uint32_t>>> hist_c;
  // categorical features (extension): ids n_dense .. F - 1; bin id = rank of the category
  // by frequency; cat_candidates[f] = bins a one-vs-rest split may name (0 for dense
  // features); cat_codes[f - n_dense][bin] = category code
  int n_dense = 1 << 30;
  std::vector<int> cat_candidates;
  std::vector<std::vector<uint32_t>> cat_codes;
};

// One boosting state bound to one data set; mirrors ContinuousGardenBuilder
// (garden.cu:78-504) + HistTreeGrower (hist_tree_grower.cu) with all per-row
// arrays kept in the reference's physical (partitioned) order.
template <typename G, typename S>
class Trainer : public TrainerBase {
 public:
  Config cfg;
  GainParams gp;
  int64_t n;
  int F, H, HW;
  std::vector<std::vector<uint16_t>> bins;  // [f][position]
  std::vector<std::vector<float>> mapping;  // [f][H] thresholds
  std::vector<int> fsize;                   // bins used per feature
  std::vector<float> y;                     // position order
  std::vector<uint8_t> label;               // position order (softmax)
  std::vector<float> yhat;                  // [k][position]
  std::vector<G> grad;                      // [k][position]
  std::vector<uint32_t> orig;               // position -> original row
  std::vector<uint8_t> go_right;            // decision of the previous level
  std::default_random_engine rnd;           // garden.cu:87
  std::vector<unsigned> active;
  // BestSplit (best_splits.h:14-38)
  std::vector<uint32_t> pcount, pcount_next;
  std::vector<S> psum, psum_next;
  // Histogram<SUM_T> (histogram.cu)
  std::vector<std::vector<S>> saved_sum;
  std::vector<std::vector<uint32_t>> saved_count;
  std::vector<int> at_level;

  Trainer(const Config &c, int64_t n_, int F_, const uint16_t *bins_fm,
          const float *mapping_, const int *fsize_, const float *y_,
          const uint8_t *label_)
      : cfg(c), n(n_), F(F_), H(c.hist_size), rnd(c.seed) {
    HW = H + (cfg.missing_bin ? 1 : 0);
    gp = {cfg.min_leaf_size, cfg.min_child_weight, cfg.gamma_absolute,
          cfg.gamma_relative, cfg.lambda,          cfg.alpha,
          cfg.max_leaf_weight};
    bins.resize(F);
    mapping.resize(F);
    fsize.assign(fsize_, fsize_ + F);
    for (int f = 0; f < F; ++f) {
      bins[f].assign(bins_fm + size_t(f) * n, bins_fm + size_t(f + 1) * n);
      mapping[f].assign(mapping_ + size_t(f) * H, mapping_ + size_t(f + 1) * H);
    }
    if (y_) y.assign(y_, y_ + n);
    if (label_) label.assign(label_, label_ + n);
    const int K = cfg.labels_count;
    // garden.cu:105: y_hat starts at IntoInternal(initial_y) (objective.h:55-57)
    float init = cfg.initial_y;
    if (cfg.objective == 1) init = std::log(init / (1 - init));
    yhat.assign(size_t(K) * n, init);
    grad.resize(size_t(K) * n);
    orig.resize(n);
    for (int64_t i = 0; i < n; ++i) orig[i] = uint32_t(i);
    go_right.assign(n, 0);
    active.resize(F);
    const int maxn = 1 << cfg.depth;
    pcount.assign(maxn + 1, 0);
    pcount_next.assign(maxn + 1, 0);
    psum.resize(maxn + 1);
    psum_next.resize(maxn + 1);
    for (auto &v : psum) zero(v);
    for (auto &v : psum_next) zero(v);
    saved_sum.resize(F);
    saved_count.resize(F);
    at_level.assign(F, -1);
  }

  void update_grad() {  // objective.cu:28-56; softmax: objective.cu:60-89 (intent)
    const int K = cfg.labels_count;
    if (cfg.objective == 3) {
      for (int64_t i = 0; i < n; ++i) {
        std::vector<double> p(K);
        double sum = 0;
        for (int k = 0; k < K; ++k) {
          p[k] = std::exp(double(yhat[size_t(k) * n + i]));
          sum += p[k];
        }
        for (int k = 0; k < K; ++k) {
          const double pred = p[k] / sum;
          set_grad(grad[size_t(k) * n + i],
                   float((k == label[i] ? 1.0 : 0.0) - pred),
                   float(2.0 * pred * (1.0 - pred)));
        }
      }
      return;
    }
    for (int64_t i = 0; i < n; ++i) {
      if (cfg.objective == 0) {
        set_grad(grad[i], y[i] - yhat[i], 1.0f);
      } else {
        const float s = sigmoid(yhat[i]);
        set_grad(grad[i], y[i] - s, s * (1.0f - s));
      }
    }
  }
  static void set_grad(float &g, float a, float) { g = a; }
  static void set_grad(f2 &g, float a, float b) { g = {a, b}; }

  void grow_round() override {  // Garden::GrowTree garden.cu:585-625
    update_grad();
    for (int k = 0; k < cfg.labels_count; ++k) grow_tree(k);
  }

  template <typename T>
  void scatter(std::vector<T> &v, size_t off, const std::vector<uint32_t> &idx) {
    std::vector<T> tmp(n);
    for (int64_t i = 0; i < n; ++i) tmp[idx[i]] = v[off + i];
    std::copy(tmp.begin(), tmp.end(), v.begin() + off);
  }

  void grow_tree(int k) {  // ContinuousGardenBuilder::GrowTree garden.cu:167-197
    const int depth = cfg.depth;
    Tree tree;
    tree.depth = depth;
    tree.label = k;
    tree.nodes.assign((1 << depth) - 1, Node{0, 0, 0.f, false, unsigned(-1)});
    tree.weights.assign(1 << (depth - 1), 0.f);
    std::vector<LevelStat> tstats;
    G *g = grad.data() + size_t(k) * n;

    // InitGrowingTree garden.cu:126-160
    int take = int(cfg.colsample_bytree * F);
    if (take == 0) throw std::string("colsample_bytree is too small");
    take = int(cfg.colsample_bytree * cfg.colsample_bylevel * F);
    if (take == 0)
      throw std::string("colsample_bytree and colsample_bylevel are too small");
    for (int i = 0; i < F; ++i) active[i] = i;
    std::shuffle(active.begin(), active.end(), rnd);
    std::fill(at_level.begin(), at_level.end(), -1);  // Histogram::Clear
    std::fill(go_right.begin(), go_right.end(), 0);

    std::vector<int> best_fid;
    std::vector<float> best_gain;
    std::vector<S> best_sum;
    std::vector<uint32_t> best_count;
    std::vector<unsigned> best_split;

    if (keep_hist) {
      hist_g.assign(depth - 1, std::vector<std::vector<double>>(F));
      hist_h.assign(depth - 1, std::vector<std::vector<double>>(F));
      hist_c.assign(depth - 1, std::vector<std::vector<uint32_t>>(F));
    }

    for (int level = 0; level + 1 < depth; ++level) {
      const int L = 1 << level;
      // InitTreeLevel garden.cu:162-165
      std::shuffle(active.begin(),
                   active.begin() + int(cfg.colsample_bytree * F), rnd);
      // UpdateNodeStat garden.cu:419-445 + BestSplit::Clear best_splits.cu:37-46
      best_fid.assign(L, -1);
      best_gain.assign(L, 0.f);
      best_count.assign(L, 0);
      best_split.assign(L, unsigned(-1));
      best_sum.resize(L);
      for (auto &v : best_sum) zero(v);
      if (level == 0) {
        pcount[0] = 0;
        pcount[1] = uint32_t(n);
        zero(psum[0]);
        S tot;
        zero(tot);
        for (int64_t i = 0; i < n; ++i) acc(tot, g[i]);
        psum[1] = tot;
      }
      // FindBestSplits garden.cu:249-347
      const unsigned takel =
        unsigned(cfg.colsample_bylevel * cfg.colsample_bytree * F);
      if (level != 0) {
        // BestSplit::NextLevel best_splits.cu:66-81
        for (int i = 1; i <= L; ++i) {
          pcount[i] = pcount_next[i];
          psum[i] = psum_next[i];
        }
        // parents are the nodes of level-1: segments pcount[0,2,4,...]
        std::vector<uint32_t> parent_begin(L / 2 + 1);
        for (int p = 0; p <= L / 2; ++p) parent_begin[p] = pcount[2 * p];
        std::vector<uint32_t> idx(n);
        partition_index(go_right.data(), parent_begin.data(), L / 2, idx.data());
        // garden.cu:271-293: every per-row array moves, for every class plane
        for (int kk = 0; kk < cfg.labels_count; ++kk) {
          scatter(grad, size_t(kk) * n, idx);
          scatter(yhat, size_t(kk) * n, idx);
        }
        if (!y.empty()) scatter(y, 0, idx);
        if (!label.empty()) scatter(label, 0, idx);
        scatter(orig, 0, idx);
#pragma omp parallel for
        for (int f = 0; f < F; ++f) scatter(bins[f], 0, idx);  // hist_tree_grower.cu:346-348
        std::fill(go_right.begin(), go_right.end(), 0);
      }
      LevelStat st;
      st.node_begin.assign(pcount.begin(), pcount.begin() + L + 1);
      std::vector<float> top1(L, 0.f), top2(L, 0.f);

      // Per-feature work (histogram, scans, gain search) is independent until the
      // candidates are folded into the per-node best, so it runs on all host
      // threads; the fold below stays in the reference's feature order.
      struct Cand {
        std::vector<float> cgain, t1, t2;
        std::vector<unsigned> cidx;
        std::vector<S> sum_at;
        std::vector<uint32_t> cnt_at;
      };
      std::vector<Cand> cands(F);
#pragma omp parallel for schedule(dynamic)
      for (int j = 0; j < F; ++j) {
        const int fid = int(active[j]);
        if (unsigned(j) >= takel) continue;  // partition_only features
        std::vector<S> sum(size_t(L) * HW), prefix(size_t(L) * HW);
        std::vector<uint32_t> cnt(size_t(L) * HW), cprefix(size_t(L) * HW);
        // ---- histogram (hist_tree_grower.cu:365-390) -----------------------
        for (auto &v : sum) zero(v);
        std::fill(cnt.begin(), cnt.end(), 0);
        const bool trick = cfg.use_trick && level != 0 &&
                           at_level[fid] + 1 == level;  // histogram.cu:46-50
        auto scan_node = [&](int node) {
          for (uint32_t i = pcount[node]; i < pcount[node + 1]; ++i) {
            const unsigned b = bins[fid][i];
            if (b >= unsigned(HW)) continue;  // reference would write out of range
            acc(sum[size_t(node) * HW + b], g[i]);
            cnt[size_t(node) * HW + b]++;
          }
        };
        if (trick) {
          for (int p = 0; p < L / 2; ++p) {
            const int lnode = 2 * p, rnode = 2 * p + 1;
            const uint32_t ls = pcount[lnode + 1] - pcount[lnode];
            const uint32_t rs = pcount[rnode + 1] - pcount[rnode];
            // hist_grad_sum.cu:288-290 / :23: ties build the left child
            const int src = ls <= rs ? lnode : rnode;
            const int dst = src == lnode ? rnode : lnode;
            scan_node(src);
            for (int b = 0; b < HW; ++b) {  // update_multi_node hist_grad_sum.cu:6-33
              sum[size_t(dst) * HW + b] =
                saved_sum[fid][size_t(p) * HW + b] - sum[size_t(src) * HW + b];
              cnt[size_t(dst) * HW + b] =
                saved_count[fid][size_t(p) * HW + b] - cnt[size_t(src) * HW + b];
            }
          }
        } else {
          for (int node = 0; node < L; ++node) scan_node(node);
        }
        if (keep_hist) {
          auto &hg = hist_g[level][fid];
          auto &hh = hist_h[level][fid];
          auto &hc = hist_c[level][fid];
          hg.resize(size_t(L) * HW);
          hh.resize(size_t(L) * HW);
          hc.resize(size_t(L) * HW);
          for (size_t i = 0; i < size_t(L) * HW; ++i) {
            hg[i] = gx(sum[i]);
            hh[i] = gy(sum[i]);
            hc[i] = cnt[i];
          }
        }
        // ---- un-segmented inclusive scans (hist_tree_grower.cu:393-403) ----
        {
          S run;
          zero(run);
          uint32_t crun = 0;
          for (size_t i = 0; i < size_t(L) * HW; ++i) {
            run = run + sum[i];
            crun += cnt[i];
            prefix[i] = run;
            cprefix[i] = crun;
          }
        }
        // ---- hist_gain_kernel hist_tree_grower.cu:9-35 ----------------------
        Cand &cd = cands[j];
        cd.cgain.assign(L, 0.f);
        cd.cidx.assign(L, 0);
        cd.t1.assign(L, 0.f);
        cd.t2.assign(L, 0.f);
        std::vector<float> &cgain = cd.cgain, &top1l = cd.t1, &top2l = cd.t2;
        std::vector<unsigned> &cidx = cd.cidx;
        const int ncand = fid >= n_dense ? cat_candidates[fid] : 0;
        for (size_t i = 0; i < size_t(L) * HW; ++i) {
          const unsigned seg = unsigned(i / HW);
          // categorical feature (extension, builder.h:75-105): one bin against the rest; the
          // bin shared by the rare categories is no candidate
          if (fid >= n_dense && int(i % HW) >= ncand) continue;
          const S lsum = fid >= n_dense ? sum[i] : prefix[i] - psum[seg];
          const uint32_t lcnt = fid >= n_dense ? cnt[i] : cprefix[i] - pcount[seg];
          const S tsum = psum[seg + 1] - psum[seg];
          const uint32_t tcnt = pcount[seg + 1] - pcount[seg];
          const float gn = gain_func(lsum, tsum, lcnt, tcnt, gp);
          if (gn > 0.0) {  // updateAtomicMax builder.h:39-49: ties -> higher index
            if (gn > top1l[seg]) {  // bookkeeping for the tests only
              top2l[seg] = top1l[seg];
              top1l[seg] = gn;
            } else if (gn < top1l[seg] && gn > top2l[seg]) {
              top2l[seg] = gn;
            }
            if (cgain[seg] < gn || (cgain[seg] == gn && cidx[seg] < unsigned(i))) {
              cgain[seg] = gn;
              cidx[seg] = unsigned(i);
            }
          }
        }
        cd.sum_at.resize(L);
        cd.cnt_at.resize(L);
        for (int node = 0; node < L; ++node) {
          if (fid >= n_dense) {  // as if the winner's rows lay first in the node
            cd.sum_at[node] = psum[node] + sum[cidx[node]];
            cd.cnt_at[node] = pcount[node] + cnt[cidx[node]];
          } else {
            cd.sum_at[node] = prefix[cidx[node]];
            cd.cnt_at[node] = cprefix[cidx[node]];
          }
        }
        if (cfg.use_trick) {  // Histogram::Update histogram.cu:30-44
          saved_sum[fid] = sum;
          saved_count[fid] = cnt;
          at_level[fid] = level;
        }
      }
      for (int j = 0; j < F; ++j) {
        const int fid = int(active[j]);
        if (unsigned(j) >= takel) continue;
        const Cand &cd = cands[j];
        const std::vector<float> &cgain = cd.cgain;
        const std::vector<unsigned> &cidx = cd.cidx;
        for (int node = 0; node < L; ++node) {  // merge the test bookkeeping
          for (float gn : {cd.t1[node], cd.t2[node]}) {
            if (gn > top1[node]) {
              top2[node] = top1[node];
              top1[node] = gn;
            } else if (gn < top1[node] && gn > top2[node]) {
              top2[node] = gn;
            }
          }
        }
        // ---- hist_apply_candidates hist_tree_grower.cu:37-102 ---------------
        for (int node = 0; node < L; ++node) {
          const uint32_t nstart = pcount[node], nend = pcount[node + 1];
          const uint32_t nsize = nend - nstart;
          const float gn = cgain[node];
          const unsigned idx = cidx[node];
          if (nsize > 0) {
            if (best_gain[node] < gn ||
                (best_gain[node] == gn && fid < best_fid[node])) {
              best_gain[node] = gn;
              best_fid[node] = fid;
              best_sum[node] = cd.sum_at[node] - psum[node];
              best_count[node] = cd.cnt_at[node] - nstart;
              const unsigned thr = idx % HW;
              best_split[node] = thr;
              // apply_split builder.h:107-123: right <=> bin >= thr + 1
              for (uint32_t i = nstart; i < nend; ++i)
                go_right[i] = fid >= n_dense ? bins[fid][i] != thr : bins[fid][i] >= thr + 1;
              pcount_next[2 * node + 1] = cd.cnt_at[node];
              pcount_next[2 * node + 2] = nend;
              psum_next[2 * node + 1] = cd.sum_at[node];
              psum_next[2 * node + 2] = psum[node + 1];
            } else if (best_gain[node] == 0 && best_fid[node] == -1) {
              best_sum[node] = psum[node + 1] - psum[node];
              best_split[node] = unsigned(-1);
              best_count[node] = nsize;
              pcount_next[2 * node + 1] = pcount_next[2 * node + 2] = nend;
              psum_next[2 * node + 1] = psum_next[2 * node + 2] = psum[node + 1];
            }
          } else {
            pcount_next[2 * node + 1] = pcount_next[2 * node + 2] = nend;
            psum_next[2 * node + 1] = psum_next[2 * node + 2] = psum[node + 1];
          }
        }
      }
      // ---- UpdateTree garden.cu:447-485 --------------------------------------
      const int offset = (1 << level) - 1;
      st.gain = best_gain;
      st.gain2 = top2;  // largest candidate gain strictly below the winner's
      st.fid.resize(L);
      st.bin.resize(L);
      st.left_g.resize(L);
      st.left_h.resize(L);
      st.tot_g.resize(L);
      st.tot_h.resize(L);
      st.left_count.resize(L);
      for (int i = 0; i < L; ++i) {
        Node &nd = tree.nodes[i + offset];
        const unsigned q = best_split[i];
        if (best_fid[i] != -1) {
          nd.fid = best_fid[i];
          nd.quantized = q;
          // split.cu / garden.cu:463-467.  Extension: a split on the last real
          // bin separates "present" from "missing": its float threshold is +INF.
          const bool last_real = cfg.missing_bin && int(q) >= fsize[best_fid[i]] - 1;
          nd.threshold = (q >= unsigned(H) || last_real)
                           ? INFINITY
                           : mapping[best_fid[i]][q];
          if (best_fid[i] >= n_dense) {
            nd.categorical = true;
            nd.category = cat_codes[best_fid[i] - n_dense][q];
            nd.threshold = INFINITY;
          }
        } else {
          nd.fid = 0;
          nd.quantized = q;
          nd.threshold = INFINITY;
          best_count[i] = pcount[i + 1] - pcount[i];
          best_sum[i] = psum[i + 1] - psum[i];
        }
        st.fid[i] = best_fid[i];
        st.bin[i] = int(q);
        st.left_g[i] = gx(best_sum[i]);
        st.left_h[i] = gy(best_sum[i]);
        const S tot = psum[i + 1] - psum[i];
        st.tot_g[i] = gx(tot);
        st.tot_h[i] = gy(tot);
        double ag = 0;
        for (uint32_t p = pcount[i]; p < pcount[i + 1]; ++p) ag += std::fabs(gx(g[p]));
        st.abs_g.push_back(ag);
        st.left_count[i] = best_count[i];
      }
      tstats.push_back(st);
    }
    // ---- UpdateLeafWeight garden.cu:487-503 ----------------------------------
    {
      const int last = depth - 2;
      const int Ll = 1 << last;
      for (int i = 0; i < Ll; ++i) {
        const S tot = psum[i + 1] - psum[i];
        const uint32_t tc = pcount[i + 1] - pcount[i];
        tree.weights[2 * i] = leaf_weight(best_sum[i], best_count[i]) * cfg.eta;
        tree.weights[2 * i + 1] =
          leaf_weight(tot - best_sum[i], tc - best_count[i]) * cfg.eta;
      }
      // ---- update_by_last_tree garden.cu:45-76 -------------------------------
      float *yh = yhat.data() + size_t(k) * n;
      for (int i = 0; i < Ll; ++i)
        for (uint32_t p = pcount[i]; p < pcount[i + 1]; ++p)
          yh[p] += go_right[p] ? tree.weights[2 * i + 1] : tree.weights[2 * i];
    }
    trees.push_back(tree);
    stats.push_back(tstats);
  }

  float leaf_weight(S s, uint32_t c) const {  // gain.cu:78-99 (TreeParam overloads)
    return weight(s, c, cfg.min_child_weight, cfg.min_leaf_size, cfg.lambda,
                  cfg.alpha, cfg.max_leaf_weight);
  }

  void get_yhat(float *out) const override {
    for (int k = 0; k < cfg.labels_count; ++k)
      for (int64_t i = 0; i < n; ++i)
        out[size_t(k) * n + orig[i]] = yhat[size_t(k) * n + i];
  }
};

// RegTree::Predict garden.h:70-90: out[row] += leaf weight; features >= F test the
// categorical column fid - F of `cat` (row-major [n][C]) for equality
static void tree_predict(const Tree &t, const float *X, int64_t n, int F,
                         float *out, const uint32_t *cat = nullptr, int C = 0) {
  const int offset = (1 << (t.depth - 1)) - 1;
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) {
    unsigned node = 0;
    for (int j = 1; j < t.depth; ++j) {
      const Node &nd = t.nodes[node];
      const bool left = nd.fid < F ? X[size_t(i) * F + nd.fid] < nd.threshold
                                   : (cat && cat[size_t(i) * C + (nd.fid - F)] == nd.category);
      node = left ? 2 * node + 1 : 2 * node + 2;
    }
    out[i] += t.weights[node - offset];
  }
}

struct Handle {
  Config cfg;
  int64_t n = 0;
  int F = 0;
  std::vector<float> X;  // row-major copy (prediction)
  std::vector<uint16_t> bins;
  std::vector<float> mapping;
  std::vector<int> fsize;
  std::vector<float> y;
  std::vector<uint8_t> label;
  // categorical columns (extension): codes row-major [n][C], set before the dense matrix
  int C = 0;
  std::vector<uint32_t> cat;
  std::vector<int> cat_candidates;
  std::vector<std::vector<uint32_t>> cat_codes;
  TrainerBase *trainer = nullptr;
  std::string error;
  ~Handle() { delete trainer; }
};

}  // namespace orc

// ===========================================================================
// C ABI (ctypes-friendly)
// ===========================================================================
using namespace orc;

extern "C" {

float orc_gain_f(float l, float t, uint64_t lc, uint64_t tc, const GainParams *p) {
  return gain_func(l, t, size_t(lc), size_t(tc), *p);
}
float orc_gain_d(double l, double t, uint64_t lc, uint64_t tc, const GainParams *p) {
  return gain_func(l, t, size_t(lc), size_t(tc), *p);
}
float orc_gain_f2(float lx, float ly, float tx, float ty, uint64_t lc, uint64_t tc,
                  const GainParams *p) {
  return gain_func(f2{lx, ly}, f2{tx, ty}, size_t(lc), size_t(tc), *p);
}
float orc_gain_d2(double lx, double ly, double tx, double ty, uint64_t lc,
                  uint64_t tc, const GainParams *p) {
  return gain_func(d2{lx, ly}, d2{tx, ty}, size_t(lc), size_t(tc), *p);
}
float orc_weight_f(float s, unsigned c, const GainParams *p) { return weight(s, c, *p); }
float orc_weight_d(double s, unsigned c, const GainParams *p) { return weight(s, c, *p); }
float orc_weight_f2(float x, float y, unsigned c, const GainParams *p) {
  return weight(f2{x, y}, c, *p);
}
float orc_weight_d2(double x, double y, unsigned c, const GainParams *p) {
  return weight(d2{x, y}, c, *p);
}

// one column: thresholds (hist_size floats), returns size; bins (uint16) out
int orc_quantize_column(const float *col, int64_t n, int hist_size, int missing_bin,
                        float *thr, uint16_t *bins) {
  const int size = find_thresholds(col, n, hist_size, thr);
  if (bins)
    for (int64_t i = 0; i < n; ++i)
      bins[i] = uint16_t(bin_of(thr, size, col[i], hist_size, missing_bin != 0));
  return size;
}

void orc_partition_index(const uint8_t *go_right, const uint32_t *seg_begin, int nseg,
                         uint32_t *index) {
  partition_index(go_right, seg_begin, nseg, index);
}

// naive per-node histogram of one feature (hist_grad_sum.cu:545-564 semantics)
void orc_hist(const uint16_t *bin, const float *g, const float *h, const uint32_t *seg_begin,
              int nseg, int hw, double *out_g, double *out_h, uint32_t *out_c) {
  for (int s = 0; s < nseg; ++s)
    for (uint32_t i = seg_begin[s]; i < seg_begin[s + 1]; ++i) {
      const size_t k = size_t(s) * hw + bin[i];
      out_g[k] += g[i];
      if (h) out_h[k] += h[i];
      out_c[k]++;
    }
}

void *orc_create(const Config *cfg) {
  Handle *h = new Handle();
  h->cfg = *cfg;
  return h;
}
void orc_free(void *p) { delete static_cast<Handle *>(p); }
const char *orc_error(void *p) { return static_cast<Handle *>(p)->error.c_str(); }

// Categorical columns (extension), to be given BEFORE orc_set_dense: uint32 codes,
// row-major [n][C].  orc_set_dense then appends them as features F .. F + C - 1.
// Bins: a category's bin is its rank by frequency (most frequent first, ties: smaller code
// first); a column with more than hist_size categories keeps the hist_size - 1 most frequent
// ones and gives all others bin hist_size - 1, which no split may name.
int orc_set_categories(void *p, const uint32_t *cat, int64_t n, int C) {
  Handle *h = static_cast<Handle *>(p);
  h->C = C;
  h->cat.assign(cat, cat + size_t(n) * C);
  return 0;
}
static void bin_categories(Handle *h) {
  const int64_t n = h->n;
  const int Fd = h->F, C = h->C, H = h->cfg.hist_size;
  h->bins.resize(size_t(n) * (Fd + C));
  h->mapping.resize(size_t(Fd + C) * H, INFINITY);
  h->fsize.resize(Fd + C);
  h->cat_candidates.assign(Fd + C, 0);
  h->cat_codes.assign(C, std::vector<uint32_t>());
  for (int c = 0; c < C; ++c) {
    std::map<uint32_t, uint64_t> count;
    for (int64_t i = 0; i < n; ++i) count[h->cat[size_t(i) * C + c]]++;
    std::vector<std::pair<uint32_t, uint64_t>> freq(count.begin(), count.end());  // codes ascending
    std::stable_sort(freq.begin(), freq.end(),
                     [](const std::pair<uint32_t, uint64_t> &a, const std::pair<uint32_t, uint64_t> &b) {
                       return a.second > b.second;
                     });
    const bool overflow = freq.size() > size_t(H);
    const size_t kept = overflow ? size_t(H - 1) : freq.size();
    std::map<uint32_t, uint16_t> bin_of_code;
    for (size_t b = 0; b < kept; ++b) {
      h->cat_codes[c].push_back(freq[b].first);
      bin_of_code[freq[b].first] = uint16_t(b);
    }
    h->fsize[Fd + c] = int(kept + (overflow ? 1 : 0));
    h->cat_candidates[Fd + c] = int(kept);
    for (int64_t i = 0; i < n; ++i) {
      auto it = bin_of_code.find(h->cat[size_t(i) * C + c]);
      h->bins[size_t(Fd + c) * n + i] = it == bin_of_code.end() ? uint16_t(kept) : it->second;
    }
  }
}
// dense fp32 row-major input; quantised here (DataMatrix::InitHist io.cu:342-347)
int orc_set_dense(void *p, const float *X, int64_t n, int F) {
  Handle *h = static_cast<Handle *>(p);
  const int H = h->cfg.hist_size;
  h->n = n;
  h->F = F;
  h->X.assign(X, X + size_t(n) * F);
  h->bins.resize(size_t(n) * F);
  h->mapping.resize(size_t(F) * H);
  h->fsize.resize(F);
#pragma omp parallel for schedule(dynamic)
  for (int f = 0; f < F; ++f) {
    std::vector<float> col(n);
    for (int64_t i = 0; i < n; ++i) col[i] = X[size_t(i) * F + f];
    h->fsize[f] = orc_quantize_column(col.data(), n, H, h->cfg.missing_bin,
                                      &h->mapping[size_t(f) * H],
                                      &h->bins[size_t(f) * n]);
  }
  if (h->C > 0) bin_categories(h);
  return 0;
}
// pre-binned feature-major input with explicit thresholds (extension)
int orc_set_binned(void *p, const uint16_t *bins_fm, int64_t n, int F,
                   const float *mapping, const int *fsize) {
  Handle *h = static_cast<Handle *>(p);
  const int H = h->cfg.hist_size;
  h->n = n;
  h->F = F;
  h->bins.assign(bins_fm, bins_fm + size_t(n) * F);
  h->mapping.assign(mapping, mapping + size_t(F) * H);
  h->fsize.assign(fsize, fsize + F);
  return 0;
}
void orc_set_y(void *p, const float *y) {
  Handle *h = static_cast<Handle *>(p);
  h->y.assign(y, y + h->n);
}
void orc_set_label(void *p, const uint8_t *l) {
  Handle *h = static_cast<Handle *>(p);
  h->label.assign(l, l + h->n);
}
void orc_get_bins(void *p, uint16_t *out, float *mapping, int *fsize) {
  Handle *h = static_cast<Handle *>(p);
  std::copy(h->bins.begin(), h->bins.end(), out);
  if (mapping) std::copy(h->mapping.begin(), h->mapping.end(), mapping);
  if (fsize) std::copy(h->fsize.begin(), h->fsize.end(), fsize);
}
void orc_keep_hist(void *p, int on) {
  Handle *h = static_cast<Handle *>(p);
  if (h->trainer) h->trainer->keep_hist = on;
}

static void ensure_trainer(Handle *h) {
  if (h->trainer) return;
  const Config &c = h->cfg;
  const int Fd = h->F;
  struct Restore {  // the trainers take the feature count from h->F
    Handle *h;
    int Fd;
    ~Restore() {
      h->F = Fd;
      if (h->trainer && h->C > 0) {
        h->trainer->n_dense = Fd;
        h->trainer->cat_candidates = h->cat_candidates;
        h->trainer->cat_codes = h->cat_codes;
      }
    }
  } restore{h, Fd};
  h->F = Fd + h->C;
  const uint8_t *lab = h->label.empty() ? nullptr : h->label.data();
  const float *y = h->y.empty() ? nullptr : h->y.data();
  // chained() dispatch garden.cu:506-569
  if (c.objective == 0) {
    if (c.double_precision)
      h->trainer = new Trainer<float, double>(c, h->n, h->F, h->bins.data(),
                                              h->mapping.data(), h->fsize.data(), y, lab);
    else
      h->trainer = new Trainer<float, float>(c, h->n, h->F, h->bins.data(),
                                             h->mapping.data(), h->fsize.data(), y, lab);
  } else {
    if (c.double_precision)
      h->trainer = new Trainer<f2, d2>(c, h->n, h->F, h->bins.data(), h->mapping.data(),
                                       h->fsize.data(), y, lab);
    else
      h->trainer = new Trainer<f2, f2>(c, h->n, h->F, h->bins.data(), h->mapping.data(),
                                       h->fsize.data(), y, lab);
  }
}

int orc_init(void *p) {
  ensure_trainer(static_cast<Handle *>(p));
  return 0;
}

int orc_grow(void *p) {
  Handle *h = static_cast<Handle *>(p);
  try {
    ensure_trainer(h);
    h->trainer->grow_round();
    return 0;
  } catch (const std::string &e) {
    h->error = e;
    return 1;
  }
}
int orc_num_trees(void *p) {
  Handle *h = static_cast<Handle *>(p);
  return h->trainer ? int(h->trainer->trees.size()) : 0;
}
// nodes: (1<<depth)-1 entries; weights: 1<<(depth-1)
void orc_get_tree(void *p, int t, int *fid, int *quantized, float *threshold,
                  float *weights) {
  Handle *h = static_cast<Handle *>(p);
  const Tree &tr = h->trainer->trees[t];
  for (size_t i = 0; i < tr.nodes.size(); ++i) {
    fid[i] = tr.nodes[i].fid;
    quantized[i] = int(tr.nodes[i].quantized);
    threshold[i] = tr.nodes[i].threshold;
  }
  std::copy(tr.weights.begin(), tr.weights.end(), weights);
}
// which nodes test a category, and which (extension)
void orc_get_tree_categories(void *p, int t, int *categorical, uint32_t *category) {
  Handle *h = static_cast<Handle *>(p);
  const Tree &tr = h->trainer->trees[t];
  for (size_t i = 0; i < tr.nodes.size(); ++i) {
    categorical[i] = tr.nodes[i].categorical ? 1 : 0;
    category[i] = tr.nodes[i].category;
  }
}
// per-level stats of tree t, level l (L = 1<<l entries; node_begin L+1)
void orc_get_level(void *p, int t, int l, uint32_t *node_begin, float *gain, float *gain2,
                   int *fid, int *bin, double *left_g, double *left_h, double *tot_g,
                   double *tot_h, uint32_t *left_count, double *abs_g) {
  Handle *h = static_cast<Handle *>(p);
  const LevelStat &s = h->trainer->stats[t][l];
  const int L = 1 << l;
  std::copy(s.node_begin.begin(), s.node_begin.end(), node_begin);
  for (int i = 0; i < L; ++i) {
    gain[i] = s.gain[i];
    gain2[i] = s.gain2[i];
    fid[i] = s.fid[i];
    bin[i] = s.bin[i];
    left_g[i] = s.left_g[i];
    left_h[i] = s.left_h[i];
    tot_g[i] = s.tot_g[i];
    tot_h[i] = s.tot_h[i];
    left_count[i] = s.left_count[i];
    abs_g[i] = s.abs_g[i];
  }
}
// histogram of (level, feature) of the last grown tree (needs orc_keep_hist)
int orc_get_hist(void *p, int level, int fid, double *g, double *hh, uint32_t *c) {
  Handle *h = static_cast<Handle *>(p);
  if (!h->trainer || h->trainer->hist_g.empty()) return 1;
  const auto &hg = h->trainer->hist_g[level][fid];
  if (hg.empty()) return 2;
  std::copy(hg.begin(), hg.end(), g);
  std::copy(h->trainer->hist_h[level][fid].begin(), h->trainer->hist_h[level][fid].end(), hh);
  std::copy(h->trainer->hist_c[level][fid].begin(), h->trainer->hist_c[level][fid].end(), c);
  return 0;
}
// training-time y_hat (internal scale) in original row order: [k][row]
void orc_get_yhat(void *p, float *out) {
  static_cast<Handle *>(p)->trainer->get_yhat(out);
}
// Garden::Predict garden.cu:643-657 over the handle's own dense rows or X given
// explicitly; out layout [row] or [row][K] (core.py:273-277)
void orc_predict_cat(void *p, const float *X, const uint32_t *cat, int64_t n, int n_rounds, float *out);
void orc_predict(void *p, const float *X, int64_t n, int n_rounds, float *out) {
  orc_predict_cat(p, X, nullptr, n, n_rounds, out);
}
// the same with the rows' category codes (row-major [n][C]; extension)
void orc_predict_cat(void *p, const float *X, const uint32_t *cat, int64_t n, int n_rounds, float *out) {
  Handle *h = static_cast<Handle *>(p);
  const Config &c = h->cfg;
  const int K = c.labels_count;
  float init = c.initial_y;
  if (c.objective == 1) init = std::log(init / (1 - init));
  std::vector<float> tmp(size_t(n) * K, init);
  const auto &trees = h->trainer->trees;
  const int cnt = std::min<int>(n_rounds < 0 ? INT32_MAX : n_rounds, int(trees.size()));
  for (int i = 0; i < cnt; ++i)
    tree_predict(trees[i], X, n, h->F, tmp.data() + size_t(trees[i].label) * n, cat, h->C);
  if (c.objective == 1) {
    for (int64_t i = 0; i < n; ++i) out[i] = sigmoid(tmp[i]);  // objective.h:58-64
  } else if (c.objective == 3) {                               // objective.h:80-113
    for (int64_t i = 0; i < n; ++i) {
      std::vector<double> pr(K);
      double sum = 0;
      for (int k = 0; k < K; ++k) {
        pr[k] = std::exp(double(tmp[i + n * k]));
        sum += pr[k];
      }
      for (int k = 0; k < K; ++k) out[i * K + k] = float(pr[k] / sum);
    }
  } else {
    for (int64_t i = 0; i < n; ++i) out[i] = tmp[i];
  }
}
}  // extern "C"
