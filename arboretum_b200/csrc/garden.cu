// Orchestration of one boosting round (rows F, N, T of the hot path; reference:
// Garden::GrowTree src/core/garden.cu:585-625 and ContinuousGardenBuilder
// :78-504).  A whole tree is enqueued on one stream without host
// synchronisation: node sizes, work lists and split records stay in device
// memory, and the host reads the finished tree back once per tree.
#include <mutex>

#include "garden.h"
#include "exchange.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <exception>
#include <limits>
#include <thread>
#include <vector>

namespace arb {

long long g_kernel_launches = 0;

namespace {
// one stream per device for the pool's allocations and frees; the pool keeps freed memory
cudaStream_t pool_stream() {
  constexpr int kMaxDevices = 64;
  static cudaStream_t streams[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!streams[dev]) {
    cudaMemPool_t pool = nullptr;
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
      unsigned long long keep = ~0ull;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    if (cudaStreamCreateWithFlags(&streams[dev], cudaStreamNonBlocking) != cudaSuccess) streams[dev] = nullptr;
  }
  return streams[dev];
}
}  // namespace

cudaError_t dev_alloc(void **p, size_t bytes) {
  cudaStream_t st = pool_stream();
  if (!st) return cudaMalloc(p, bytes);
  cudaError_t e = cudaMallocAsync(p, bytes, st);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(st);
}

void dev_free(void *p) {
  if (!p) return;
  cudaDeviceSynchronize();  // nothing on any stream may still use the block
  cudaStream_t st = pool_stream();
  if (!st || cudaFreeAsync(p, st) != cudaSuccess) cudaFree(p);
}

namespace {
constexpr size_t kPinnedKeepBlock = size_t(16) << 20, kPinnedKeepTotal = size_t(64) << 20;
struct PinnedBlock {
  void *p;
  size_t cap;
};
// never destroyed: a buffer may be given back while the process is already on its way out
std::mutex &g_pinned_mutex = *new std::mutex;
std::vector<PinnedBlock> &g_pinned_free = *new std::vector<PinnedBlock>;
size_t g_pinned_kept = 0;
void pinned_drop_all() {
  std::lock_guard<std::mutex> lock(g_pinned_mutex);
  for (const PinnedBlock &b : g_pinned_free) cudaFreeHost(b.p);
  g_pinned_free.clear();
  g_pinned_kept = 0;
}
}  // namespace

cudaError_t pinned_alloc(void **p, size_t bytes, size_t *cap) {
  {
    std::lock_guard<std::mutex> lock(g_pinned_mutex);
    int best = -1;  // the smallest kept block that is large enough, and not wastefully large
    for (int i = 0; i < int(g_pinned_free.size()); ++i)
      if (g_pinned_free[i].cap >= bytes && g_pinned_free[i].cap <= 2 * bytes + 4096 &&
          (best < 0 || g_pinned_free[i].cap < g_pinned_free[best].cap))
        best = i;
    if (best >= 0) {
      *p = g_pinned_free[best].p;
      *cap = g_pinned_free[best].cap;
      g_pinned_kept -= *cap;
      g_pinned_free.erase(g_pinned_free.begin() + best);
      return cudaSuccess;
    }
  }
  *cap = bytes;
  return cudaMallocHost(p, bytes);
}

void pinned_free(void *p, size_t cap) {
  if (!p) return;
  // a copy that still uses the block must be over before it is handed out again
  cudaDeviceSynchronize();
  {
    std::lock_guard<std::mutex> lock(g_pinned_mutex);
    if (cap <= kPinnedKeepBlock && g_pinned_kept + cap <= kPinnedKeepTotal) {
      g_pinned_free.push_back(PinnedBlock{p, cap});
      g_pinned_kept += cap;
      return;
    }
  }
  cudaFreeHost(p);
}

cudaError_t dev_trim() {
  pinned_drop_all();
  int dev = 0;
  cudaMemPool_t pool = nullptr;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetDefaultMemPool(&pool, dev);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemPoolTrimTo(pool, 0);
  return e;
}

cudaError_t dev_available(size_t *bytes) {
  size_t free_b = 0, total_b = 0;
  cudaError_t e = cudaMemGetInfo(&free_b, &total_b);
  if (e != cudaSuccess) return e;
  int dev = 0;
  cudaMemPool_t pool = nullptr;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
    unsigned long long reserved = 0, used = 0;
    if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved) == cudaSuccess &&
        cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &used) == cudaSuccess && reserved > used)
      free_b += size_t(reserved - used);
  }
  *bytes = free_b;
  return cudaSuccess;
}

// ---------------------------------------------------------------------------
// DataMatrix
// ---------------------------------------------------------------------------
namespace {
// unpadded rows -> padded rows on the host, rows dealt to a few threads
void pad_rows_host(const unsigned char *src, size_t F, size_t n, unsigned char *dst, size_t pitch) {
  const unsigned hw = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
  const size_t per = (n + hw - 1) / hw;
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < hw; ++t) {
    const size_t lo = std::min(n, t * per), hi = std::min(n, lo + per);
    if (lo == hi) break;
    pool.emplace_back([=]() {
      for (size_t r = lo; r < hi; ++r) {
        std::memcpy(dst + r * pitch, src + r * F, F);
        std::memset(dst + r * pitch + F, 0, pitch - F);
      }
    });
  }
  for (auto &th : pool) th.join();
}
}  // namespace

// Thresholds of the whole data set when every rank holds a shard of the rows (same result
// as InitHist on the unsharded matrix, bit for bit).  A block of 32 columns at a time: every
// rank makes its rows' columns contiguous, pads them with NaN (which sorts last) to the
// longest shard and all ranks all-gather the block; rank r then sorts the whole columns
// f with f % world == r and scans them for thresholds, so the sorts are spread over the
// GPUs; the threshold tables are all-gathered at the end.
void DataMatrix::ShardedThresholds(const float *d_x_local, int hs, const ShardInfo &sh, cudaStream_t s) {
  const int F = cols_dense, world = sh.world;
  const size_t n = size_t(rows);
  // row counts of all ranks
  DevBuf d_cnt;
  d_cnt.alloc(sizeof(unsigned long long) * (world + 1));
  const unsigned long long mine = n;
  ARB_CUDA(cudaMemcpyAsync(d_cnt.as<unsigned long long>() + world, &mine, sizeof mine, cudaMemcpyHostToDevice, s));
  if (sh.allgather(sh.ctx, d_cnt.as<unsigned long long>() + world, d_cnt.p, sizeof mine, s) != 0)
    throw std::runtime_error("row-count all-gather failed");
  std::vector<unsigned long long> counts(world);
  ARB_CUDA(cudaMemcpyAsync(counts.data(), d_cnt.p, sizeof(unsigned long long) * world, cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaStreamSynchronize(s));
  size_t n_total = 0, n_max = 0;
  for (unsigned long long c : counts) {
    n_total += size_t(c);
    n_max = std::max(n_max, size_t(c));
  }
  const int block_cols = std::min(F, 32);
  const size_t whole = size_t(world) * n_max;  // a whole column with its padding
  DevBuf arena, d_local, d_send, d_recv, d_full, d_sorted, d_tmp, d_scratch, d_thr_f, d_thr_all;
  {
    struct Want {
      DevBuf *buf;
      size_t bytes;
    };
    const Want wants[] = {
      {&d_local, n * block_cols * sizeof(float)},
      {&d_send, n_max * block_cols * sizeof(float)},
      {&d_recv, whole * block_cols * sizeof(float)},
      {&d_full, whole * sizeof(float)},
      {&d_sorted, whole * sizeof(float)},
      {&d_tmp, sort_floats_temp_bytes(whole)},
      {&d_scratch, thresholds_scratch_words(n_total) * sizeof(unsigned)},
      {&d_thr_f, size_t(F) * hs * sizeof(float)},
      {&d_thr_all, size_t(world) * F * hs * sizeof(float)},
    };
    size_t total = 0;
    for (const Want &w : wants) total += (w.bytes + 255) / 256 * 256;
    arena.alloc(total);
    size_t at = 0;
    for (const Want &w : wants) {
      w.buf->view(static_cast<char *>(arena.p) + at, w.bytes);
      at += (w.bytes + 255) / 256 * 256;
    }
  }
  ARB_CUDA(cudaMemsetAsync(d_thr_f.p, 0, d_thr_f.bytes, s));
  const float pad = std::numeric_limits<float>::quiet_NaN();  // 0x7fc00000, like the transposed NaNs
  for (int f0 = 0; f0 < F; f0 += block_cols) {
    const int nf = std::min(block_cols, F - f0);
    launch_transpose_columns(d_x_local, n, F, f0, nf, d_local.as<float>(), s);
    launch_fill(d_send.as<float>(), n_max * nf, pad, s);
    ARB_CUDA(cudaMemcpy2DAsync(d_send.p, n_max * sizeof(float), d_local.p, n * sizeof(float), n * sizeof(float),
                               nf, cudaMemcpyDeviceToDevice, s));
    const size_t block_bytes = n_max * nf * sizeof(float);
    if (sh.allgather(sh.ctx, d_send.p, d_recv.p, block_bytes, s) != 0)
      throw std::runtime_error("column all-gather failed");
    for (int c = 0; c < nf; ++c) {
      const int f = f0 + c;
      if (f % world != sh.rank) continue;
      // column c of every rank's block, rank after rank
      ARB_CUDA(cudaMemcpy2DAsync(d_full.p, n_max * sizeof(float), d_recv.as<float>() + size_t(c) * n_max,
                                 block_bytes, n_max * sizeof(float), world, cudaMemcpyDeviceToDevice, s));
      sort_floats(d_full.as<float>(), d_sorted.as<float>(), whole, d_tmp, s);
      launch_thresholds(d_sorted.as<float>(), n_total, hs, d_thr_f.as<float>() + size_t(f) * hs,
                        d_scratch.as<unsigned>(), s);
    }
  }
  if (sh.allgather(sh.ctx, d_thr_f.p, d_thr_all.p, d_thr_f.bytes, s) != 0)
    throw std::runtime_error("threshold all-gather failed");
  std::vector<float> all(size_t(world) * F * hs);
  ARB_CUDA(cudaMemcpyAsync(all.data(), d_thr_all.p, d_thr_all.bytes, cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaStreamSynchronize(s));
  thr.resize(size_t(F) * hs);
  for (int f = 0; f < F; ++f) {
    const float *src = all.data() + (size_t(f % world) * F + f) * hs;
    std::copy(src, src + hs, thr.begin() + size_t(f) * hs);
  }
}

// Bins of the categorical columns (this build's completion of the reference's stub,
// hist_tree_grower.h:55-63; the intended split is one category against the rest,
// builder.h:75-105, garden.h:79-84).  A category's bin id is its rank by frequency (most
// frequent first, ties: smaller code first).  A column with more than hist_size categories
// keeps the hist_size - 1 most frequent ones; the others share bin hist_size - 1, which no
// split may name.  Appends the columns' entries to fsize and fills cat_codes /
// cat_candidates; the bin ids go into columns cols_dense.. of d_bins.
void DataMatrix::BinCategories(cudaStream_t s) {
  const size_t n = size_t(rows);
  const int C = cols_cat, hs = hist_size;
  ARB_CHECK(cat.size() == n * size_t(C), "categories are missing");
  fsize.resize(size_t(cols_dense));
  cat_codes.assign(size_t(C), std::vector<unsigned>());
  // bin ids column by column ([c][r]): the columns are worked on side by side by a few threads
  std::vector<unsigned char> ids8;
  std::vector<unsigned short> ids16;
  if (bin_bytes == 1) ids8.resize(n * C); else ids16.resize(n * C);
  std::vector<int> col_fsize(C, 0), col_kept(C, 0);
  auto bin_column = [&](int c) {
    // (code, rows) of the column, codes ascending: counted in a table while the codes are
    // small (the usual case), from a sorted copy otherwise
    std::vector<std::pair<unsigned, size_t>> freq;
    unsigned max_code = 0;
    for (size_t r = 0; r < n; ++r) max_code = std::max(max_code, cat[r * C + c]);
    const bool table = max_code < (1u << 22);
    std::vector<unsigned> count;
    if (table) {
      count.assign(size_t(max_code) + 1, 0u);
      for (size_t r = 0; r < n; ++r) ++count[cat[r * C + c]];
      for (size_t code = 0; code < count.size(); ++code)
        if (count[code]) freq.emplace_back(unsigned(code), size_t(count[code]));
    } else {
      std::vector<unsigned> col(n);
      for (size_t r = 0; r < n; ++r) col[r] = cat[r * C + c];
      std::sort(col.begin(), col.end());
      for (size_t i = 0; i < n;) {
        size_t k = i;
        while (k < n && col[k] == col[i]) ++k;
        freq.emplace_back(col[i], k - i);
        i = k;
      }
    }
    std::stable_sort(freq.begin(), freq.end(),
                     [](const std::pair<unsigned, size_t> &a, const std::pair<unsigned, size_t> &b) {
                       return a.second > b.second;  // codes ascend within equal counts (stable)
                     });
    const bool overflow = freq.size() > size_t(hs);
    const size_t kept = overflow ? size_t(hs - 1) : freq.size();
    std::vector<std::pair<unsigned, unsigned>> by_code;  // (code, bin)
    for (size_t b = 0; b < kept; ++b) {
      cat_codes[c].push_back(freq[b].first);
      by_code.emplace_back(freq[b].first, unsigned(b));
    }
    std::sort(by_code.begin(), by_code.end());
    col_fsize[c] = int(kept + (overflow ? 1 : 0));
    col_kept[c] = int(kept);
    if (table) {  // the table now maps a code to its bin
      std::fill(count.begin(), count.end(), unsigned(kept));
      for (const auto &cb : by_code) count[cb.first] = cb.second;
    }
    for (size_t r = 0; r < n; ++r) {
      const unsigned code = cat[r * C + c];
      unsigned b;
      if (table) {
        b = count[code];
      } else {
        auto it = std::lower_bound(by_code.begin(), by_code.end(), std::make_pair(code, 0u));
        b = (it != by_code.end() && it->first == code) ? it->second : unsigned(kept);
      }
      if (bin_bytes == 1) ids8[size_t(c) * n + r] = (unsigned char)b; else ids16[size_t(c) * n + r] = (unsigned short)b;
    }
  };
  {
    const int workers = std::max(1, std::min<int>(C, int(std::min(16u, std::thread::hardware_concurrency()))));
    std::vector<std::thread> pool;
    std::vector<std::exception_ptr> failed(workers);
    for (int t = 0; t < workers; ++t)
      pool.emplace_back([&, t]() {
        try {
          for (int c = t; c < C; c += workers) bin_column(c);
        } catch (...) {
          failed[t] = std::current_exception();
        }
      });
    for (auto &th : pool) th.join();
    for (auto &e : failed)
      if (e) std::rethrow_exception(e);
  }
  for (int c = 0; c < C; ++c) {
    fsize.push_back(col_fsize[c]);
    cat_candidates[size_t(cols_dense + c)] = col_kept[c];
  }
  DevBuf d_ids;
  d_ids.alloc(n * C * size_t(bin_bytes));
  const void *src = bin_bytes == 1 ? static_cast<const void *>(ids8.data()) : static_cast<const void *>(ids16.data());
  ARB_CUDA(cudaMemcpyAsync(d_ids.p, src, d_ids.bytes, cudaMemcpyHostToDevice, s));
  launch_place_columns(d_ids.p, n, C, cols_dense, d_bins.as<unsigned char>(), pitch, bin_bytes, s, true);
  ARB_CUDA(cudaStreamSynchronize(s));
}

void DataMatrix::InitHist(int hs, bool missing_bin, bool verbose, cudaStream_t s, long long chunk_rows,
                          const ShardInfo *shards) {
  if (binned) return;
  out_of_core = chunk_rows > 0 && chunk_rows < rows;
  const int F = cols_dense;
  ARB_CHECK(hs > 0 && hs < 2048, "hist_size must be in [1, 2047]");
  ARB_CHECK(F > 0 && rows > 0, "empty data matrix");
  hist_size = hs;
  // io.cu:342-347: hist_size < 256 -> uint8 bins, else uint16
  bin_bytes = hs < 256 ? 1 : 2;
  pitch = PitchFor(cols(), bin_bytes);
  const size_t n = size_t(rows);
  StageTrace trace("InitHist");
  ARB_CHECK(cols_cat == 0 || !(shards && shards->world > 1),
            "categorical columns are not supported with row shards (their bins follow the category "
            "frequencies of the whole data set)");
  if (!prebinned) {
    DevBuf d_quant_arena, d_x_tmp, d_col, d_sorted, d_tmp, d_scratch, d_thr_f;
    if (!d_x.p) {
      d_x_tmp.alloc(n * F * sizeof(float));
      ARB_CUDA(cudaMemcpyAsync(d_x_tmp.p, x.data(), n * F * sizeof(float), cudaMemcpyHostToDevice, s));
    }
    const DevBuf &d_x = this->d_x.p ? this->d_x : d_x_tmp;
    if (!thresholds_given && shards && shards->world > 1 && shards->allgather) {
      ShardedThresholds(d_x.as<float>(), hs, *shards, s);
      trace.lap("sharded column sorts + thresholds");
    } else if (!thresholds_given) {
      const int block_cols = std::min(F, 32);  // columns made contiguous at a time
      // short columns are sorted a block at a time (one sort over (column, value) keys): a
      // 1 M-row column alone is launch-bound; long ones one by one (half the bytes per key)
      const bool batched = block_cols > 1 && n <= (size_t(1) << 21) &&
                           std::getenv("ARBORETUM_NO_BATCHED_SORT") == nullptr;
      DevBuf d_keys_a, d_keys_b;
      const int sort_cols = std::min(block_cols, 8);  // columns per sort: keeps the key buffers small
      {  // one allocation (and later one free) for the quantizer's temporaries
        struct Want {
          DevBuf *buf;
          size_t bytes;
        };
        const size_t key_bytes = batched ? n * sort_cols * sizeof(unsigned long long) : 0;
        const Want wants[] = {
          {&d_col, n * block_cols * sizeof(float)},
          {&d_sorted, batched ? 0 : n * sizeof(float)},
          {&d_tmp, batched ? sort_columns_temp_bytes(n, sort_cols) : sort_floats_temp_bytes(n)},
          {&d_scratch, thresholds_scratch_words(n) * sizeof(unsigned) * (batched ? block_cols : 1)},
          {&d_thr_f, size_t(F) * hs * sizeof(float)},
          {&d_keys_a, key_bytes},
          {&d_keys_b, key_bytes},
        };
        size_t total = 0;
        for (const Want &w : wants) total += (w.bytes + 255) / 256 * 256;
        d_quant_arena.alloc(total);
        size_t at = 0;
        for (const Want &w : wants) {
          if (w.bytes) w.buf->view(static_cast<char *>(d_quant_arena.p) + at, w.bytes);
          at += (w.bytes + 255) / 256 * 256;
        }
      }
      for (int f0 = 0; f0 < F; f0 += block_cols) {
        const int nf = std::min(block_cols, F - f0);
        launch_transpose_columns(d_x.as<float>(), n, F, f0, nf, d_col.as<float>(), s);
        if (batched) {
          for (int c0 = 0; c0 < nf; c0 += sort_cols)
            sort_columns(d_col.as<float>() + size_t(c0) * n, n, std::min(sort_cols, nf - c0),
                         d_keys_a.as<unsigned long long>(), d_keys_b.as<unsigned long long>(), d_tmp, s);
          launch_thresholds_columns(d_col.as<float>(), n, nf, hs, d_thr_f.as<float>() + size_t(f0) * hs,
                                    d_scratch.as<unsigned>(), s);
          continue;
        }
        for (int f = f0; f < f0 + nf; ++f) {
          const float *sorted = d_col.as<float>() + size_t(f - f0) * n;
          if (!batched) {
            sort_floats(sorted, d_sorted.as<float>(), n, d_tmp, s);
            sorted = d_sorted.as<float>();
          }
          launch_thresholds(sorted, n, hs, d_thr_f.as<float>() + size_t(f) * hs, d_scratch.as<unsigned>(), s);
        }
      }
      trace.lap("column sorts + thresholds");
      thr.resize(size_t(F) * hs);
      ARB_CUDA(cudaMemcpyAsync(thr.data(), d_thr_f.p, thr.size() * sizeof(float),
                               cudaMemcpyDeviceToHost, s));
      ARB_CUDA(cudaStreamSynchronize(s));
    }
    if (!thresholds_given) {
      fsize.resize(F);
      for (int f = 0; f < F; ++f) {  // io.cu:403-410
        int unique = 0;
        while (unique < hs && !std::isinf(thr[size_t(f) * hs + unique])) ++unique;
        ++unique;
        fsize[f] = std::min(unique, hs);
      }
    }
    ARB_CHECK(int(thr.size()) == F * hs && int(fsize.size()) == F, "threshold table has the wrong shape");
    DevBuf d_thr_arena, d_thr, d_fsize;
    {
      const size_t a = (thr.size() * sizeof(float) + 255) / 256 * 256;
      d_thr_arena.alloc(a + F * sizeof(int));
      d_thr.view(d_thr_arena.p, thr.size() * sizeof(float));
      d_fsize.view(static_cast<char *>(d_thr_arena.p) + a, F * sizeof(int));
    }
    ARB_CUDA(cudaMemcpyAsync(d_thr.p, thr.data(), thr.size() * sizeof(float), cudaMemcpyHostToDevice, s));
    ARB_CUDA(cudaMemcpyAsync(d_fsize.p, fsize.data(), F * sizeof(int), cudaMemcpyHostToDevice, s));
    d_bins.alloc(n * pitch);
    ARB_CUDA(cudaMemsetAsync(d_bins.p, 0, n * pitch, s));
    launch_binning(d_x.as<float>(), n, F, d_thr.as<float>(), d_fsize.as<int>(), hs, missing_bin,
                   d_bins.as<unsigned char>(), pitch, bin_bytes, s);
    cat_candidates.assign(size_t(cols()), 0);
    if (cols_cat > 0) BinCategories(s);
    if (out_of_core) {  // the bins live in pinned host memory and are streamed per level
      host_pitch = HostPitchFor(cols(), bin_bytes);
      h_bins.alloc(n * host_pitch);
      if (host_pitch == pitch)
        ARB_CUDA(cudaMemcpyAsync(h_bins.p, d_bins.p, n * pitch, cudaMemcpyDeviceToHost, s));
      else
        ARB_CUDA(cudaMemcpy2DAsync(h_bins.p, host_pitch, d_bins.p, pitch, host_pitch, n,
                                   cudaMemcpyDeviceToHost, s));
    }
    ARB_CUDA(cudaStreamSynchronize(s));
    if (out_of_core) d_bins.release();
    trace.lap("binning");
  } else if (out_of_core) {
    ARB_CHECK(bin_bytes == 1, "pre-binned input is uint8: hist_size must be < 256");
    host_pitch = HostPitchFor(F, bin_bytes);
    h_bins.alloc(n * host_pitch);
    if (d_raw.p && host_pitch == size_t(F)) {  // the rows as they are
      ARB_CUDA(cudaMemcpyAsync(h_bins.p, d_raw.p, n * size_t(F), cudaMemcpyDeviceToHost, s));
      ARB_CUDA(cudaStreamSynchronize(s));
    } else if (d_raw.p) {  // pad on the device, a slab of rows at a time, and bring the slabs back
      const size_t slab = std::min<size_t>(n, size_t(1) << 24);
      DevBuf d_slab;
      d_slab.alloc(slab * host_pitch);
      for (size_t first = 0; first < n; first += slab) {
        const size_t count = std::min(slab, n - first);
        launch_pad_rows(d_raw.as<unsigned char>() + first * F, F, count, d_slab.as<unsigned char>(), host_pitch, s);
        ARB_CUDA(cudaMemcpyAsync(h_bins.as<unsigned char>() + first * host_pitch, d_slab.p, count * host_pitch,
                                 cudaMemcpyDeviceToHost, s));
      }
      ARB_CUDA(cudaStreamSynchronize(s));
    } else {
      pad_rows_host(host_bins.data(), size_t(F), n, h_bins.as<unsigned char>(), host_pitch);
    }
    if (thr.empty()) {
      thr.resize(size_t(F) * hs);
      fsize.assign(F, hs);
      for (int f = 0; f < F; ++f)
        for (int q = 0; q < hs; ++q) thr[size_t(f) * hs + q] = q + 0.5f;
    }
  } else {
    // rows arrive already binned: copy them into the padded row-major layout
    ARB_CHECK(bin_bytes == 1, "pre-binned input is uint8: hist_size must be < 256");
    d_bins.alloc(n * pitch);
    if (d_raw.p) {
      launch_pad_rows(d_raw.as<unsigned char>(), F, n, d_bins.as<unsigned char>(), pitch, s);
    } else {
      ARB_CUDA(cudaMemsetAsync(d_bins.p, 0, n * pitch, s));
      ARB_CUDA(cudaMemcpy2DAsync(d_bins.p, pitch, host_bins.data(), size_t(F), size_t(F), n,
                                 cudaMemcpyHostToDevice, s));
    }
    if (thr.empty()) {  // threshold of bin q is q + 0.5: "bin <= q" <=> "value < q + 0.5"
      thr.resize(size_t(F) * hs);
      fsize.assign(F, hs);
      for (int f = 0; f < F; ++f)
        for (int q = 0; q < hs; ++q) thr[size_t(f) * hs + q] = q + 0.5f;
    }
    ARB_CUDA(cudaStreamSynchronize(s));
  }
  if (!out_of_core) {  // feature-major copy: F x N bins more, cheap next to the row-major matrix
    d_bins_cm.alloc(size_t(cols()) * n * bin_bytes);
    launch_transpose_bins(d_bins.as<unsigned char>(), pitch, bin_bytes, n, cols(),
                          d_bins_cm.as<unsigned char>(), s);
    ARB_CUDA(cudaStreamSynchronize(s));
  }
  trace.lap("feature-major copy (and temporaries freed)");
  if (cat_candidates.empty()) cat_candidates.assign(size_t(cols()), 0);
  max_reduced_bits = 0;
  for (int f = 0; f < F; ++f) {
    int bits = 0;
    for (int v = fsize[f]; v > 0; v >>= 1) ++bits;  // io.cu:411  32 - clz(size)
    max_reduced_bits = std::max(max_reduced_bits, bits);
    if (verbose) printf("feature %d has been reduced to %d bits \n", f, bits);
  }
  if (verbose) printf("max feature size %d \n", max_reduced_bits);
  binned = true;
}

namespace {
// rows of `data` as fp32 on the device, `chunk` rows at a time
struct RowFeeder {
  DataMatrix *d;
  DevBuf buf;
  std::vector<float> staged;
  size_t chunk;
  explicit RowFeeder(DataMatrix *dm) : d(dm) {
    const size_t row_bytes = size_t(d->cols_dense) * sizeof(float);
    chunk = std::max<size_t>(1, std::min<size_t>(size_t(d->rows), (size_t(1) << 30) / row_bytes));
    if (!d->d_x.p) buf.alloc(chunk * row_bytes);
  }
  // category codes of the rows from `first` on (device), or nullptr
  const unsigned *categories(size_t first) const {
    return d->d_cat.p ? d->d_cat.as<unsigned>() + first * size_t(d->cols_cat) : nullptr;
  }
  const float *load(size_t first, size_t count, cudaStream_t s) {
    const int F = d->cols_dense;
    if (d->d_x.p) return d->d_x.as<float>() + first * F;  // already in HBM
    if (d->prebinned && d->d_raw.p) {  // pre-binned rows predict on their bin ids as values
      launch_u8_to_f32(d->d_raw.as<unsigned char>() + first * F, buf.as<float>(), count * F, s);
    } else if (d->prebinned) {
      staged.resize(count * F);
      for (size_t i = 0; i < count * F; ++i) staged[i] = float(d->host_bins[first * F + i]);
      ARB_CUDA(cudaMemcpyAsync(buf.p, staged.data(), count * F * sizeof(float), cudaMemcpyHostToDevice, s));
    } else {
      ARB_CUDA(cudaMemcpyAsync(buf.p, d->x.data() + first * F, count * F * sizeof(float),
                               cudaMemcpyHostToDevice, s));
    }
    return buf.as<float>();
  }
};
}  // namespace

// ---------------------------------------------------------------------------
// Builder: device state of one (Garden, DataMatrix) pair
// ---------------------------------------------------------------------------
class Builder {
 public:
  Builder(Garden *g, DataMatrix *d);
  ~Builder();
  Builder(const Builder &) = delete;
  Builder &operator=(const Builder &) = delete;
  void UpdateGrad();
  void GrowTree(int label, Tree *tree);
  void Resume();
  DataMatrix *data;

 private:
  Garden *g_;
  size_t n_;
  int F_, K_, levels_, max_nodes_, nb_stride_;
  bool pair_;
  Geometry geo_;
  int qb_ = 18;        // fixed-point bits of a gradient
  int item_cap_;       // rows an int32 sub-histogram may take (2^(31 - quant_bits))
  int max_hist_items_, max_hist_runs_;
  std::default_random_engine rnd_;  // garden.cu:87
  std::vector<unsigned> active_fids_;
  std::vector<unsigned char> active_host_;
  GainParams gp_;

  DevBuf d_y_, d_label_, d_yhat_, d_grad_, d_node_begin_, d_rec_, d_hist_[2], d_keys_, d_qs_,
    d_leaf_w_, d_active_, d_fsize_, d_cat_candidates_;
  DevBuf d_compact_;  // row shards: the built nodes' histograms of a level, the part the ranks sum
  // (gradient, hessian) objectives with min_leaf_size > 1 keep a second histogram that counts
  // rows (the reference's count histogram, gain.cu:125-134): the reg:linear kernel run on a
  // "gradient" array of ones; same level buffers, same subtraction, same exchange
  PeerExchange *xchg_ = nullptr;  // row shards of one box: the level exchange over peer memory
                                  // (the process's; not owned)
  PinnedBuf h_xchg_status_;
  // the histogram kernel's row gather through the TMA unit: a tensor map of the resident bin
  // matrix and the word in which a kernel reports a gather that never arrived
  RowGatherMap row_map_;
  bool has_row_map_ = false;
  DevBuf d_hist_status_;
  PinnedBuf h_hist_status_;
  bool count_plane_ = false;
  // colsample_bytree < 1: the columns a tree samples are copied side by side once per tree and
  // the histograms and the split search cover those alone (feature ids in the records stay the
  // matrix's); used when that saves feature tiles, in core, without row shards
  bool sampled_cols_ = false;
  Geometry geo_tree_;          // the copy's geometry (no feature-major copy: the descend step reads the matrix)
  DevBuf d_bins_tree_, d_fmap_;
  std::vector<int> fmap_host_;
  DevBuf d_ones_, d_cnt_hist_[2], d_compact_cnt_;
  // records of every tree of the last round (multi:softmax grows labels_count of them)
  std::vector<std::vector<NodeRec>> round_rec_;
  std::vector<std::vector<unsigned>> round_nb_;
  void SampleFeatures();
  DevBuf d_node_of_;  // per row: the node (inside the current level) it stands on
  DevBuf d_list_;     // row lists of the built nodes of the current level, back to back
  DevBuf d_list_grad_;  // their gradient records in the same order (uint8 data)
  DevBuf d_partials_, d_hist_items_, d_counters_, d_first_, d_slot_first_, d_item_slot_, d_built_, d_scratch_, d_list_base_,
    d_cursor_, d_child_count_;
  DevBuf d_arena_;      // backs the small per-level arrays below
  DevBuf d_rows_arena_; // backs the per-row arrays
  unsigned long long row_offset_ = 0;  // index of this shard's first row in the whole data set
  unsigned round_ = 0;                 // boosting rounds so far (keys the gradients' dither)
  bool events_made_ = false;
  void EnsureEvents();
  PinnedBuf h_arena_;   // backs the read-back buffers
  PinnedBuf h_rec_, h_leaf_w_, h_node_begin_;
  std::vector<unsigned> h_nb_total_;
  PlanBuffers pb_;
  cudaEvent_t ev_[2 * 8 * kMaxLevels];
  cudaEvent_t ev_hist_[kMaxLevels];  // behind the first histogram launch of a level (profile mode)
  cudaEvent_t ev_tree_[2];
  // Row chunks (out-of-core): a chunk is a contiguous range of rows whose bins are
  // either resident in HBM or streamed from pinned host memory into one of two
  // staging buffers once per level.  In-core training is one resident chunk.
  struct Chunk {
    size_t begin, rows;
    const unsigned char *resident;  // device bins of the chunk, or nullptr (streamed)
  };
  std::vector<Chunk> chunks_;
  DevBuf d_stage_[2], d_resident_;
  DevBuf d_stage_raw_[2];  // host rows without padding land here and are padded into d_stage_
  cudaStream_t copy_stream_ = nullptr;
  cudaEvent_t stage_ready_[2], stage_free_[2];
  int stage_of_next_ = 0;
  std::vector<int> streamed_;       // indices of the streamed chunks, in visiting order
  size_t issued_ = 0, consumed_ = 0;  // position in the endless cyclic sequence of `streamed_`
  const unsigned char *Acquire(int chunk);
  void Release(int chunk);
  void IssueCopy();
  friend class Garden;
  friend struct BuilderView;

  unsigned *node_begin(int chunk, int level) {
    return d_node_begin_.as<unsigned>() + (size_t(chunk) * (levels_ + 1) + level) * nb_stride_;
  }
  NodeRec *rec(int level) { return d_rec_.as<NodeRec>() + size_t(level) * max_nodes_; }
};

Builder::Builder(Garden *g, DataMatrix *d) : data(d), g_(g), rnd_(g->cfg.internal.seed) {
  const Configuration &cfg = g->cfg;
  const TreeParam &tp = cfg.tree;
  cudaStream_t s = g->stream;
  StageTrace trace("Builder");
  n_ = size_t(d->rows);
  F_ = d->cols();
  K_ = int(tp.labels_count);
  ARB_CHECK(tp.depth >= 2 && tp.depth <= kMaxLevels, "max_depth must be in [1, 15]");
  ARB_CHECK(n_ < (size_t(1) << 31), "row count must be below 2^31");
  ARB_CHECK(F_ < 65535, "more than 65534 features");
  if (d->device >= 0) {
    int cur = -1;
    ARB_CUDA(cudaGetDevice(&cur));
    ARB_CHECK(cur == d->device, "the DMatrix was created on another CUDA device than the Garden uses");
  }
  levels_ = int(tp.depth) - 1;
  max_nodes_ = 1 << (levels_ - 1);
  nb_stride_ = 2 * max_nodes_ + 1;
  pair_ = cfg.objective != kLinearRegression;
  count_plane_ = pair_ && tp.min_leaf_size > 1;
  if (cfg.objective == kSoftMaxOneVsAll)
    ARB_CHECK(d->has_labels(), "multi:softmax needs labels (ASetLabel)");
  else
    ARB_CHECK(d->has_y(), "labels are not set (ASetY)");

  geo_.bins = d->d_bins.as<unsigned char>();
  geo_.pitch = d->pitch;
  geo_.bin_bytes = d->bin_bytes;
  geo_.F = F_;
  geo_.n_dense = d->cols_dense;
  geo_.hist_size = d->hist_size;
  int bins_pad = 256;
  while (bins_pad < d->hist_size + 1) bins_pad <<= 1;
  geo_.BINS = bins_pad;
  geo_.TW = kHistWords / bins_pad;
  geo_.NT = (F_ + geo_.TW - 1) / geo_.TW;
  geo_.bins_cm = d->d_bins_cm.as<unsigned char>();
  geo_.cm_rows = n_;
  if (geo_.bins && geo_.bin_bytes == 1 && geo_.TW == 32 &&
      make_row_gather_map(&row_map_, geo_.bins, geo_.pitch, n_)) {
    has_row_map_ = true;
    d_hist_status_.alloc(sizeof(int));
    ARB_CUDA(cudaMemsetAsync(d_hist_status_.p, 0, sizeof(int), s));
    h_hist_status_.alloc(sizeof(int));
    *h_hist_status_.as<int>() = 0;
  }

  size_t n_global = n_;
  if (g->shards.world > 1 && g->shards.allgather) {
    // where this shard's rows lie in the whole data set (shards are contiguous, in rank order)
    const int world = g->shards.world;
    DevBuf d_cnt;
    d_cnt.alloc(sizeof(unsigned long long) * (world + 1));
    const unsigned long long mine = n_;
    ARB_CUDA(cudaMemcpyAsync(d_cnt.as<unsigned long long>() + world, &mine, sizeof mine, cudaMemcpyHostToDevice, s));
    if (g->shards.allgather(g->shards.ctx, d_cnt.as<unsigned long long>() + world, d_cnt.p, sizeof mine, s) != 0)
      throw std::runtime_error("row-count all-gather failed");
    std::vector<unsigned long long> counts(world);
    ARB_CUDA(cudaMemcpyAsync(counts.data(), d_cnt.p, sizeof(unsigned long long) * world, cudaMemcpyDeviceToHost, s));
    ARB_CUDA(cudaStreamSynchronize(s));
    for (int r = 0; r < g->shards.rank; ++r) row_offset_ += counts[r];
    n_global = 0;
    for (unsigned long long c : counts) n_global += size_t(c);
  }
  // Fixed-point bits of a gradient.  More bits mean smaller rounding errors in the sums (a
  // node's gain is good to about 2 x 0.4 x step x sqrt(rows) / |sum g|) but fewer rows per
  // int32 sub-histogram (2^(31 - bits)) and so more of them to store and add up.  Unless the
  // configuration names a value, the whole data set's row count decides (so that shards and
  // row chunks quantise like one GPU) together with the feature tiles every row is
  // histogrammed in (a sub-histogram is 64 KB per tile: with 32 tiles a thousand rows per
  // sub-histogram would store and re-read twice the bytes of the bins themselves): about a
  // thousand sub-histograms for the root level, between 18 bits (from 4 M row-tiles) and 22
  // (up to half a million).
  qb_ = cfg.internal.quant_bits;
  if (qb_ == 0) {
    const int cols_hist = std::min(F_, std::max(1, int(tp.colsample_bytree * F_)));
    const size_t tiles_hist = size_t((cols_hist + geo_.TW - 1) / geo_.TW);
    int lg = 0;
    while ((size_t(1) << lg) < std::max<size_t>(512, n_global * tiles_hist / 1024)) ++lg;
    qb_ = std::min(22, std::max(18, 31 - lg));
  }
  const int qb = qb_;
  ARB_CHECK(qb >= 10 && qb <= 22, "internals.quant_bits must be 0 (chosen by the row count) or in [10, 22]");
  item_cap_ = 1 << (31 - qb);
  // A level's rows are cut into items of item_cap_ >> j rows (a power-of-two share of what an
  // int32 plane holds), about kItemsPerCta for every histogram CTA of a feature tile so that
  // contiguous shares of items come out even; neighbouring items of a node that one CTA takes
  // are accumulated as one run (see make_items in partition.cu).
  //   items <= rows / item_rows + nodes <= 2 x (kItemsPerCta x CTAs) + rows / item_cap_ + nodes
  //   runs  <= CTAs + nodes + rows / item_cap_ (+ nodes: the short last item of a node)
  const int cols_tree = int(tp.colsample_bytree * F_);  // columns a tree samples (SampleFeatures)
  const int NT_tree = (std::max(1, cols_tree) + geo_.TW - 1) / geo_.TW;
  // fewer tiles get more CTAs each: size the item arrays for either geometry
  const int hist_ctas = std::max(hist_grid_x(1 << 30, geo_.NT), hist_grid_x(1 << 30, NT_tree));
  max_hist_items_ = 2 * kItemsPerCta * hist_ctas + int(n_ / item_cap_) + 2 * max_nodes_ + 8;
  max_hist_runs_ = hist_ctas + int(n_ / item_cap_) + 2 * max_nodes_ + 8;

  gp_ = GainParams{tp.min_leaf_size, tp.min_child_weight, tp.gamma_absolute, tp.gamma_relative,
                   tp.lambda,        tp.alpha,            tp.max_leaf_weight};

  // per-row state
  if (cfg.objective == kSoftMaxOneVsAll) {
    if (!d->d_labels.p) {
      d_label_.alloc(n_);
      ARB_CUDA(cudaMemcpyAsync(d_label_.p, d->labels.data(), n_, cudaMemcpyHostToDevice, s));
    }
  } else {
    if (!d->d_y.p) {
      d_y_.alloc(n_ * sizeof(float));
      ARB_CUDA(cudaMemcpyAsync(d_y_.p, d->y.data(), n_ * sizeof(float), cudaMemcpyHostToDevice, s));
    }
  }
  {  // one allocation for the per-row arrays
    struct Want {
      DevBuf *buf;
      size_t bytes;
    };
    // the histogram kernel of uint8 data reads the gradient records in list order
    const bool listed_grads = geo_.bin_bytes == 1 && geo_.TW == 32;
    const Want wants[] = {
      {&d_yhat_, n_ * K_ * sizeof(float)},
      {&d_grad_, n_ * K_ * (pair_ ? sizeof(float2) : sizeof(float))},
      {&d_list_, n_ * sizeof(unsigned)},
      {&d_list_grad_, listed_grads ? n_ * (pair_ ? sizeof(int2) : sizeof(int)) : 0},
      {&d_node_of_, n_ * sizeof(unsigned short)},
    };
    size_t total = 0;
    for (const Want &w : wants) total += (w.bytes + 255) / 256 * 256;
    d_rows_arena_.alloc(total);
    size_t at = 0;
    for (const Want &w : wants) {
      if (w.bytes) w.buf->view(static_cast<char *>(d_rows_arena_.p) + at, w.bytes);
      at += (w.bytes + 255) / 256 * 256;
    }
  }
  // garden.cu:105: y_hat starts at IntoInternal(initial_y)
  launch_fill(d_yhat_.as<float>(), n_ * K_, g->InternalInitialY(), s);
  trace.lap("per-row state");
  // level state
  {
    const size_t chunk_rows = d->out_of_core ? size_t(cfg.internal.chunk_rows) : n_;
    for (size_t b = 0; b < n_; b += chunk_rows)
      chunks_.push_back(Chunk{b, std::min(chunk_rows, n_ - b), nullptr});
  }
  // the small per-level arrays share one allocation (a cudaMalloc costs far more than they do)
  {
    struct Want {
      DevBuf *buf;
      size_t bytes;
    };
    const Want wants[] = {
      {&d_node_begin_, chunks_.size() * size_t(levels_ + 1) * nb_stride_ * sizeof(unsigned)},
      {&d_rec_, size_t(levels_) * max_nodes_ * sizeof(NodeRec)},
      {&d_keys_, max_nodes_ * (sizeof(unsigned long long) + sizeof(unsigned))},
      {&d_qs_, sizeof(QuantScale)},
      {&d_leaf_w_, 2 * max_nodes_ * sizeof(float)},
      {&d_active_, size_t(levels_) * F_},
      {&d_fsize_, F_ * sizeof(int)},
      {&d_cat_candidates_, F_ * sizeof(int)},
      {&d_hist_items_, max_hist_items_ * sizeof(WorkItem)},
      {&d_counters_, sizeof(int)},
      {&d_first_, (max_nodes_ + 2) * sizeof(int)},
      {&d_slot_first_, (max_nodes_ + 2) * sizeof(int)},
      {&d_item_slot_, (2 * size_t(max_hist_items_) + 2) * sizeof(int)},
      {&d_built_, max_nodes_ * sizeof(int)},
      {&d_scratch_, 3 * size_t(max_nodes_ + 1) * sizeof(unsigned)},
      {&d_list_base_, max_nodes_ * sizeof(unsigned)},
      {&d_cursor_, size_t(max_nodes_) * kCounterStride * sizeof(unsigned)},
      {&d_child_count_, size_t(max_nodes_) * kCounterStride * sizeof(unsigned)},
    };
    size_t total = 0;
    for (const Want &w : wants) total += (w.bytes + 255) / 256 * 256;
    d_arena_.alloc(total);
    ARB_CUDA(cudaMemsetAsync(d_arena_.p, 0, total, s));  // node_begin, rec and qs start as zeros
    size_t at = 0;
    for (const Want &w : wants) {
      w.buf->view(static_cast<char *>(d_arena_.p) + at, w.bytes);
      at += (w.bytes + 255) / 256 * 256;
    }
  }
  for (size_t c = 0; c < chunks_.size(); ++c) {
    const unsigned root[2] = {0u, unsigned(chunks_[c].rows)};
    ARB_CUDA(cudaMemcpyAsync(node_begin(int(c), 0), root, sizeof root, cudaMemcpyHostToDevice, s));
  }
  ARB_CHECK(int(d->fsize.size()) == F_ && int(d->cat_candidates.size()) == F_, "feature tables have the wrong size");
  ARB_CUDA(cudaMemcpyAsync(d_fsize_.p, d->fsize.data(), F_ * sizeof(int), cudaMemcpyHostToDevice, s));
  ARB_CUDA(cudaMemcpyAsync(d_cat_candidates_.p, d->cat_candidates.data(), F_ * sizeof(int), cudaMemcpyHostToDevice, s));
  const size_t level_hist_bytes = size_t(max_nodes_) * geo_.NT * kHistWords * 2 * sizeof(long long);
  d_hist_[0].alloc(level_hist_bytes);
  d_hist_[1].alloc(level_hist_bytes);
  d_partials_.alloc(size_t(max_hist_runs_) * geo_.NT * 2 * kHistWords * sizeof(int));
  const bool sharded = g->allreduce != nullptr;
  const size_t compact_bytes = size_t(std::max(1, max_nodes_ / 2)) * geo_.NT * kHistWords * 2 * sizeof(long long);
  // made here, not inside a round: an allocation that fails between two collectives would
  // leave the other ranks waiting inside theirs
  if (sharded && std::getenv("ARBORETUM_NO_PEER_EXCHANGE") == nullptr) {
    // what the ranks exchange per level: the built nodes' histograms (with the subtraction
    // trick one child per parent below the root), for every histogram set
    const size_t root_bytes = size_t(geo_.NT) * kHistWords * 2 * sizeof(long long);
    const size_t most = cfg.internal.use_hist_subtraction_trick ? std::max(compact_bytes, root_bytes) : level_hist_bytes;
    xchg_ = PeerExchange::Acquire((count_plane_ ? 2 : 1) * most, g->shards, s);
    if (xchg_) h_xchg_status_.alloc(sizeof(int));
    g->peer_exchange = xchg_ != nullptr;
  }
  if (sharded && cfg.internal.use_hist_subtraction_trick && !xchg_) d_compact_.alloc(compact_bytes);
  if (count_plane_) {
    d_ones_.alloc(n_ * sizeof(int));
    launch_fill_u32(d_ones_.as<unsigned>(), n_, 1u, s);
    d_cnt_hist_[0].alloc(level_hist_bytes);
    d_cnt_hist_[1].alloc(level_hist_bytes);
    if (sharded && cfg.internal.use_hist_subtraction_trick && !xchg_) d_compact_cnt_.alloc(compact_bytes);
  }
  round_rec_.resize(K_);
  round_nb_.resize(K_);
  pb_.hist_items = d_hist_items_.as<WorkItem>();
  pb_.n_hist_items = d_counters_.as<int>();
  pb_.hist_item_first = d_first_.as<int>();
  pb_.item_slot = d_item_slot_.as<int>();
  pb_.slot_first = d_slot_first_.as<int>();
  pb_.built_child = d_built_.as<int>();
  pb_.list_base = d_list_base_.as<unsigned>();
  pb_.cursor = d_cursor_.as<unsigned>();
  pb_.scratch_begin = d_scratch_.as<unsigned>();
  pb_.scratch_len = d_scratch_.as<unsigned>() + (max_nodes_ + 1);
  pb_.scratch_node = reinterpret_cast<int *>(d_scratch_.as<unsigned>() + 2 * (max_nodes_ + 1));
  pb_.right_count = d_child_count_.as<unsigned>();
  pb_.split_scratch = d_keys_.as<unsigned>();
  pb_.split_scratch_words = int(d_keys_.bytes / sizeof(unsigned));
  trace.lap("level buffers");
  {  // one pinned allocation for the three read-back buffers
    const size_t a = (d_rec_.bytes + 255) / 256 * 256, b = (d_leaf_w_.bytes + 255) / 256 * 256;
    h_arena_.alloc(a + b + d_node_begin_.bytes);
    h_rec_.view(h_arena_.p, d_rec_.bytes);
    h_leaf_w_.view(static_cast<char *>(h_arena_.p) + a, d_leaf_w_.bytes);
    h_node_begin_.view(static_cast<char *>(h_arena_.p) + a + b, d_node_begin_.bytes);
  }
  active_fids_.resize(F_);
  active_host_.resize(size_t(levels_) * F_);
  ARB_CUDA(cudaStreamSynchronize(s));
  trace.lap("pinned read-back buffers");
  if (!d->out_of_core) {
    chunks_[0].resident = d->d_bins.as<unsigned char>();
    // a tree that samples its columns: histograms over a side-by-side copy of those columns,
    // when that saves feature tiles and the copy fits (ARBORETUM_NO_COLUMN_COPY turns it off)
    const int cols_t = int(tp.colsample_bytree * F_);
    const int NT_t = (std::max(1, cols_t) + geo_.TW - 1) / geo_.TW;
    size_t free_b = 0;
    ARB_CUDA(dev_available(&free_b));
    const size_t pitch_t = DataMatrix::PitchFor(std::max(1, cols_t), geo_.bin_bytes);
    if (cols_t >= 1 && NT_t < geo_.NT && chunks_.size() == 1 && g->shards.world <= 1 && !g->allreduce &&
        n_ * pitch_t < free_b / 2 && std::getenv("ARBORETUM_NO_COLUMN_COPY") == nullptr) {
      sampled_cols_ = true;
      d_bins_tree_.alloc(n_ * pitch_t);
      d_fmap_.alloc(size_t(cols_t) * sizeof(int));
      fmap_host_.resize(cols_t);
      geo_tree_ = geo_;
      geo_tree_.bins = d_bins_tree_.as<unsigned char>();
      geo_tree_.pitch = pitch_t;
      geo_tree_.F = cols_t;
      geo_tree_.NT = NT_t;
      geo_tree_.bins_cm = nullptr;
      geo_tree_.cm_rows = 0;
      // uint8 tiles of 32 features: the copy is kept tile by tile, so that a tile's histogram
      // reads rows that lie back to back (in a row-major matrix of many tiles every row of a
      // tile is a 32-byte island)
      if (geo_.TW == 32 && NT_t > 1 && geo_.cm_rows == n_ &&
          compact_columns_tile_major_ok(geo_.bin_bytes, n_, geo_.bins_cm)) {
        geo_tree_.tile_stride = n_ * 32;
        geo_tree_.pitch = 32;
      }
    }
  } else {
    // as many leading chunks as fit stay in HBM; the rest cycle through two buffers
    const size_t chunk_bytes = chunks_[0].rows * d->pitch;
    int resident = cfg.internal.resident_chunks;
    if (resident < 0) {
      size_t free_b = 0;
      ARB_CUDA(dev_available(&free_b));
      const size_t budget = free_b / 10 * 8;
      // two padded staging buffers, and two unpadded ones where the host rows go without padding
      const size_t staging = 2 * chunk_bytes + (d->host_pitch != d->pitch ? 2 * chunks_[0].rows * d->host_pitch : 0);
      resident = budget > staging ? int((budget - staging) / chunk_bytes) : 0;
    }
    resident = std::min<int>(resident, int(chunks_.size()));
    size_t resident_rows = 0;
    for (int c = 0; c < resident; ++c) resident_rows += chunks_[c].rows;
    const bool tight_rows = d->host_pitch != d->pitch;
    if (resident_rows) {
      d_resident_.alloc(resident_rows * d->pitch);
      if (!tight_rows) {
        ARB_CUDA(cudaMemcpyAsync(d_resident_.p, d->h_bins.p, resident_rows * d->pitch,
                                 cudaMemcpyHostToDevice, s));
      } else {  // a slab of unpadded rows at a time, padded into place
        const size_t slab = std::min<size_t>(resident_rows, size_t(1) << 24);
        DevBuf d_slab;
        d_slab.alloc(slab * d->host_pitch);
        for (size_t first = 0; first < resident_rows; first += slab) {
          const size_t count = std::min(slab, resident_rows - first);
          ARB_CUDA(cudaMemcpyAsync(d_slab.p, d->h_bins.as<unsigned char>() + first * d->host_pitch,
                                   count * d->host_pitch, cudaMemcpyHostToDevice, s));
          launch_pad_rows(d_slab.as<unsigned char>(), int(d->host_pitch), count,
                          d_resident_.as<unsigned char>() + first * d->pitch, d->pitch, s);
        }
        ARB_CUDA(cudaStreamSynchronize(s));  // the slab goes out of scope
      }
      for (int c = 0; c < resident; ++c)
        chunks_[c].resident = d_resident_.as<unsigned char>() + chunks_[c].begin * d->pitch;
    }
    for (size_t c = resident; c < chunks_.size(); ++c) streamed_.push_back(int(c));
    if (!streamed_.empty()) {
      d_stage_[0].alloc(chunk_bytes);
      d_stage_[1].alloc(chunk_bytes);
      if (tight_rows) {
        d_stage_raw_[0].alloc(chunks_[0].rows * d->host_pitch);
        d_stage_raw_[1].alloc(chunks_[0].rows * d->host_pitch);
      }
      ARB_CUDA(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
      for (int i = 0; i < 2; ++i) {
        ARB_CUDA(cudaEventCreateWithFlags(&stage_ready_[i], cudaEventDisableTiming));
        ARB_CUDA(cudaEventCreateWithFlags(&stage_free_[i], cudaEventDisableTiming));
      }
    }
    ARB_CUDA(cudaStreamSynchronize(s));
  }
}

Builder::~Builder() {
  if (events_made_) {
    for (auto &e : ev_) cudaEventDestroy(e);
    for (auto &e : ev_hist_) cudaEventDestroy(e);
    for (auto &e : ev_tree_) cudaEventDestroy(e);
  }
  if (copy_stream_) {
    cudaStreamSynchronize(copy_stream_);
    for (int i = 0; i < 2; ++i) {
      cudaEventDestroy(stage_ready_[i]);
      cudaEventDestroy(stage_free_[i]);
    }
    cudaStreamDestroy(copy_stream_);
  }
}

// Copy the next chunk of the endless cyclic visiting sequence into its staging buffer.
void Builder::IssueCopy() {
  const Chunk &ch = chunks_[streamed_[issued_ % streamed_.size()]];
  const int buf = int(issued_ & 1);
  ARB_CUDA(cudaStreamWaitEvent(copy_stream_, stage_free_[buf], 0));  // kernels done with it
  const size_t hp = data->host_pitch;
  if (hp == data->pitch) {
    ARB_CUDA(cudaMemcpyAsync(d_stage_[buf].p, data->h_bins.as<unsigned char>() + ch.begin * hp, ch.rows * hp,
                             cudaMemcpyHostToDevice, copy_stream_));
  } else {  // unpadded rows cross the link; a kernel on the copy stream pads them
    ARB_CUDA(cudaMemcpyAsync(d_stage_raw_[buf].p, data->h_bins.as<unsigned char>() + ch.begin * hp,
                             ch.rows * hp, cudaMemcpyHostToDevice, copy_stream_));
    launch_pad_rows(d_stage_raw_[buf].as<unsigned char>(), int(hp), ch.rows, d_stage_[buf].as<unsigned char>(),
                    data->pitch, copy_stream_);
  }
  ARB_CUDA(cudaEventRecord(stage_ready_[buf], copy_stream_));
  if (g_->profile) g_->times.h2d_bytes += double(ch.rows * hp);
  ++issued_;
}

// Device address of a chunk's bins for the kernels about to be enqueued; streamed
// chunks must be visited in the cyclic order of `streamed_`.
const unsigned char *Builder::Acquire(int chunk) {
  if (chunks_[chunk].resident) return chunks_[chunk].resident;
  ARB_CHECK(streamed_[consumed_ % streamed_.size()] == chunk, "row chunks visited out of order");
  while (issued_ <= consumed_) IssueCopy();
  if (issued_ == consumed_ + 1) IssueCopy();  // the next chunk travels while this one is used
  const int buf = int(consumed_ & 1);
  ARB_CUDA(cudaStreamWaitEvent(g_->stream, stage_ready_[buf], 0));
  return d_stage_[buf].as<unsigned char>();
}

void Builder::Release(int chunk) {
  if (chunks_[chunk].resident) return;
  ARB_CUDA(cudaEventRecord(stage_free_[int(consumed_ & 1)], g_->stream));
  ++consumed_;
}

// the profiling events are made on first use: two hundred cudaEventCreate calls are
// not free, and most trainings never profile
void Builder::EnsureEvents() {
  if (events_made_) return;
  for (auto &e : ev_) ARB_CUDA(cudaEventCreate(&e));
  for (auto &e : ev_hist_) ARB_CUDA(cudaEventCreate(&e));
  for (auto &e : ev_tree_) ARB_CUDA(cudaEventCreate(&e));
  events_made_ = true;
}

void Builder::UpdateGrad() {  // objective.cu:28-56
  cudaStream_t s = g_->stream;
  if (g_->profile) EnsureEvents();
  if (g_->profile) ARB_CUDA(cudaEventRecord(ev_[0], s));
  // targets uploaded with the matrix are read where they are (a later ASetY is seen too)
  const float *y = data->d_y.p ? data->d_y.as<float>() : d_y_.as<float>();
  const unsigned char *labels = data->d_labels.p ? data->d_labels.as<unsigned char>() : d_label_.as<unsigned char>();
  // pass 1: the round's largest |gradient| and hessian (they fix the fixed-point scale)
  launch_gradients(g_->cfg.objective, K_, n_, y, labels, d_yhat_.as<float>(), d_grad_.p,
                   d_qs_.as<QuantScale>(), false, s, row_offset_, round_, qb_);
  // row shards must share one fixed-point scale: take the maxima over all ranks
  if (xchg_)
    xchg_->AllMax(&d_qs_.as<QuantScale>()->max_g_bits, 2, s);
  else if (g_->allreduce_max &&
           g_->allreduce_max(g_->allreduce_ctx, &d_qs_.as<QuantScale>()->max_g_bits, 2, s) != 0)
    throw std::runtime_error("gradient-scale allreduce failed");
  // reg:linear targets may have outliers: the scale also looks at how many gradients come
  // near the largest one (see QuantScale); row shards agree on the coarsest scale
  const bool tails = g_->cfg.objective == kLinearRegression;
  if (tails) launch_gradient_tails(n_, y, d_yhat_.as<float>(), d_qs_.as<QuantScale>(), s);
  if (tails && g_->allreduce_max) {
    launch_finish_scales(d_qs_.as<QuantScale>(), K_, qb_, pair_, s, true, 1);
    if (xchg_)
      xchg_->AllMax(&d_qs_.as<QuantScale>()->neg_s, 1, s);
    else if (g_->allreduce_max(g_->allreduce_ctx, &d_qs_.as<QuantScale>()->neg_s, 1, s) != 0)
      throw std::runtime_error("gradient-scale allreduce failed");
    launch_finish_scales(d_qs_.as<QuantScale>(), K_, qb_, pair_, s, true, 2);
  } else {
    launch_finish_scales(d_qs_.as<QuantScale>(), K_, qb_, pair_, s, tails, 0);
  }
  // pass 2: the gradients as fixed-point integers
  launch_gradients(g_->cfg.objective, K_, n_, y, labels, d_yhat_.as<float>(), d_grad_.p,
                   d_qs_.as<QuantScale>(), true, s, row_offset_, round_, qb_);
  ++round_;
  if (g_->profile) {
    ARB_CUDA(cudaEventRecord(ev_[1], s));
    ARB_CUDA(cudaEventSynchronize(ev_[1]));
    float ms;
    ARB_CUDA(cudaEventElapsedTime(&ms, ev_[0], ev_[1]));
    g_->times.grad += ms;
  }
}

// Training continues a model that was loaded (ALoadModel) or grown on another matrix: the
// predictions start from what the existing trees give on this matrix's raw values, and the
// feature-sampling engine and the round counter stand where they would after growing those
// trees here.  (The reference restores the trees only: a builder made after `load` starts
// from initial_y, garden.cu:585-606,659-677.)
void Builder::Resume() {
  Garden *g = g_;
  cudaStream_t s = g->stream;
  ARB_CHECK(g->max_fid < data->cols(), "the model tests a feature the matrix does not have");
  g->SyncForest();
  const PackedTree pt{g->d_fid.as<int>(), g->d_thr.as<float>(), g->d_w.as<float>(), g->d_label.as<int>(),
                      g->d_category.as<unsigned>()};
  RowFeeder feed(data);
  for (size_t first = 0; first < n_; first += feed.chunk) {
    const size_t count = std::min(feed.chunk, n_ - first);
    const float *X = feed.load(first, count, s);
    launch_predict(X, count, data->cols_dense, pt, 0, int(g->trees.size()), int(g->cfg.tree.depth),
                   d_yhat_.as<float>() + first, s, n_, feed.categories(first), data->cols_cat);
    ARB_CUDA(cudaStreamSynchronize(s));
  }
  for (size_t t = 0; t < g->trees.size(); ++t) SampleFeatures();
  round_ = unsigned(g->trees.size() / size_t(K_));
}

// Feature sampling of one tree (garden.cu:126-165,252-253 of the reference): the same
// shuffles of the same engine in the same order, also when both ratios are 1.
void Builder::SampleFeatures() {
  const TreeParam &tp = g_->cfg.tree;
  int take = int(tp.colsample_bytree * F_);
  if (take == 0) throw std::runtime_error("colsample_bytree is too small");
  take = int(tp.colsample_bytree * tp.colsample_bylevel * F_);
  if (take == 0) throw std::runtime_error("colsample_bytree and colsample_bylevel are too small");
  for (int i = 0; i < F_; ++i) active_fids_[i] = i;
  std::shuffle(active_fids_.begin(), active_fids_.end(), rnd_);
  std::fill(active_host_.begin(), active_host_.end(), 0);
  for (int l = 0; l < levels_; ++l) {
    std::shuffle(active_fids_.begin(), active_fids_.begin() + int(tp.colsample_bytree * F_), rnd_);
    const unsigned take_l = unsigned(tp.colsample_bylevel * tp.colsample_bytree * F_);
    for (unsigned j = 0; j < take_l && j < unsigned(F_); ++j)
      active_host_[size_t(l) * F_ + active_fids_[j]] = 1;
  }
}

void Builder::GrowTree(int label, Tree *tree) {  // garden.cu:167-197
  const auto host_t0 = std::chrono::steady_clock::now();
  const Configuration &cfg = g_->cfg;
  const TreeParam &tp = cfg.tree;
  cudaStream_t s = g_->stream;
  const bool prof = g_->profile;
  if (prof) EnsureEvents();
  QuantScale *qs = d_qs_.as<QuantScale>();
  const void *grad = static_cast<const char *>(d_grad_.p) +
                     size_t(label) * n_ * (pair_ ? sizeof(float2) : sizeof(float));

  SampleFeatures();
  ARB_CUDA(cudaMemcpyAsync(d_active_.p, active_host_.data(), active_host_.size(),
                           cudaMemcpyHostToDevice, s));
  if (sampled_cols_) {
    // the tree's columns (the head of the shuffled list; the per-level shuffles only permute
    // it), in feature order so that ties between columns fall like ties between features
    fmap_host_.assign(active_fids_.begin(), active_fids_.begin() + fmap_host_.size());
    std::sort(fmap_host_.begin(), fmap_host_.end());
    // pageable source: the call returns once the ids are staged, so the vector may change again
    ARB_CUDA(cudaMemcpyAsync(d_fmap_.p, fmap_host_.data(), fmap_host_.size() * sizeof(int),
                             cudaMemcpyHostToDevice, s));
    launch_compact_columns(geo_.bins, geo_.pitch, geo_.bin_bytes, n_, d_fmap_.as<int>(), geo_tree_.F,
                           d_bins_tree_.as<unsigned char>(), DataMatrix::PitchFor(geo_tree_.F, geo_.bin_bytes), s,
                           geo_.cm_rows == n_ ? geo_.bins_cm : nullptr, geo_tree_.tile_stride != 0);
  }
  if (prof) ARB_CUDA(cudaEventRecord(ev_tree_[0], s));
  // a tree that threw half way (an exchange that failed) leaves the cyclic visiting order of
  // the streamed chunks out of step: start over from the first one
  if (!streamed_.empty() && consumed_ % streamed_.size() != 0) {
    ARB_CUDA(cudaStreamSynchronize(copy_stream_));
    ARB_CUDA(cudaStreamSynchronize(s));
    issued_ = consumed_ = 0;
  }

  const bool use_trick = cfg.internal.use_hist_subtraction_trick;
  const int n_chunks = int(chunks_.size());
  const bool multi = n_chunks > 1;  // row chunks add their histograms like GPUs do
  const bool by_hessian = g_->allreduce != nullptr || multi;
  const size_t gsz = pair_ ? sizeof(float2) : sizeof(float);
  const int n_sets = count_plane_ ? 2 : 1;  // histogram sets: (g, h) sums, then row counts
  int ev = 0;
  auto mark = [&]() {
    if (prof && !multi) ARB_CUDA(cudaEventRecord(ev_[ev], s));
    ++ev;
  };
  // events per level: 0 begin, 1 descend done, 2 plan + lists done, 3 histogram done,
  // 4 allreduce done, 5 subtraction done, 6 split search done
  for (int l = 0; l < levels_; ++l) {
    const int L = 1 << l;
    const bool trick_level = use_trick && l > 0;
    const int n_build = trick_level ? L / 2 : L;
    // Row shards sum only what they built: below the root that is one child per parent, so
    // the exchanged buffer holds those alone and the siblings follow from the parents after
    // the exchange.
    const bool compact = trick_level && g_->allreduce != nullptr;
    // words of one histogram set that the ranks exchange at this level
    const int NTh = sampled_cols_ ? geo_tree_.NT : geo_.NT;  // feature tiles of the histograms
    const size_t xwords = size_t(compact ? n_build : L) * NTh * kHistWords * 2;
    long long *hist[2], *reduce_to[2];
    const long long *parent_hist[2];
    for (int k = 0; k < n_sets; ++k) {
      DevBuf *levels = k == 0 ? d_hist_ : d_cnt_hist_;
      hist[k] = levels[l & 1].as<long long>();
      parent_hist[k] = l > 0 ? levels[(l - 1) & 1].as<long long>() : nullptr;
      if (xchg_)  // summed where the peers will read it; the sets lie back to back
        reduce_to[k] = xchg_->send_buffer() + size_t(k) * xwords;
      else
        reduce_to[k] = compact ? (k == 0 ? d_compact_ : d_compact_cnt_).as<long long>() : hist[k];
      if (multi)
        ARB_CUDA(cudaMemsetAsync(reduce_to[k], 0, size_t(compact ? n_build : L) * NTh * kHistWords * 2 * sizeof(long long), s));
    }
    for (int c = 0; c < n_chunks; ++c) {
      const Chunk &ch = chunks_[c];
      const bool last = c + 1 == n_chunks;
      Geometry geo = geo_;
      geo.bins = Acquire(c);
      const size_t rows = ch.rows;
      const void *grad_c = static_cast<const char *>(grad) + ch.begin * gsz;
      unsigned short *node_of = d_node_of_.as<unsigned short>() + ch.begin;
      unsigned *list = d_list_.as<unsigned>() + ch.begin;
      if (c == 0) mark();
      void *list_grad = d_list_grad_.p ? static_cast<char *>(d_list_grad_.p) + ch.begin * gsz : nullptr;
      if (l > 0) {  // every row of the chunk steps from its node of level l - 1 to a child
        DescendLaunch d;
        d.geo = geo;
        d.rec = rec(l - 1);
        d.L = L / 2;
        d.node_of = node_of;
        d.child_count = d_child_count_.as<unsigned>();
        d.leaf_w = nullptr;
        d.yhat = nullptr;
        d.n = rows;
        launch_descend(d, s);
      }
      if (last) mark();
      // rows scanned this level: all at the root, at most half with the trick (the hessian
      // rule of multi-GPU / multi-chunk runs has no such bound)
      const bool half = trick_level && !by_hessian;
      const size_t level_rows = half ? rows / 2 + 1 : rows;
      // the histogram pass reads the tree's side-by-side columns where there are any
      const Geometry &hgeo = sampled_cols_ ? geo_tree_ : geo;
      const int hist_ctas = hist_grid_x(1 << 30, hgeo.NT);
      int item_rows = item_cap_;  // the largest power-of-two share of a plane's rows that gives
                                  // every CTA about kItemsPerCta items
      while (item_rows > kMinItemRows && level_rows / size_t(item_rows) < size_t(kItemsPerCta) * hist_ctas) item_rows >>= 1;
      LevelPlanLaunch pl;
      pl.child_count = l > 0 ? d_child_count_.as<unsigned>() : nullptr;
      pl.parent_begin = l > 0 ? node_begin(c, l - 1) : nullptr;
      pl.node_begin = node_begin(c, l);
      pl.parent_rec = l > 0 ? rec(l - 1) : nullptr;
      pl.L = L;
      pl.item_rows = item_rows;
      pl.hist_grid_x = hist_ctas;
      pl.items_per_run = item_cap_ / item_rows;
      pl.use_trick = use_trick;
      pl.by_hessian = by_hessian;
      pl.pb = pb_;
      pl.max_items = max_hist_items_;
      launch_plan_level(pl, s);
      if (l > 0) launch_gather_lists(node_of, rows, L, pb_, list, grad_c, list_grad, pair_, s);
      if (last) mark();
      for (int k = 0; k < n_sets; ++k) {
        HistLaunch h;
        h.geo = hgeo;
        h.rowid = l == 0 ? nullptr : list;
        // the count set: every row's "gradient" is 1 and the hessian plane of the
        // reg:linear kernel counts the rows
        h.grad = k == 0 ? grad_c : static_cast<const void *>(d_ones_.as<int>() + ch.begin);
        h.pair = k == 0 ? pair_ : false;
        h.items = pb_.hist_items;
        h.n_items = pb_.n_hist_items;
        h.item_slot = pb_.item_slot;
        h.grid_x = hist_ctas;
        h.max_items = int(std::min<size_t>(max_hist_items_, level_rows / item_rows + n_build + 1));
        h.partials = d_partials_.as<int>();
        h.list_grad = (l == 0 || k > 0) ? nullptr : list_grad;
        if (has_row_map_ && hgeo.bins == geo_.bins) {
          h.row_map = &row_map_;
          h.status = d_hist_status_.as<int>();
        }
        launch_hist(h, s);
        if (prof && !multi && k == 0) ARB_CUDA(cudaEventRecord(ev_hist_[l], s));
        ReduceLaunch rd;
        rd.partials = d_partials_.as<int>();
        rd.item_first = pb_.slot_first;  // the planes of a node's runs
        rd.build_node = compact ? nullptr : pb_.scratch_node;
        rd.n_build = n_build;
        rd.NT = hgeo.NT;
        rd.level_hist = reduce_to[k];
        rd.parent_hist = parent_hist[k];
        rd.subtract = trick_level && !g_->allreduce && !multi;
        rd.level_nodes = compact ? n_build : L;
        rd.built_child = pb_.built_child;
        rd.accumulate = multi;
        launch_reduce(rd, s);
      }
      Release(c);
    }
    mark();
    if (xchg_) {
      xchg_->AllReduce(size_t(n_sets) * xwords, s);
    } else if (g_->allreduce) {
      for (int k = 0; k < n_sets; ++k)
        if (g_->allreduce(g_->allreduce_ctx, reduce_to[k], xwords, s) != 0)
          throw std::runtime_error("histogram allreduce failed");
    }
    mark();
    for (int k = 0; k < n_sets; ++k) {
      const long long *summed = xchg_ ? xchg_->result_buffer() + size_t(k) * xwords : reduce_to[k];
      if (xchg_ && !compact)  // a whole level (the root, or no subtraction): straight to its buffer
        ARB_CUDA(cudaMemcpyAsync(hist[k], summed, xwords * sizeof(long long), cudaMemcpyDeviceToDevice, s));
      if (compact)
        launch_expand(summed, parent_hist[k], hist[k], pb_.built_child, L / 2, NTh, s);
      else if (trick_level && multi)
        launch_subtract(hist[k], parent_hist[k], pb_.built_child, L / 2, NTh, s);
    }
    mark();
    SplitLaunch sp;
    sp.geo = sampled_cols_ ? geo_tree_ : geo_;
    sp.feature_map = sampled_cols_ ? d_fmap_.as<int>() : nullptr;
    sp.hist = hist[0];
    sp.count_hist = count_plane_ ? hist[1] : nullptr;
    sp.node_begin = node_begin(0, l);
    sp.feature_active = d_active_.as<unsigned char>() + size_t(l) * F_;
    sp.feature_size = d_fsize_.as<int>();
    sp.cat_candidates = data->cols_cat > 0 ? d_cat_candidates_.as<int>() : nullptr;
    sp.keys = d_keys_.as<unsigned long long>();
    sp.max_nodes = max_nodes_;
    sp.rec = rec(l);
    sp.parent_rec = l > 0 ? rec(l - 1) : nullptr;
    sp.qs = qs;
    sp.gp = gp_;
    sp.pair = pair_;
    sp.L = L;
    launch_split(sp, s);
    mark();
  }
  // ---- leaves and prediction update (garden.cu:487-503, :45-76) -----------------
  LeafLaunch lf;
  lf.last_rec = rec(levels_ - 1);
  lf.L = max_nodes_;
  lf.leaf_w = d_leaf_w_.as<float>();
  lf.qs = qs;
  lf.mcw = tp.min_child_weight;
  lf.mls = tp.min_leaf_size;
  lf.lambda = tp.lambda;
  lf.alpha = tp.alpha;
  lf.mlw = tp.max_leaf_weight;
  lf.eta = tp.eta;
  lf.pair = pair_;
  lf.counts = count_plane_;
  launch_leaf_weights(lf, s);
  for (int c = 0; c < n_chunks; ++c) {  // the tree walk needs the bins once more
    Geometry geo = geo_;
    geo.bins = Acquire(c);
    float *yhat_c = d_yhat_.as<float>() + size_t(label) * n_ + chunks_[c].begin;
    // one more step down from the last level, straight into the prediction
    DescendLaunch d;
    d.geo = geo;
    d.rec = rec(levels_ - 1);
    d.L = max_nodes_;
    d.node_of = d_node_of_.as<unsigned short>() + chunks_[c].begin;
    d.child_count = nullptr;
    d.leaf_w = d_leaf_w_.as<float>();
    d.yhat = yhat_c;
    d.n = chunks_[c].rows;
    launch_descend(d, s);
    Release(c);
  }
  mark();
  if (prof) ARB_CUDA(cudaEventRecord(ev_tree_[1], s));
  ARB_CUDA(cudaMemcpyAsync(h_rec_.p, d_rec_.p, d_rec_.bytes, cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaMemcpyAsync(h_leaf_w_.p, d_leaf_w_.p, d_leaf_w_.bytes, cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaMemcpyAsync(h_node_begin_.p, d_node_begin_.p, d_node_begin_.bytes,
                           cudaMemcpyDeviceToHost, s));
  if (xchg_) ARB_CUDA(cudaMemcpyAsync(h_xchg_status_.p, xchg_->device_status(), sizeof(int), cudaMemcpyDeviceToHost, s));
  if (has_row_map_)
    ARB_CUDA(cudaMemcpyAsync(h_hist_status_.p, d_hist_status_.p, sizeof(int), cudaMemcpyDeviceToHost, s));
  if (g_->allreduce && !xchg_ && g_->comm_check) {
    // Row shards over a collective library: a rank that died leaves its peers inside a
    // collective for good.  The host therefore does not block in the synchronisation: it
    // polls the stream, asks the communicator for asynchronous errors meanwhile, and gives
    // up after a time limit (ARBORETUM_EXCHANGE_TIMEOUT_S, 300 s by default); either way the
    // communicator is aborted and the caller gets an error string.
    static const double limit_s = [] {
      const char *e = std::getenv("ARBORETUM_EXCHANGE_TIMEOUT_S");
      const double v = e ? std::atof(e) : 300.0;
      return v > 0 ? v : 300.0;
    }();
    cudaEvent_t done;
    ARB_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    ARB_CUDA(cudaEventRecord(done, s));
    const auto t0 = std::chrono::steady_clock::now();
    unsigned polls = 0;
    char msg[256] = "";
    for (;;) {
      const cudaError_t q = cudaEventQuery(done);
      if (q == cudaSuccess) break;
      if (q != cudaErrorNotReady) {
        cudaEventDestroy(done);
        ARB_CUDA(q);
      }
      if ((++polls & 255u) == 0u) {
        const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        const int give_up = waited > limit_s ? 1 : 0;
        if (g_->comm_check(g_->allreduce_ctx, give_up, msg, sizeof msg) != 0 || give_up) {
          cudaEventDestroy(done);
          cudaStreamSynchronize(s);  // the aborted collectives end
          cudaGetLastError();
          throw std::runtime_error(std::string("the exchange between the GPUs failed: ") +
                                   (msg[0] ? msg : "no answer from a peer within the time limit"));
        }
      } else {
        std::this_thread::yield();
      }
    }
    cudaEventDestroy(done);
  }
  const auto host_t1 = std::chrono::steady_clock::now();
  ARB_CUDA(cudaStreamSynchronize(s));
  {
    const auto host_t2 = std::chrono::steady_clock::now();
    g_->times.enqueue += std::chrono::duration<double, std::milli>(host_t1 - host_t0).count();
    g_->times.host_wait += std::chrono::duration<double, std::milli>(host_t2 - host_t1).count();
    g_->times.host_trees += 1;
  }
  if (has_row_map_ && *h_hist_status_.as<int>() != 0)
    throw std::runtime_error("a row gather of the histogram kernel did not arrive within its time limit: "
                             "the tree is incomplete");
  if (xchg_ && *h_xchg_status_.as<int>() != 0)
    throw std::runtime_error("a peer GPU did not answer within the time limit (exchange step " +
                             std::to_string(*h_xchg_status_.as<int>()) + "): the tree is incomplete");
  {  // per-level prefix counts of the whole data set = sums over the row chunks
    const size_t per_chunk = size_t(levels_ + 1) * nb_stride_;
    h_nb_total_.assign(per_chunk, 0u);
    const unsigned *all = h_node_begin_.as<unsigned>();
    for (int c = 0; c < n_chunks; ++c)
      for (size_t i = 0; i < per_chunk; ++i) h_nb_total_[i] += all[size_t(c) * per_chunk + i];
  }
  round_rec_[label].assign(h_rec_.as<NodeRec>(), h_rec_.as<NodeRec>() + size_t(levels_) * max_nodes_);
  round_nb_[label] = h_nb_total_;

  // ---- UpdateTree garden.cu:447-485 -----------------------------------------------
  const int depth = int(tp.depth);
  tree->depth = depth;
  tree->label = label;
  tree->nodes.assign((size_t(1) << depth) - 1, TreeNode());
  tree->weights.assign(size_t(1) << (depth - 1), 0.0f);
  const NodeRec *hrec = h_rec_.as<NodeRec>();
  const int H = data->hist_size;
  for (int l = 0; l < levels_; ++l) {
    const int L = 1 << l, offset = L - 1;
    for (int i = 0; i < L; ++i) {
      const NodeRec &r = hrec[size_t(l) * max_nodes_ + i];
      TreeNode &nd = tree->nodes[i + offset];
      if (r.fid >= 0) {
        nd.fid = r.fid;
        g_->max_fid = std::max(g_->max_fid, r.fid);
        nd.quantized = unsigned(r.bin);
        if (r.fid >= data->cols_dense) {  // one category against the rest
          nd.categorical = true;
          nd.category = data->cat_codes[size_t(r.fid - data->cols_dense)][size_t(r.bin)];
          nd.threshold = std::numeric_limits<float>::infinity();
          continue;
        }
        // a split on the last bin in use separates present from missing values
        const bool last_real = r.bin >= data->fsize[r.fid] - 1;
        nd.threshold = (r.bin >= H || last_real) ? std::numeric_limits<float>::infinity()
                                                 : data->thr[size_t(r.fid) * H + r.bin];
      } else {
        nd.fid = 0;
        nd.quantized = unsigned(-1);
        nd.threshold = std::numeric_limits<float>::infinity();
      }
    }
  }
  const float *hw = h_leaf_w_.as<float>();
  for (int i = 0; i < 2 * max_nodes_; ++i) tree->weights[i] = hw[i];

  if (prof) {
    float ms;
    ARB_CUDA(cudaEventElapsedTime(&ms, ev_tree_[0], ev_tree_[1]));
    g_->times.tree += ms;
  }
  if (prof && multi) g_->times.trees += 1;
  if (prof && !multi) {
    PhaseTimes &t = g_->times;
    const unsigned *hnb = h_nb_total_.data();
    int e = 0;
    auto span = [&](int a, int b) {
      float ms;
      ARB_CUDA(cudaEventElapsedTime(&ms, ev_[a], ev_[b]));
      return double(ms);
    };
    for (int l = 0; l < levels_; ++l) {
      t.partition += span(e, e + 1);
      t.plan += span(e + 1, e + 2);
      t.hist += span(e + 2, e + 3);
      {
        float ms;
        ARB_CUDA(cudaEventElapsedTime(&ms, ev_[e + 2], ev_hist_[l]));
        t.hist_kernel += double(ms);
      }
      t.allreduce += span(e + 3, e + 4);
      t.subtract += span(e + 4, e + 5);
      t.split += span(e + 5, e + 6);
      e += 7;
      // rows scanned by this level's histogram launch
      double rows = 0;
      const int L = 1 << l;
      const unsigned *nb = hnb + size_t(l) * nb_stride_;
      if (l == 0 || !use_trick) {
        rows = double(n_);
      } else {
        for (int p = 0; p < L / 2; ++p) {
          const unsigned ls = nb[2 * p + 1] - nb[2 * p], rs = nb[2 * p + 2] - nb[2 * p + 1];
          if (by_hessian) {
            const NodeRec &pr = hrec[size_t(l - 1) * max_nodes_ + p];
            rows += (pr.lh <= pr.th - pr.lh) ? ls : rs;
          } else {
            rows += std::min(ls, rs);
          }
        }
      }
      t.hist_rows += rows;
      const double hist_cols = sampled_cols_ ? double(geo_tree_.F) : double(F_);
      t.hist_features += hist_cols;
      t.hist_bytes += rows * (hist_cols * geo_.bin_bytes + (pair_ ? 8.0 : 4.0));
      t.hist_launches += 1;
    }
    t.update += span(e - 1, e);
    t.trees += 1;
  }
}

const NodeRec *BuilderView::host_rec(const Garden *g, int tree_in_round, int *max_nodes, int *levels) {
  ARB_CHECK(g->builder && !g->builder->round_rec_.back().empty(), "no tree has been grown yet");
  const int K = int(g->builder->round_rec_.size());
  ARB_CHECK(tree_in_round >= -1 && tree_in_round < K, "tree index out of range");
  *max_nodes = g->builder->max_nodes_;
  *levels = g->builder->levels_;
  return g->builder->round_rec_[tree_in_round < 0 ? K - 1 : tree_in_round].data();
}
const unsigned *BuilderView::host_node_begin(const Garden *g, int tree_in_round, int *stride) {
  ARB_CHECK(g->builder && !g->builder->round_nb_.back().empty(), "no tree has been grown yet");
  const int K = int(g->builder->round_nb_.size());
  ARB_CHECK(tree_in_round >= -1 && tree_in_round < K, "tree index out of range");
  *stride = g->builder->nb_stride_;
  return g->builder->round_nb_[tree_in_round < 0 ? K - 1 : tree_in_round].data();
}
void BuilderView::scales(Garden *g, QuantScale *out) {
  ARB_CHECK(g->builder, "no tree has been grown yet");
  ARB_CUDA(cudaMemcpy(out, g->builder->d_qs_.p, sizeof(QuantScale), cudaMemcpyDeviceToHost));
}
namespace {
// Device -> pageable host memory for large results.  A plain cudaMemcpy into memory the
// caller has just allocated spends most of its time in one thread that takes the page
// faults of the destination; here a few threads each bring their share through their own
// small pinned buffer (kept for the life of the process) and copy it out, so the faults
// and the copies run side by side with the DMA.
void copy_to_host(void *dst, const void *src_device, size_t bytes) {
  constexpr int kMaxThreads = 8;
  static const int kThreads =
    int(std::max(1u, std::min(unsigned(kMaxThreads), std::thread::hardware_concurrency() / 2)));
  constexpr size_t kPiece = size_t(2) << 20;
  if (bytes < 4 * kPiece) {
    ARB_CUDA(cudaMemcpy(dst, src_device, bytes, cudaMemcpyDeviceToHost));
    return;
  }
  static void *bounce[kMaxThreads] = {};
  for (int t = 0; t < kThreads; ++t)
    if (!bounce[t]) ARB_CUDA(cudaMallocHost(&bounce[t], kPiece));
  int device = 0;
  ARB_CUDA(cudaGetDevice(&device));
  const size_t pieces = (bytes + kPiece - 1) / kPiece;
  cudaError_t status[kMaxThreads];
  for (cudaError_t &e : status) e = cudaSuccess;
  std::vector<std::thread> pool;
  for (int t = 0; t < kThreads; ++t) {
    status[t] = cudaSuccess;
    pool.emplace_back([=, &status]() {
      cudaError_t e = cudaSetDevice(device);
      cudaStream_t st = nullptr;
      if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
      for (size_t p = size_t(t); p < pieces && e == cudaSuccess; p += kThreads) {
        const size_t off = p * kPiece, len = std::min(kPiece, bytes - off);
        e = cudaMemcpyAsync(bounce[t], static_cast<const char *>(src_device) + off, len,
                            cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e == cudaSuccess) std::memcpy(static_cast<char *>(dst) + off, bounce[t], len);
      }
      if (st) cudaStreamDestroy(st);
      status[t] = e;
    });
  }
  for (auto &th : pool) th.join();
  for (cudaError_t e : status) ARB_CUDA(e);
}
}  // namespace

bool BuilderView::exchange_clock(Garden *g, double ms[3], long long *exchanges, bool reset) {
  if (!g->builder || !g->builder->xchg_) return false;
  ARB_CUDA(cudaStreamSynchronize(g->stream));
  g->builder->xchg_->Clock(ms, exchanges, reset);
  return true;
}

void BuilderView::train_yhat(Garden *g, float *out) {
  ARB_CHECK(g->builder, "no tree has been grown yet");
  ARB_CUDA(cudaStreamSynchronize(g->stream));
  copy_to_host(out, g->builder->d_yhat_.p, g->builder->d_yhat_.bytes);
}

// ---------------------------------------------------------------------------
// Garden
// ---------------------------------------------------------------------------
Garden::Garden(const Configuration &c) : cfg(c) {
  // garden.cu:571-583: only these objectives exist (multi:softmax is this
  // build's completion of the reference's stub)
  if (cfg.objective != kLinearRegression && cfg.objective != kLogisticRegression &&
      cfg.objective != kSoftMaxOneVsAll)
    throw std::runtime_error("Unknown objective function " + std::to_string(cfg.objective));
  if (cfg.method != kHist)
    throw std::runtime_error("method 0 (exact) is not part of this build; use method 1 (hist)");
  if (cfg.objective == kSoftMaxOneVsAll && cfg.tree.labels_count < 2)
    throw std::runtime_error("multi:softmax needs tree.labels_count >= 2");
}

// The stream is made by the first call that needs the device, so that a Garden can be made,
// loaded and dumped on a host without one.
void Garden::EnsureStream() {
  if (stream) return;
  if (cfg.internal.device >= 0) ARB_CUDA(cudaSetDevice(cfg.internal.device));
  ARB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
}

void Garden::ReleaseBuilder() {
  delete builder;
  builder = nullptr;
}

Garden::~Garden() {
  delete builder;
  if (stream) cudaStreamDestroy(stream);
}

float Garden::InternalInitialY() const {  // objective.h:19,55-57
  const float v = cfg.tree.initial_y;
  if (cfg.objective == kLogisticRegression) return std::log(v / (1 - v));
  return v;
}

void Garden::GrowTree(DataMatrix *data, const float *grad) {
  (void)grad;  // custom gradients are ignored by the reference as well (garden.cu:609-614)
  EnsureStream();
  data->InitHist(cfg.internal.hist_size, cfg.internal.missing_bin, cfg.verbose.data, stream,
                 cfg.internal.chunk_rows, &shards);
  if (!builder) {
    builder = new Builder(this, data);
    if (!trees.empty()) builder->Resume();
  } else if (builder->data != data) {
    throw std::runtime_error("this Garden is already bound to another DMatrix");
  }
  builder->UpdateGrad();
  for (unsigned k = 0; k < cfg.tree.labels_count; ++k) {
    Tree t;
    builder->GrowTree(int(k), &t);
    trees.push_back(std::move(t));
  }
}

void Garden::SyncForest() {
  EnsureStream();
  if (forest_trees_on_device == trees.size()) return;
  const int depth = int(cfg.tree.depth);
  const size_t nodes = (size_t(1) << depth) - 1, leaves = size_t(1) << (depth - 1);
  std::vector<int> fid(trees.size() * nodes), label(trees.size());
  std::vector<unsigned> category(trees.size() * nodes);
  std::vector<float> thr(trees.size() * nodes), w(trees.size() * leaves);
  for (size_t t = 0; t < trees.size(); ++t) {
    ARB_CHECK(trees[t].depth == depth, "tree depth differs from the configuration");
    for (size_t i = 0; i < nodes; ++i) {
      fid[t * nodes + i] = trees[t].nodes[i].fid;
      thr[t * nodes + i] = trees[t].nodes[i].threshold;
      category[t * nodes + i] = trees[t].nodes[i].category;
    }
    std::copy(trees[t].weights.begin(), trees[t].weights.end(), w.begin() + t * leaves);
    label[t] = trees[t].label;
  }
  d_fid.alloc(fid.size() * sizeof(int));
  d_thr.alloc(thr.size() * sizeof(float));
  d_w.alloc(w.size() * sizeof(float));
  d_label.alloc(label.size() * sizeof(int));
  d_category.alloc(category.size() * sizeof(unsigned));
  ARB_CUDA(cudaMemcpyAsync(d_category.p, category.data(), d_category.bytes, cudaMemcpyHostToDevice, stream));
  ARB_CUDA(cudaMemcpyAsync(d_fid.p, fid.data(), d_fid.bytes, cudaMemcpyHostToDevice, stream));
  ARB_CUDA(cudaMemcpyAsync(d_thr.p, thr.data(), d_thr.bytes, cudaMemcpyHostToDevice, stream));
  ARB_CUDA(cudaMemcpyAsync(d_w.p, w.data(), d_w.bytes, cudaMemcpyHostToDevice, stream));
  ARB_CUDA(cudaMemcpyAsync(d_label.p, label.data(), d_label.bytes, cudaMemcpyHostToDevice, stream));
  ARB_CUDA(cudaStreamSynchronize(stream));
  forest_trees_on_device = trees.size();
}


// Garden::Predict garden.cu:643-657; n_rounds counts trees, like the reference
void Garden::Predict(DataMatrix *data, std::vector<float> &out, int n_rounds) {
  const int K = int(cfg.tree.labels_count);
  const size_t n = size_t(data->rows);
  ARB_CHECK(max_fid < data->cols(), "the model tests a feature the matrix does not have");
  out.resize(n * K);
  SyncForest();
  const int use = int(std::min<long long>(n_rounds, (long long)trees.size()));
  RowFeeder feed(data);
  DevBuf d_int, d_out;
  d_int.alloc(feed.chunk * K * sizeof(float));
  d_out.alloc(feed.chunk * K * sizeof(float));
  const PackedTree pt{d_fid.as<int>(), d_thr.as<float>(), d_w.as<float>(), d_label.as<int>(),
                      d_category.as<unsigned>()};
  for (size_t first = 0; first < n; first += feed.chunk) {
    const size_t count = std::min(feed.chunk, n - first);
    const float *X = feed.load(first, count, stream);
    launch_fill(d_int.as<float>(), count * K, InternalInitialY(), stream);
    launch_predict(X, count, data->cols_dense, pt, 0, use, int(cfg.tree.depth), d_int.as<float>(), stream, 0,
                   feed.categories(first), data->cols_cat);
    launch_link(cfg.objective, K, count, d_int.as<float>(), d_out.as<float>(), stream);
    ARB_CUDA(cudaMemcpyAsync(out.data() + first * K, d_out.p, count * K * sizeof(float),
                             cudaMemcpyDeviceToHost, stream));
    ARB_CUDA(cudaStreamSynchronize(stream));
  }
}

// Garden::UpdateByLastTree garden.cu:627-635: add the last round's trees to the
// matrix's accumulated prediction (kept on the device here)
void Garden::UpdateByLastTree(DataMatrix *data) {
  const int K = int(cfg.tree.labels_count);
  const size_t n = size_t(data->rows);
  ARB_CHECK(trees.size() >= size_t(K), "no tree has been grown yet");
  ARB_CHECK(max_fid < data->cols(), "the model tests a feature the matrix does not have");
  EnsureStream();
  if (!data->d_yhat.p || data->yhat_planes != K) {
    data->d_yhat.alloc(n * K * sizeof(float));
    data->yhat_planes = K;
    launch_fill(data->d_yhat.as<float>(), n * K, InternalInitialY(), stream);
  }
  SyncForest();
  RowFeeder feed(data);
  const PackedTree pt{d_fid.as<int>(), d_thr.as<float>(), d_w.as<float>(), d_label.as<int>(),
                      d_category.as<unsigned>()};
  DevBuf d_tmp;
  d_tmp.alloc(feed.chunk * K * sizeof(float));
  for (size_t first = 0; first < n; first += feed.chunk) {
    const size_t count = std::min(feed.chunk, n - first);
    const float *X = feed.load(first, count, stream);
    // gather the chunk's planes, add the trees, scatter back
    for (int k = 0; k < K; ++k)
      ARB_CUDA(cudaMemcpyAsync(d_tmp.as<float>() + size_t(k) * count,
                               data->d_yhat.as<float>() + size_t(k) * n + first, count * sizeof(float),
                               cudaMemcpyDeviceToDevice, stream));
    launch_predict(X, count, data->cols_dense, pt, int(trees.size()) - K, K, int(cfg.tree.depth),
                   d_tmp.as<float>(), stream, 0, feed.categories(first), data->cols_cat);
    for (int k = 0; k < K; ++k)
      ARB_CUDA(cudaMemcpyAsync(data->d_yhat.as<float>() + size_t(k) * n + first,
                               d_tmp.as<float>() + size_t(k) * count, count * sizeof(float),
                               cudaMemcpyDeviceToDevice, stream));
    ARB_CUDA(cudaStreamSynchronize(stream));
  }
}

// Garden::GetY garden.cu:637-641: link-transformed accumulated prediction
void Garden::GetY(DataMatrix *data, std::vector<float> &out) {
  const int K = int(cfg.tree.labels_count);
  const size_t n = size_t(data->rows);
  if (!data->d_yhat.p) {  // nothing appended yet: the reference returns an empty vector
    out.clear();
    return;
  }
  EnsureStream();
  out.resize(n * K);
  DevBuf d_out;
  d_out.alloc(n * K * sizeof(float));
  launch_link(cfg.objective, K, n, data->d_yhat.as<float>(), d_out.as<float>(), stream);
  ARB_CUDA(cudaMemcpyAsync(out.data(), d_out.p, n * K * sizeof(float), cudaMemcpyDeviceToHost, stream));
  ARB_CUDA(cudaStreamSynchronize(stream));
}

// model_helper.cpp:16-23, json_conversion.h:13-49
std::string Garden::GetModel() const {
  Json root = Json::object();
  root["configuration"] = cfg.ToJson();
  Json model = Json::array();
  for (const Tree &t : trees) {
    Json jt = Json::object();
    jt["depth"] = Json::integer(t.depth);
    Json nodes = Json::array();
    const unsigned first_leaf = (1u << (t.depth - 1)) - 1;
    for (unsigned i = 0; i < t.nodes.size(); ++i) {
      Json jn = Json::object();
      jn["id"] = Json::integer(i);
      const bool leaf = i >= first_leaf;
      jn["leaf"] = Json::boolean(leaf);
      if (!leaf) {
        jn["left"] = Json::integer(2 * i + 1);
        jn["right"] = Json::integer(2 * i + 2);
        jn["threshold"] = Json::number(double(t.nodes[i].threshold));  // +inf -> null
        jn["fid"] = Json::integer(t.nodes[i].fid);
        // additive key (the reference does not serialise categories, json_conversion.h:13-35)
        if (t.nodes[i].categorical) jn["category"] = Json::integer(t.nodes[i].category);
      } else {
        jn["idx"] = Json::integer(i - first_leaf);
      }
      nodes.arr.push_back(jn);
    }
    jt["nodes"] = nodes;
    Json w = Json::array();
    for (float v : t.weights) w.arr.push_back(Json::number(double(v)));
    jt["weights"] = w;
    model.arr.push_back(jt);
  }
  root["model"] = model;
  std::string out;
  json_write(root, out);
  return out;
}

// Garden::Restore garden.cu:659-677 (every restored tree gets label 0, as there)
void Garden::Restore(const char *json_model) {
  const Json j = JsonParser(json_model).parse();
  const Json &model = j.at("model");
  ARB_CHECK(model.type == Json::Arr, "model must be an array of trees");
  const int K = std::max(1, int(cfg.tree.labels_count));
  for (const Json &jt : model.arr) {
    Tree t;
    const double depth_num = jt.at("depth").as_num();
    ARB_CHECK(depth_num >= 1 && depth_num <= kMaxLevels, "tree depth out of range");
    t.depth = int(depth_num);
    // the reference gives every restored tree label 0 (garden.cu:659-677), which is right for
    // its single-output objectives; the trees of a multi:softmax model were dumped class after
    // class, round after round
    t.label = int(trees.size() % size_t(K));
    const Json &nodes = jt.at("nodes");
    t.nodes.assign(nodes.arr.size(), TreeNode());
    for (const Json &jn : nodes.arr) {
      const size_t id = size_t(jn.at("id").as_num());
      ARB_CHECK(id < t.nodes.size(), "node id out of range");
      if (jn.has("threshold")) {
        const Json &th = jn.at("threshold");
        t.nodes[id].threshold = th.type == Json::Null ? std::numeric_limits<float>::infinity()
                                                      : float(th.as_num());
      }
      if (jn.has("category")) {
        t.nodes[id].categorical = true;
        t.nodes[id].category = unsigned(jn.at("category").as_num());
      }
      if (jn.has("fid")) {
        // inference indexes a row of the matrix with it, on the device
        const double fid = jn.at("fid").as_num();
        ARB_CHECK(fid >= 0 && fid < 65535, "feature id out of range");
        t.nodes[id].fid = int(fid);
        max_fid = std::max(max_fid, int(fid));
      }
    }
    for (const Json &w : jt.at("weights").arr) t.weights.push_back(float(w.as_num()));
    ARB_CHECK(t.depth >= 1 && t.nodes.size() == (size_t(1) << t.depth) - 1 &&
                t.weights.size() == (size_t(1) << (t.depth - 1)),
              "tree shape does not match its depth");
    trees.push_back(std::move(t));
  }
}

}  // namespace arb
