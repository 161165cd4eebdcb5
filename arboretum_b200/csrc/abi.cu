// extern "C" boundary of libarboretum.so: the reference's fourteen entry points
// (python-wrapper/arboretum_wrapper.cu:16-205) plus the additive ones declared in
// include/arboretum_b200.h.  Every exception becomes the returned message.
#include <dlfcn.h>
#include <nccl.h>

#include <climits>
#include <cstring>
#include <mutex>

#include "../../include/arboretum_b200.h"
#include "exchange.h"
#include "garden.h"

using namespace arb;

namespace {

thread_local std::string g_error;

const char *fail(const std::exception &e) {
  g_error = e.what();
  return g_error.c_str();
}
const char *fail(const char *msg) {
  g_error = msg;
  return g_error.c_str();
}

#define ARB_TRY try {
#define ARB_CATCH                                 \
  return nullptr;                                 \
  }                                               \
  catch (const std::exception &e) { return fail(e); } \
  catch (const char *e) { return fail(e); }       \
  catch (...) { return fail("unknown error"); }

// ---- NCCL through dlopen: the library has no link-time dependency on it -------
struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;  // optional
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;                          // optional
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  void load() {
    if (handle) return;
    // a copy that the process already loaded (torch ships one) is found first
    handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!handle) handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!handle) throw std::runtime_error(std::string("cannot load libnccl.so.2: ") + dlerror());
    GetUniqueId = reinterpret_cast<decltype(GetUniqueId)>(dlsym(handle, "ncclGetUniqueId"));
    CommInitRank = reinterpret_cast<decltype(CommInitRank)>(dlsym(handle, "ncclCommInitRank"));
    AllReduce = reinterpret_cast<decltype(AllReduce)>(dlsym(handle, "ncclAllReduce"));
    AllGather = reinterpret_cast<decltype(AllGather)>(dlsym(handle, "ncclAllGather"));
    CommDestroy = reinterpret_cast<decltype(CommDestroy)>(dlsym(handle, "ncclCommDestroy"));
    GetErrorString = reinterpret_cast<decltype(GetErrorString)>(dlsym(handle, "ncclGetErrorString"));
    CommGetAsyncError = reinterpret_cast<decltype(CommGetAsyncError)>(dlsym(handle, "ncclCommGetAsyncError"));
    CommAbort = reinterpret_cast<decltype(CommAbort)>(dlsym(handle, "ncclCommAbort"));
    if (!GetUniqueId || !CommInitRank || !AllReduce || !AllGather || !CommDestroy || !GetErrorString)
      throw std::runtime_error("libnccl.so.2 lacks a required symbol");
  }
};
NcclApi g_nccl;

// The first communicator a process makes is kept for the life of the process and can be
// attached to later Gardens (AInitNccl with a NULL id): bringing one up takes a second or
// more, far longer than a short training job.  It is never destroyed (at exit the CUDA
// context may already be gone).
ncclComm_t g_process_comm = nullptr;
int g_process_world = 0, g_process_rank = -1;

struct NcclCtx {
  bool shared = false;  // comm is g_process_comm: not destroyed with the Garden
  ncclComm_t comm = nullptr;
};

int nccl_allreduce(void *ctx, long long *buf, size_t count, cudaStream_t s) {
  NcclCtx *c = static_cast<NcclCtx *>(ctx);
  const ncclResult_t r = g_nccl.AllReduce(buf, buf, count, ncclInt64, ncclSum, c->comm, s);
  return r == ncclSuccess ? 0 : 1;
}

int nccl_allgather(void *ctx, const void *send, void *recv, size_t bytes, cudaStream_t s) {
  NcclCtx *c = static_cast<NcclCtx *>(ctx);
  const ncclResult_t r = g_nccl.AllGather(send, recv, bytes, ncclChar, c->comm, s);
  return r == ncclSuccess ? 0 : 1;
}

int nccl_allreduce_max(void *ctx, unsigned *buf, size_t count, cudaStream_t s) {
  NcclCtx *c = static_cast<NcclCtx *>(ctx);
  const ncclResult_t r = g_nccl.AllReduce(buf, buf, count, ncclUint32, ncclMax, c->comm, s);
  return r == ncclSuccess ? 0 : 1;
}

// CommCheckFn of the NCCL path (see garden.h)
int nccl_check(void *ctx, int give_up, char *msg, size_t msg_len) {
  NcclCtx *c = static_cast<NcclCtx *>(ctx);
  ncclResult_t state = ncclSuccess;
  if (g_nccl.CommGetAsyncError && g_nccl.CommGetAsyncError(c->comm, &state) != ncclSuccess) state = ncclInternalError;
  if (state == ncclInProgress) state = ncclSuccess;
  if (state == ncclSuccess && !give_up) return 0;
  if (state != ncclSuccess && msg_len)
    std::snprintf(msg, msg_len, "NCCL reports %s", g_nccl.GetErrorString(state));
  if (g_nccl.CommAbort) g_nccl.CommAbort(c->comm);
  if (c->comm == g_process_comm) g_process_comm = nullptr;  // never handed out again
  c->comm = nullptr;
  return 1;
}

void host_scales(float max_g, float max_h, int qb, bool pair, QuantScale *q) {
  int eg = 0, eh = 0;
  if (max_g > 0.0f && std::isfinite(max_g)) std::frexp(max_g, &eg);
  if (max_h > 0.0f && std::isfinite(max_h)) std::frexp(max_h, &eh);
  q->sg = std::ldexp(1.0f, qb - eg);
  q->inv_sg = std::ldexp(1.0, eg - qb);
  q->sh = pair ? std::ldexp(1.0f, qb - eh) : 1.0f;
  q->inv_sh = pair ? std::ldexp(1.0, eh - qb) : 1.0;
  q->max_g_bits = q->max_h_bits = 0;
}

// Targets follow the matrix: when it sits in HBM they are copied straight from the
// caller's buffer to the same device (no host copy is kept); false = keep them on the host.
// true when `p` points into device memory (such a buffer can only be copied, not read, here)
bool is_device_pointer(const void *p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice;
}

bool upload_beside_matrix(DataMatrix *d, DevBuf &dst, const void *src, size_t bytes) {
  if (d->device < 0) return false;
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess) return false;
  if (cur != d->device && cudaSetDevice(d->device) != cudaSuccess) return false;
  bool ok = true;
  if (dst.bytes != bytes) {
    dst.release();
    void *p = nullptr;
    ok = dev_alloc(&p, bytes) == cudaSuccess;
    if (ok) {
      dst.p = p;
      dst.bytes = bytes;
    }
  }
  ok = ok && cudaMemcpy(dst.p, src, bytes, cudaMemcpyDefault) == cudaSuccess;  // host or device source
  if (!ok) {
    cudaGetLastError();
    dst.release();
  }
  if (cur != d->device) cudaSetDevice(cur);
  return ok;
}

}  // namespace

extern "C" {

const char *ACreateFromDenseMatrix(const float *data, const unsigned int *categories, int nrow,
                                   int ncol, int ccol, float missing, VoidPointer *out) {
  ARB_TRY
  (void)missing;     // never read by the reference either (arboretum_wrapper.cu:16-39)
  ARB_CHECK(out != nullptr, "out is NULL");
  ARB_CHECK(nrow > 0 && ncol > 0 && ccol >= 0, "bad matrix shape");
  ARB_CHECK(data != nullptr, "data is NULL");
  ARB_CHECK(ccol == 0 || categories != nullptr, "categories is NULL");
  std::unique_ptr<DataMatrix> m(new DataMatrix(nrow, ncol, ccol));
  if (ccol > 0) {  // arboretum_wrapper.cu:30-33; kept on the host for the quantiser
    ARB_CHECK(!is_device_pointer(categories), "category codes are read on the host: pass host memory");
    m->cat.assign(categories, categories + size_t(nrow) * ccol);
  }
  StageTrace trace("ACreateFromDenseMatrix");
  // The matrix goes straight into HBM (one host->device copy from the caller's buffer,
  // no staging copy on the host); quantisation and inference read it there.  Without a
  // usable device, or when it does not fit beside the training state, a host copy is kept.
  const size_t bytes = size_t(nrow) * ncol * sizeof(float);
  size_t free_b = 0;
  bool on_device = false;
  if (dev_available(&free_b) == cudaSuccess && bytes < free_b / 2) {
    void *p = nullptr;
    if (dev_alloc(&p, bytes) == cudaSuccess) {
      m->d_x.p = p;
      m->d_x.bytes = bytes;
      // `data` may be host memory or (additive) device memory, e.g. an array another
      // library left on the GPU: the copy takes either
      on_device = cudaMemcpy(p, data, bytes, cudaMemcpyDefault) == cudaSuccess &&
                  cudaGetDevice(&m->device) == cudaSuccess;
      if (!on_device) m->d_x.release();
    }
  }
  if (!on_device) {
    cudaGetLastError();  // clear the error state: the host copy below is the fallback storage
    ARB_CHECK(!is_device_pointer(data), "a matrix in device memory that does not fit beside its training state");
    m->x.assign(data, data + size_t(nrow) * ncol);
  }
  trace.lap("matrix to HBM");
  if (ccol > 0 && on_device) {  // inference reads the category codes beside the matrix
    m->d_cat.alloc(m->cat.size() * sizeof(unsigned));
    ARB_CUDA(cudaMemcpy(m->d_cat.p, m->cat.data(), m->d_cat.bytes, cudaMemcpyHostToDevice));
  }
  ARB_CHECK(ccol == 0 || on_device, "categorical columns need the matrix in device memory");
  *out = m.release();
  ARB_CATCH
}

const char *ACreateFromBinnedMatrix(const uint8_t *bins, int64_t nrow, int ncol, int hist_size,
                                    VoidPointer *out) {
  ARB_TRY
  ARB_CHECK(out != nullptr && bins != nullptr, "NULL argument");
  ARB_CHECK(nrow > 0 && ncol > 0, "bad matrix shape");
  ARB_CHECK(hist_size > 0 && hist_size < 256, "pre-binned input needs 0 < hist_size < 256");
  std::unique_ptr<DataMatrix> m(new DataMatrix(nrow, ncol, 0));
  m->prebinned = true;
  m->hist_size = hist_size;
  // Like the dense constructor: the rows go to HBM right away when they take at most a
  // quarter of the free memory (training needs the padded copy and its transpose too);
  // larger inputs stay on the host, for out-of-core training.
  const size_t bytes = size_t(nrow) * ncol;
  size_t free_b = 0;
  bool on_device = false;
  if (dev_available(&free_b) == cudaSuccess && bytes <= free_b / 4) {
    void *p = nullptr;
    if (dev_alloc(&p, bytes) == cudaSuccess) {
      m->d_raw.p = p;
      m->d_raw.bytes = bytes;
      // the rows may already be in device memory (generated or decoded there): any source works
      on_device = cudaMemcpy(p, bins, bytes, cudaMemcpyDefault) == cudaSuccess &&
                  cudaGetDevice(&m->device) == cudaSuccess;
      if (!on_device) m->d_raw.release();
    }
  }
  if (!on_device) {
    cudaGetLastError();
    ARB_CHECK(!is_device_pointer(bins), "rows in device memory that do not fit beside their training state");
    m->host_bins.assign(bins, bins + bytes);
  }
  *out = m.release();
  ARB_CATCH
}

const char *ASetY(VoidPointer data, const float *y) {
  ARB_TRY
  ARB_CHECK(data && y, "NULL argument");
  DataMatrix *d = static_cast<DataMatrix *>(data);
  if (!upload_beside_matrix(d, d->d_y, y, size_t(d->rows) * sizeof(float))) {
    ARB_CHECK(!is_device_pointer(y), "targets in device memory need the matrix in device memory");
    d->y.assign(y, y + d->rows);
  }
  ARB_CATCH
}

const char *ASetLabel(VoidPointer data, const unsigned char *labels) {
  ARB_TRY
  ARB_CHECK(data && labels, "NULL argument");
  DataMatrix *d = static_cast<DataMatrix *>(data);
  if (!upload_beside_matrix(d, d->d_labels, labels, size_t(d->rows)))
    d->labels.assign(labels, labels + d->rows);
  ARB_CATCH
}

const char *ASetWeights(VoidPointer data, const float *weights) {
  ARB_TRY
  ARB_CHECK(data && weights, "NULL argument");
  DataMatrix *d = static_cast<DataMatrix *>(data);
  d->weights.assign(weights, weights + d->rows);  // stored, unused: as in the reference
  ARB_CATCH
}

const char *ASetThresholds(VoidPointer data, const float *thr, const int *size, int hist_size) {
  ARB_TRY
  ARB_CHECK(data && thr && size, "NULL argument");
  DataMatrix *d = static_cast<DataMatrix *>(data);
  ARB_CHECK(!d->binned, "the matrix is already quantised");
  ARB_CHECK(hist_size > 0 && hist_size < 2048, "hist_size must be in [1, 2047]");
  // bin ids index the threshold table and the shared-memory histograms: a size outside
  // [1, hist_size] would send both out of range
  for (int f = 0; f < d->cols_dense; ++f)
    ARB_CHECK(size[f] >= 1 && size[f] <= hist_size, "size[f] must be in [1, hist_size]");
  d->thr.assign(thr, thr + size_t(d->cols_dense) * hist_size);
  d->fsize.assign(size, size + d->cols_dense);
  d->thresholds_given = true;
  d->hist_size = hist_size;
  ARB_CATCH
}

const char *AQuantize(VoidPointer data, int hist_size, int missing_bin, float *thr, int *size,
                      uint16_t *bins) {
  ARB_TRY
  ARB_CHECK(data, "NULL argument");
  DataMatrix *d = static_cast<DataMatrix *>(data);
  ARB_CHECK(!d->thresholds_given || d->hist_size == hist_size, "hist_size differs from ASetThresholds");
  d->InitHist(hist_size, missing_bin != 0, false, nullptr);
  ARB_CHECK(d->hist_size == hist_size, "the matrix was quantised with another hist_size");
  const int F = d->cols_dense;
  if (thr) std::copy(d->thr.begin(), d->thr.end(), thr);
  if (size) std::copy(d->fsize.begin(), d->fsize.end(), size);
  if (bins) {
    std::vector<unsigned char> raw(size_t(d->rows) * d->pitch);
    ARB_CUDA(cudaMemcpy(raw.data(), d->d_bins.p, raw.size(), cudaMemcpyDeviceToHost));
    for (int64_t r = 0; r < d->rows; ++r)
      for (int f = 0; f < F; ++f)
        bins[r * F + f] = d->bin_bytes == 1
                            ? raw[r * d->pitch + f]
                            : reinterpret_cast<const uint16_t *>(raw.data() + r * d->pitch)[f];
  }
  ARB_CATCH
}

const char *AInitGarden(const char *configuration, VoidPointer *out) {
  ARB_TRY
  ARB_CHECK(configuration && out, "NULL argument");
  const Configuration cfg = Configuration::Parse(configuration);
  *out = new Garden(cfg);
  ARB_CATCH
}

const char *AGrowTree(VoidPointer garden, VoidPointer data, const float *grad) {
  ARB_TRY
  ARB_CHECK(garden && data, "NULL argument");
  static_cast<Garden *>(garden)->GrowTree(static_cast<DataMatrix *>(data), grad);
  ARB_CATCH
}

static const char *to_new_array(const std::vector<float> &v, const float **out) {
  float *p = new (std::nothrow) float[v.size() ? v.size() : 1];
  if (!p) return fail("unable to allocate the result array");
  std::copy(v.begin(), v.end(), p);
  *out = p;
  return nullptr;
}

const char *APredict(VoidPointer garden, VoidPointer data, const float **out, const int n_rounds) {
  ARB_TRY
  ARB_CHECK(garden && data && out, "NULL argument");
  std::vector<float> result;
  static_cast<Garden *>(garden)->Predict(static_cast<DataMatrix *>(data), result,
                                         n_rounds == -1 ? INT_MAX : n_rounds);
  if (const char *e = to_new_array(result, out)) return e;
  ARB_CATCH
}

const char *AGetY(VoidPointer garden, VoidPointer data, const float **out) {
  ARB_TRY
  ARB_CHECK(garden && data && out, "NULL argument");
  std::vector<float> result;
  static_cast<Garden *>(garden)->GetY(static_cast<DataMatrix *>(data), result);
  if (const char *e = to_new_array(result, out)) return e;
  ARB_CATCH
}

const char *AAppendLastTree(VoidPointer garden, VoidPointer data) {
  ARB_TRY
  ARB_CHECK(garden && data, "NULL argument");
  static_cast<Garden *>(garden)->UpdateByLastTree(static_cast<DataMatrix *>(data));
  ARB_CATCH
}

const char *ADumpModel(const char **model, VoidPointer garden) {
  ARB_TRY
  ARB_CHECK(garden && model, "NULL argument");
  const std::string s = static_cast<Garden *>(garden)->GetModel();
  char *c = new char[s.size() + 1];  // owned by the caller side, as in model_helper.cpp:19-22
  std::memcpy(c, s.c_str(), s.size() + 1);
  *model = c;
  ARB_CATCH
}

const char *ALoadModel(const char *model, VoidPointer garden) {
  ARB_TRY
  ARB_CHECK(garden && model, "NULL argument");
  static_cast<Garden *>(garden)->Restore(model);
  ARB_CATCH
}

const char *AFreeDMatrix(VoidPointer ptr) {
  ARB_TRY
  delete static_cast<DataMatrix *>(ptr);
  ARB_CATCH
}

const char *AFreeGarden(VoidPointer ptr) {
  ARB_TRY
  Garden *g = static_cast<Garden *>(ptr);
  if (g && g->allreduce_ctx) {
    NcclCtx *c = static_cast<NcclCtx *>(g->allreduce_ctx);
    g->ReleaseBuilder();  // before the communicator it may still be using
    if (c->comm && !c->shared) g_nccl.CommDestroy(c->comm);
    delete c;
    g->allreduce_ctx = nullptr;
  }
  delete g;
  ARB_CATCH
}

const char *ADeleteArray(float *in) {
  delete[] in;
  return nullptr;
}

const char *AGetTrainY(VoidPointer garden, float *out) {
  ARB_TRY
  ARB_CHECK(garden && out, "NULL argument");
  BuilderView::train_yhat(static_cast<Garden *>(garden), out);
  ARB_CATCH
}

const char *AGetLevelStats(VoidPointer garden, int level, unsigned *node_begin, float *gain, int *fid,
                           int *bin, double *left_g, double *left_h, double *tot_g, double *tot_h,
                           unsigned *left_count) {
  return AGetLevelStatsOf(garden, -1, level, node_begin, gain, fid, bin, left_g, left_h, tot_g, tot_h,
                          left_count);
}

const char *AGetLevelStatsOf(VoidPointer garden, int tree_in_round, int level, unsigned *node_begin,
                             float *gain, int *fid, int *bin, double *left_g, double *left_h,
                             double *tot_g, double *tot_h, unsigned *left_count) {
  ARB_TRY
  ARB_CHECK(garden, "NULL argument");
  Garden *g = static_cast<Garden *>(garden);
  int max_nodes = 0, levels = 0, stride = 0;
  const NodeRec *rec = BuilderView::host_rec(g, tree_in_round, &max_nodes, &levels);
  const unsigned *nb = BuilderView::host_node_begin(g, tree_in_round, &stride);
  ARB_CHECK(level >= 0 && level < levels, "level out of range");
  QuantScale q;
  BuilderView::scales(g, &q);
  const int L = 1 << level;
  for (int i = 0; i <= L && node_begin; ++i) node_begin[i] = nb[size_t(level) * stride + i];
  for (int i = 0; i < L; ++i) {
    const NodeRec &r = rec[size_t(level) * max_nodes + i];
    if (gain) gain[i] = r.gain;
    if (fid) fid[i] = r.fid;
    if (bin) bin[i] = r.bin;
    if (left_g) left_g[i] = double(r.lg) * q.inv_sg;
    if (left_h) left_h[i] = double(r.lh) * q.inv_sh;
    if (tot_g) tot_g[i] = double(r.tg) * q.inv_sg;
    if (tot_h) tot_h[i] = double(r.th) * q.inv_sh;
    if (left_count) left_count[i] = r.left_count;
  }
  ARB_CATCH
}

const char *AGetGradientStep(VoidPointer garden, double *g_step, double *h_step) {
  ARB_TRY
  ARB_CHECK(garden, "NULL argument");
  QuantScale q;
  BuilderView::scales(static_cast<Garden *>(garden), &q);
  if (g_step) *g_step = q.inv_sg;
  if (h_step) *h_step = q.inv_sh;
  ARB_CATCH
}

const char *ASetProfile(VoidPointer garden, int on) {
  ARB_TRY
  ARB_CHECK(garden, "NULL argument");
  Garden *g = static_cast<Garden *>(garden);
  g->profile = on != 0;
  g->times = PhaseTimes();
  double xms[3];
  long long xn = 0;
  BuilderView::exchange_clock(g, xms, &xn, true);  // the exchange clocks start over as well
  ARB_CATCH
}

const char *AGetTimings(VoidPointer garden, const char **json) {
  ARB_TRY
  ARB_CHECK(garden && json, "NULL argument");
  Garden *g = static_cast<Garden *>(garden);
  const PhaseTimes &t = g->times;
  Json j = Json::object();
  j["trees"] = Json::integer(t.trees);
  j["grad_ms"] = Json::number(t.grad);
  j["hist_ms"] = Json::number(t.hist);
  j["hist_kernel_ms"] = Json::number(t.hist_kernel);
  j["plan_ms"] = Json::number(t.plan);
  j["subtract_ms"] = Json::number(t.subtract);
  j["split_ms"] = Json::number(t.split);
  j["partition_ms"] = Json::number(t.partition);
  j["update_ms"] = Json::number(t.update);
  j["allreduce_ms"] = Json::number(t.allreduce);
  j["hist_launches"] = Json::integer(t.hist_launches);
  j["hist_rows"] = Json::number(t.hist_rows);
  j["hist_row_features"] = Json::number(t.hist_features);
  j["hist_bytes"] = Json::number(t.hist_bytes);
  j["tree_ms"] = Json::number(t.tree);
  j["host_enqueue_ms"] = Json::number(t.enqueue);
  j["host_wait_ms"] = Json::number(t.host_wait);
  j["host_trees"] = Json::number(double(t.host_trees));
  j["h2d_bytes"] = Json::number(t.h2d_bytes);
  j["kernel_launches"] = Json::integer(g_kernel_launches);
  double xms[3];
  long long xn = 0;
  if (BuilderView::exchange_clock(g, xms, &xn, false)) {
    j["exchange_wait_peers_ms"] = Json::number(xms[0]);
    j["exchange_move_ms"] = Json::number(xms[1]);
    j["exchange_wait_done_ms"] = Json::number(xms[2]);
    j["exchanges"] = Json::integer(xn);
  }
  j["level_exchange"] = Json::string(g->peer_exchange ? "peer memory" : g->allreduce ? "ncclAllReduce" : "none");
  static thread_local std::string text;
  text.clear();
  json_write(j, text);
  *json = text.c_str();
  ARB_CATCH
}

const char *AReleaseCachedMemory() {
  ARB_TRY
  ARB_CUDA(dev_trim());
  ARB_CATCH
}

const char *ASharedAtomicPeak(int steps, double *pair_updates_per_s) {
  ARB_TRY
  ARB_CHECK(pair_updates_per_s != nullptr, "NULL argument");
  ARB_CHECK(steps > 0 && steps <= (1 << 20), "steps must be in [1, 2^20]");
  *pair_updates_per_s = measure_shared_atomic_peak(steps, nullptr);
  ARB_CATCH
}

static const char *build_histogram(const void *bins, int bin_bytes, int64_t nrow, int ncol, int hist_size,
                                   const float *grad, int pair, const unsigned *rowid,
                                   const unsigned *node_begin, int n_nodes, int quant_bits, double *out_g,
                                   double *out_h, int reps, float *ms, const double *parent_g,
                                   const double *parent_h) {
  ARB_TRY
  const bool trick = parent_g != nullptr;
  ARB_CHECK(!trick || (parent_h != nullptr && n_nodes % 2 == 0), "the subtraction needs both parent arrays and an even node count");
  ARB_CHECK(bins && grad && node_begin && out_g && out_h, "NULL argument");
  ARB_CHECK(bin_bytes == 1 || bin_bytes == 2, "bin_bytes must be 1 or 2");
  ARB_CHECK(nrow > 0 && ncol > 0 && n_nodes > 0, "bad shape");
  ARB_CHECK(hist_size > 0 && hist_size < 2048 && (bin_bytes == 2 || hist_size < 256), "bad hist_size");
  ARB_CHECK(quant_bits >= 10 && quant_bits <= 22, "quant_bits must be in [10, 22]");
  ARB_CHECK(nrow < (int64_t(1) << 31), "row count must be below 2^31");
  const size_t n = size_t(nrow);
  // The arrays below drive gathers and shared-memory updates on the device; anything out of
  // range is refused here, where it is an error string and not a memory fault.
  for (int i = 0; i < n_nodes; ++i)
    ARB_CHECK(node_begin[i] <= node_begin[i + 1], "node_begin must be non-decreasing");
  ARB_CHECK(node_begin[n_nodes] <= n, "node_begin exceeds the row count");
  if (rowid)
    for (size_t i = 0; i < n; ++i) ARB_CHECK(rowid[i] < n, "rowid out of range");
  {
    const size_t cells = n * size_t(ncol);
    bool ok = true;
    if (bin_bytes == 1) {
      const unsigned char *b = static_cast<const unsigned char *>(bins);
      for (size_t i = 0; i < cells; ++i) ok = ok && b[i] <= hist_size;
    } else {
      const unsigned short *b = static_cast<const unsigned short *>(bins);
      for (size_t i = 0; i < cells; ++i) ok = ok && b[i] <= hist_size;
    }
    ARB_CHECK(ok, "bin id above hist_size (ids 0..hist_size-1 are bins, hist_size is the missing-value bin)");
  }
  Geometry geo;
  geo.pitch = DataMatrix::PitchFor(ncol, bin_bytes);
  geo.bin_bytes = bin_bytes;
  geo.F = ncol;
  geo.n_dense = ncol;
  geo.hist_size = hist_size;
  int bins_pad = 256;
  while (bins_pad < hist_size + 1) bins_pad <<= 1;
  geo.BINS = bins_pad;
  geo.TW = kHistWords / bins_pad;
  geo.NT = (ncol + geo.TW - 1) / geo.TW;
  struct StreamGuard {  // destroyed on every way out, also when something below throws
    cudaStream_t s = nullptr;
    ~StreamGuard() {
      if (s) cudaStreamDestroy(s);
    }
  } stream_guard;
  ARB_CUDA(cudaStreamCreateWithFlags(&stream_guard.s, cudaStreamNonBlocking));
  cudaStream_t s = stream_guard.s;
  DevBuf d_bins, d_grad, d_rowid, d_items, d_nitems, d_hist, d_qs;
  d_bins.alloc(n * geo.pitch);
  ARB_CUDA(cudaMemsetAsync(d_bins.p, 0, d_bins.bytes, s));
  ARB_CUDA(cudaMemcpy2DAsync(d_bins.p, geo.pitch, bins, size_t(ncol) * bin_bytes,
                             size_t(ncol) * bin_bytes, n, cudaMemcpyHostToDevice, s));
  geo.bins = d_bins.as<unsigned char>();
  const size_t gsz = pair ? 2 : 1;
  d_grad.alloc(n * gsz * sizeof(float));
  ARB_CUDA(cudaMemcpyAsync(d_grad.p, grad, d_grad.bytes, cudaMemcpyHostToDevice, s));
  if (rowid) {
    d_rowid.alloc(n * sizeof(unsigned));
    ARB_CUDA(cudaMemcpyAsync(d_rowid.p, rowid, d_rowid.bytes, cudaMemcpyHostToDevice, s));
  }
  float max_g = 0.f, max_h = 0.f;
  for (size_t i = 0; i < n; ++i) {
    max_g = std::max(max_g, std::fabs(grad[i * gsz]));
    if (pair) max_h = std::max(max_h, grad[i * gsz + 1]);
  }
  QuantScale q;
  host_scales(max_g, max_h, quant_bits, pair != 0, &q);
  d_qs.alloc(sizeof q);
  ARB_CUDA(cudaMemcpyAsync(d_qs.p, &q, sizeof q, cudaMemcpyHostToDevice, s));
  launch_quantize_grads(d_grad.p, n, pair != 0, d_qs.as<QuantScale>(), quant_bits, s);
  const unsigned cap = 1u << (31 - quant_bits);
  std::vector<WorkItem> items;
  // with parents: one child per pair is built, the smaller one, ties the left
  // (hist_grad_sum.cu:288-290 of the reference); the other is parent - built
  const int n_build = trick ? n_nodes / 2 : n_nodes;
  std::vector<int> first(n_build + 1, 0), ids(n_build), built(std::max(1, n_nodes / 2), 0);
  for (int b = 0; b < n_build; ++b) {
    int node = b;
    if (trick) {
      const unsigned ls = node_begin[2 * b + 1] - node_begin[2 * b], rs = node_begin[2 * b + 2] - node_begin[2 * b + 1];
      built[b] = ls <= rs ? 0 : 1;
      node = 2 * b + built[b];
    }
    first[b] = int(items.size());
    ids[b] = node;
    for (unsigned at = node_begin[node]; at < node_begin[node + 1]; at += cap)
      items.push_back(WorkItem{at, std::min(cap, node_begin[node + 1] - at), node, 0});
  }
  first[n_build] = int(items.size());
  ARB_CHECK(!items.empty(), "no rows");
  const int n_items = int(items.size());
  DevBuf d_first, d_ids, d_partials;
  d_items.alloc(items.size() * sizeof(WorkItem));
  d_nitems.alloc(sizeof(int));
  d_first.alloc(first.size() * sizeof(int));
  d_ids.alloc(ids.size() * sizeof(int));
  d_partials.alloc(size_t(n_items) * geo.NT * 2 * kHistWords * sizeof(int));
  ARB_CUDA(cudaMemcpyAsync(d_items.p, items.data(), d_items.bytes, cudaMemcpyHostToDevice, s));
  ARB_CUDA(cudaMemcpyAsync(d_nitems.p, &n_items, sizeof(int), cudaMemcpyHostToDevice, s));
  ARB_CUDA(cudaMemcpyAsync(d_first.p, first.data(), d_first.bytes, cudaMemcpyHostToDevice, s));
  ARB_CUDA(cudaMemcpyAsync(d_ids.p, ids.data(), d_ids.bytes, cudaMemcpyHostToDevice, s));
  const size_t words = size_t(n_nodes) * geo.NT * kHistWords * 2;
  d_hist.alloc(words * sizeof(long long));
  ARB_CUDA(cudaMemsetAsync(d_hist.p, 0, d_hist.bytes, s));
  DevBuf d_parent, d_built;
  if (trick) {  // the parents' sums as the fixed-point integers the kernels subtract from
    const int HWp = hist_size + 1;
    std::vector<long long> parent(words / 2, 0);
    for (int p = 0; p < n_nodes / 2; ++p)
      for (int f = 0; f < ncol; ++f)
        for (int b = 0; b < HWp; ++b) {
          const size_t src = (size_t(p) * ncol + f) * HWp + b;
          const size_t dst = (((size_t(p) * geo.NT + f / geo.TW) * geo.BINS + b) * geo.TW + f % geo.TW) * 2;
          parent[dst] = std::llrint(parent_g[src] * double(q.sg));
          parent[dst + 1] = std::llrint(parent_h[src] * double(q.sh));
        }
    d_parent.alloc(parent.size() * sizeof(long long));
    d_built.alloc(built.size() * sizeof(int));
    ARB_CUDA(cudaMemcpyAsync(d_parent.p, parent.data(), d_parent.bytes, cudaMemcpyHostToDevice, s));
    ARB_CUDA(cudaMemcpyAsync(d_built.p, built.data(), d_built.bytes, cudaMemcpyHostToDevice, s));
    ARB_CUDA(cudaStreamSynchronize(s));  // `parent` and `built` leave scope below
  }
  HistLaunch h;
  h.geo = geo;
  h.rowid = rowid ? d_rowid.as<unsigned>() : nullptr;
  h.grad = d_grad.p;
  h.pair = pair != 0;
  h.items = d_items.as<WorkItem>();
  h.n_items = d_nitems.as<int>();
  h.max_items = n_items;
  h.partials = d_partials.as<int>();
  // rows named by `rowid` are gathered through the TMA unit where that is possible, like in training
  RowGatherMap row_map;
  DevBuf d_gather_status;
  if (rowid && make_row_gather_map(&row_map, geo.bins, geo.pitch, n)) {
    d_gather_status.alloc(sizeof(int));
    ARB_CUDA(cudaMemsetAsync(d_gather_status.p, 0, sizeof(int), s));
    h.row_map = &row_map;
    h.status = d_gather_status.as<int>();
  }
  ReduceLaunch rd;
  rd.partials = d_partials.as<int>();
  rd.item_first = d_first.as<int>();
  rd.build_node = d_ids.as<int>();
  rd.n_build = n_build;
  rd.NT = geo.NT;
  rd.level_hist = d_hist.as<long long>();
  rd.parent_hist = trick ? d_parent.as<long long>() : nullptr;
  rd.subtract = trick;
  rd.level_nodes = n_nodes;
  rd.built_child = trick ? d_built.as<int>() : nullptr;
  if (reps > 0) {
    struct EventPair {
      cudaEvent_t e0 = nullptr, e1 = nullptr;
      ~EventPair() {
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
      }
    } ev;
    ARB_CUDA(cudaEventCreate(&ev.e0));
    ARB_CUDA(cudaEventCreate(&ev.e1));
    for (int i = 0; i < 3; ++i) launch_hist(h, s);
    ARB_CUDA(cudaEventRecord(ev.e0, s));
    for (int i = 0; i < reps; ++i) launch_hist(h, s);
    ARB_CUDA(cudaEventRecord(ev.e1, s));
    ARB_CUDA(cudaEventSynchronize(ev.e1));
    float t = 0;
    ARB_CUDA(cudaEventElapsedTime(&t, ev.e0, ev.e1));
    if (ms) *ms = t / reps;
  }
  launch_hist(h, s);
  launch_reduce(rd, s);
  std::vector<long long> host(words);
  ARB_CUDA(cudaMemcpyAsync(host.data(), d_hist.p, d_hist.bytes, cudaMemcpyDeviceToHost, s));
  int gather_status = 0;
  if (h.status)
    ARB_CUDA(cudaMemcpyAsync(&gather_status, h.status, sizeof(int), cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaStreamSynchronize(s));
  ARB_CHECK(gather_status == 0, "a row gather of the histogram kernel did not arrive within its time limit");
  const int HW = hist_size + 1;
  for (int node = 0; node < n_nodes; ++node)
    for (int f = 0; f < ncol; ++f) {
      const int tile = f / geo.TW, lane = f % geo.TW;
      for (int b = 0; b < HW; ++b) {
        const size_t src = (((size_t(node) * geo.NT + tile) * geo.BINS + b) * geo.TW + lane) * 2;
        const size_t dst = (size_t(node) * ncol + f) * HW + b;
        out_g[dst] = double(host[src]) * q.inv_sg;
        out_h[dst] = double(host[src + 1]) * q.inv_sh;
      }
    }
  ARB_CATCH
}

const char *ABuildHistogram(const void *bins, int bin_bytes, int64_t nrow, int ncol, int hist_size,
                            const float *grad, int pair, const unsigned *rowid,
                            const unsigned *node_begin, int n_nodes, int quant_bits, double *out_g,
                            double *out_h, int reps, float *ms) {
  return build_histogram(bins, bin_bytes, nrow, ncol, hist_size, grad, pair, rowid, node_begin, n_nodes,
                         quant_bits, out_g, out_h, reps, ms, nullptr, nullptr);
}

const char *ABuildHistogramFromParents(const void *bins, int bin_bytes, int64_t nrow, int ncol, int hist_size,
                                       const float *grad, int pair, const unsigned *rowid,
                                       const unsigned *node_begin, int n_nodes, int quant_bits,
                                       const double *parent_g, const double *parent_h, double *out_g,
                                       double *out_h) {
  if (!parent_g || !parent_h) return fail("NULL argument");
  return build_histogram(bins, bin_bytes, nrow, ncol, hist_size, grad, pair, rowid, node_begin, n_nodes,
                         quant_bits, out_g, out_h, 0, nullptr, parent_g, parent_h);
}

const char *APeerWaitProbe(double limit_ms, int *timed_out, double *waited_ms) {
  ARB_TRY
  ARB_CHECK(timed_out && waited_ms, "NULL argument");
  ARB_CHECK(limit_ms > 0 && limit_ms <= 2000, "limit_ms must be in (0, 2000]");
  peer_wait_probe(limit_ms, timed_out, waited_ms);
  ARB_CATCH
}

const char *ANcclUniqueId(char *id128) {
  ARB_TRY
  ARB_CHECK(id128, "NULL argument");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  g_nccl.load();
  ncclUniqueId id;
  const ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != ncclSuccess) throw std::runtime_error(std::string("ncclGetUniqueId: ") + g_nccl.GetErrorString(r));
  std::memcpy(id128, &id, 128);
  ARB_CATCH
}

const char *AInitNccl(VoidPointer garden, int rank, int world, const char *id128) {
  ARB_TRY
  ARB_CHECK(garden, "NULL argument");
  ARB_CHECK(world >= 1 && rank >= 0 && rank < world, "bad rank / world size");
  Garden *g = static_cast<Garden *>(garden);
  ARB_CHECK(g->builder == nullptr, "AInitNccl must precede the first AGrowTree");
  ARB_CHECK(g->allreduce_ctx == nullptr, "the Garden already has a communicator");
  g_nccl.load();
  std::unique_ptr<NcclCtx> c(new NcclCtx());
  if (id128 == nullptr) {  // attach the communicator this process already has
    ARB_CHECK(g_process_comm != nullptr, "no communicator to reuse: pass the ncclUniqueId");
    ARB_CHECK(g_process_world == world && g_process_rank == rank,
              "the process's communicator was made for another rank / world size");
    c->comm = g_process_comm;
    c->shared = true;
  } else {
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    const ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) throw std::runtime_error(std::string("ncclCommInitRank: ") + g_nccl.GetErrorString(r));
    if (g_process_comm == nullptr) {
      g_process_comm = c->comm;
      g_process_world = world;
      g_process_rank = rank;
      c->shared = true;
    }
  }
  g->allreduce = nccl_allreduce;
  g->allreduce_max = nccl_allreduce_max;
  g->comm_check = nccl_check;
  g->shards.rank = rank;
  g->shards.world = world;
  g->shards.allgather = nccl_allgather;
  g->shards.ctx = c.get();
  g->allreduce_ctx = c.release();
  ARB_CATCH
}

}  // extern "C"
