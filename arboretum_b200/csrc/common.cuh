// Shared host/device utilities of the B200 training core.
#pragma once
#include <cuda_runtime.h>

#include <chrono>
#include <cstring>
#include <cstdio>
#include <cstdlib>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

namespace arb {

// Every CUDA failure becomes a C++ exception; the C-ABI layer turns it into the
// error string the caller receives.  (The reference prints and calls exit():
// src/core/cuda_helpers.h:12-20.)
#define ARB_CUDA(cmd)                                                          \
  do {                                                                         \
    cudaError_t e__ = (cmd);                                                   \
    if (e__ != cudaSuccess) {                                                  \
      throw std::runtime_error(std::string("CUDA error ") +                   \
                               cudaGetErrorString(e__) + " at " + __FILE__ +   \
                               ":" + std::to_string(__LINE__));                \
    }                                                                          \
  } while (0)

#define ARB_CHECK(cond, msg)                                                   \
  do {                                                                         \
    if (!(cond)) throw std::runtime_error(std::string(msg));                   \
  } while (0)

// Owning device allocation.
// Device memory comes from the device's stream-ordered pool, set to keep what is freed:
// cudaMalloc / cudaFree of gigabytes cost milliseconds (and on a busy host tens of them)
// every time a matrix or a model is built, the pool hands a freed block back in
// microseconds.  dev_alloc returns only when the block may be used on any stream;
// dev_free first waits for the device, like cudaFree does.
cudaError_t dev_alloc(void **p, size_t bytes);
void dev_free(void *p);
// free device memory as cudaMemGetInfo reports it, plus what the pool holds unused
cudaError_t dev_available(size_t *bytes);
// give the pool's unused memory back to the driver (and the kept pinned blocks, below)
cudaError_t dev_trim();
// Pinned host memory: cudaMallocHost / cudaFreeHost cost about a millisecond per call, and a
// process that builds one model after another asks for the same few small buffers every time.
// Freed blocks of up to 16 MB are kept (64 MB in all) and handed out again; *cap receives the
// size of the block that was handed out, which pinned_free wants back.
cudaError_t pinned_alloc(void **p, size_t bytes, size_t *cap);
void pinned_free(void *p, size_t cap);

struct DevBuf {
  void *p = nullptr;
  size_t bytes = 0;
  bool owned = true;  // false: a window on another buffer's memory (see view)
  DevBuf() {}
  DevBuf(const DevBuf &) = delete;
  DevBuf &operator=(const DevBuf &) = delete;
  ~DevBuf() { release(); }
  void alloc(size_t n) {
    release();
    if (n == 0) return;
    ARB_CUDA(dev_alloc(&p, n));
    bytes = n;
  }
  // n bytes at `ptr`, owned by someone else who outlives this object
  void view(void *ptr, size_t n) {
    release();
    p = ptr;
    bytes = n;
    owned = false;
  }
  void release() {
    if (p && owned) dev_free(p);
    p = nullptr;
    bytes = 0;
    owned = true;
  }
  template <typename T>
  T *as() const {
    return static_cast<T *>(p);
  }
};

// Owning pinned host allocation.
struct PinnedBuf {
  void *p = nullptr;
  size_t bytes = 0;
  size_t cap = 0;  // size of the block behind p (>= bytes), when owned
  bool owned = true;
  PinnedBuf() {}
  PinnedBuf(const PinnedBuf &) = delete;
  PinnedBuf &operator=(const PinnedBuf &) = delete;
  ~PinnedBuf() { release(); }
  void alloc(size_t n) {
    release();
    if (n == 0) return;
    ARB_CUDA(pinned_alloc(&p, n, &cap));
    bytes = n;
  }
  void view(void *ptr, size_t n) {
    release();
    p = ptr;
    bytes = n;
    owned = false;
  }
  void release() {
    if (p && owned) pinned_free(p, cap);
    p = nullptr;
    bytes = 0;
    cap = 0;
    owned = true;
  }
  template <typename T>
  T *as() const {
    return static_cast<T *>(p);
  }
};

static inline int ceil_div(int64_t a, int64_t b) { return int((a + b - 1) / b); }

// Per-device facts are cached by device ordinal: one process may drive several devices, and
// what was asked of the first says nothing about the second.
constexpr int kMaxDevices = 64;
inline int current_device() {
  int dev = 0;
  ARB_CUDA(cudaGetDevice(&dev));
  ARB_CHECK(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
  return dev;
}
inline int device_sm_count() {
  static int sms[kMaxDevices] = {};
  const int dev = current_device();
  if (!sms[dev]) ARB_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
  return sms[dev];
}

// Kernels of this library launched so far in this process (reported by AGetTimings).
extern long long g_kernel_launches;
static inline void count_launch(int n = 1) { g_kernel_launches += n; }

// Programmatic dependent launch: a kernel launched with launch_overlapped() may be put on
// the SMs while the kernel before it on the stream still runs, so that its launch latency
// and whatever it does before overlap_wait() (clearing shared memory, index arithmetic)
// hide behind that kernel's tail.  overlap_wait() returns once the earlier kernel has
// finished and its writes are visible: every kernel launched this way calls it before its
// first access to global memory.  overlap_release() lets the next kernel on the stream
// start its own preamble; that kernel's overlap_wait() still waits for this whole grid.
// ARBORETUM_NO_LAUNCH_OVERLAP in the environment turns the launches back into plain ones.
#ifdef __CUDACC__
__device__ __forceinline__ void overlap_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void overlap_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool launch_overlap_enabled() {
  static const bool on = std::getenv("ARBORETUM_NO_LAUNCH_OVERLAP") == nullptr;
  return on;
}

template <typename... P, typename... A>
inline void launch_overlapped(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_overlap_enabled() ? 1 : 0;
  ARB_CUDA(cudaLaunchKernelEx(&cfg, kernel, P(args)...));
}
#endif

// Host-side stage timer of the set-up paths: with ARBORETUM_TRACE set in the environment,
// lap("name") synchronises the device and prints the wall time since the previous lap.
struct StageTrace {
  bool on, sync;
  std::chrono::steady_clock::time_point t;
  const char *scope;
  // ARBORETUM_TRACE=host: the host's own time per stage, without waiting for the device
  explicit StageTrace(const char *scope_name)
      : on(std::getenv("ARBORETUM_TRACE") != nullptr),
        sync(on && std::strcmp(std::getenv("ARBORETUM_TRACE"), "host") != 0),
        t(std::chrono::steady_clock::now()),
        scope(scope_name) {}
  void lap(const char *what) {
    if (!on) return;
    if (sync) cudaDeviceSynchronize();
    const auto now = std::chrono::steady_clock::now();
    std::fprintf(stderr, "[arboretum] %s: %s %.3f ms\n", scope, what,
                 std::chrono::duration<double, std::milli>(now - t).count());
    t = now;
  }
};

// ---------------------------------------------------------------------------
// Device-side records of the level loop.
// ---------------------------------------------------------------------------

// Best split of one node at one level.  Sums are the fixed-point integers the
// histograms are built from (see hist.cu); `fid < 0` means "no split: all rows
// go left" (hist_tree_grower.cu:84-93 of the reference).
struct NodeRec {
  float gain;
  int fid;
  int bin;
  unsigned left_count;  // rows that went left (filled by the level's plan kernel from the
                        // descend step's counts)
  long long lg, lh;     // left child sums
  long long tg, th;     // node totals
  unsigned lcnt, tcnt;  // rows left of the split / in the node, from the count histogram that
                        // (gradient, hessian) objectives keep when min_leaf_size > 1; else 0
};

// A contiguous piece of one node's row list, the unit of work of the histogram
// kernels.
struct WorkItem {
  unsigned begin;  // first position in the level's row list (or first row, at the root)
  unsigned len;
  int node;        // node index inside its level
  int pad;
};

// Scales of the per-round fixed-point gradient representation:
// g_q = rint(g * sg), h_q = max(1, rint(h * sh)); sums convert back with
// inv_sg / inv_sh (both scales are powers of two, so this is exact).
struct QuantScale {
  float sg, sh;
  double inv_sg, inv_sh;
  unsigned max_g_bits, max_h_bits;  // float bit patterns, written by atomicMax
  // reg:linear, whose targets may have outliers: tail[j] = rows with |g| >= max|g| / 2^(j + 1).
  // From them follows a bound on the sum of the |g| of ANY 2^(31 - quant_bits) rows -- what an
  // int32 sub-histogram must hold -- that is far below rows x max|g| when the largest
  // gradients are few, and the scale is taken from that bound: up to `extra_bits` more bits
  // for every gradient.  neg_s = 1024 - log2(sg): row shards agree on the coarsest scale with
  // the element-wise maximum they already exchange.
  unsigned neg_s;
  int lim_g;  // |g_q| <= lim_g
  unsigned tail[8];
};
constexpr int kTailLevels = 8;

}  // namespace arb
