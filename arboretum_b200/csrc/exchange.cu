// Peer-memory exchange between row shards (see exchange.h).
//
// Protocol of one AllReduce (sequence number q, the same on every rank):
//   1. rank r tells every peer "my send buffer holds level q" (arrive[r] := q in the peer's
//      memory; the buffer was written by the kernel before this one on the stream);
//   2. it waits until every peer has said so (its own arrive[] words, in its own memory);
//   3. it sums slice r of all send buffers (its own and, through NVLink, the peers') and
//      stores the sums into slice r of every rank's result buffer;
//   4. when all its CTAs have done that, it tells every peer "slice r is in your result
//      buffer" (done[r] := q), and waits until every peer has said the same to it.
// After step 4 the kernel ends and the next kernel on the stream reads the complete result.
// A send buffer may be rewritten as soon as the kernel has ended (every peer has read it:
// they all reached step 4); a result buffer is only stored to by peers that have seen this
// rank's arrive[q + 1], which it sends after it has consumed result q.  So one buffer of each
// kind suffices.  Every wait is bounded by a time limit; when it runs out the kernel records
// where, skips the data movement and returns, and the host reports it after the tree.
#include "exchange.h"

#include <cstdlib>
#include <cstring>

namespace arb {

namespace {

typedef unsigned long long u64;

__device__ __forceinline__ u64 ld_acquire_sys(const u64 *p) {
  u64 v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(u64 *p, u64 v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 global_timer_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// true once *flag >= seq; false when `limit_ns` have passed first
__device__ bool wait_flag(const u64 *flag, u64 seq, u64 limit_ns) {
  const u64 t0 = global_timer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(flag) < seq) {
    if ((++spins & 31u) == 0u && global_timer_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
  return true;
}

__global__ void __launch_bounds__(256)
peer_allreduce_kernel(const PeerPointers p, const int rank, const int world, const size_t pairs,
                      const u64 seq, unsigned *counter, int *status, const u64 limit_ns, u64 *clock) {
  __shared__ int ok;
  __shared__ bool last;
  const u64 t_begin = global_timer_ns();
  if (threadIdx.x == 0) ok = 1;
  if (blockIdx.x == 0 && threadIdx.x < world) st_release_sys(&p.arrive[threadIdx.x][rank], seq);
  __syncthreads();
  if (threadIdx.x < world && !wait_flag(&p.arrive[rank][threadIdx.x], seq, limit_ns)) {
    ok = 0;
    atomicCAS(status, 0, 1);
  }
  __syncthreads();
  const u64 t_arrived = global_timer_ns();
  if (ok) {
    const size_t per = (pairs + size_t(world) - 1) / size_t(world);
    const size_t lo = size_t(rank) * per, hi = min(pairs, lo + per);
    for (size_t i = lo + size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
         i += size_t(gridDim.x) * blockDim.x) {
      longlong2 v[kMaxPeers];
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)  // all loads in flight before the first use
        if (q < world) v[q] = __ldcg(reinterpret_cast<const longlong2 *>(p.send[q]) + i);
      longlong2 acc = make_longlong2(0, 0);
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)
        if (q < world) {
          acc.x += v[q].x;
          acc.y += v[q].y;
        }
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)
        if (q < world) __stcg(reinterpret_cast<longlong2 *>(p.recv[q]) + i, acc);
    }
  }
  __syncthreads();  // the CTA's stores are issued ...
  if (threadIdx.x == 0) {
    __threadfence_system();  // ... and ordered, for every observer, before the CTA counts as finished
    last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence_system();  // the other CTAs' stores (seen through the counter) before the flags
  if (threadIdx.x == 0) *counter = 0;
  const u64 t_moved = global_timer_ns();
  if (threadIdx.x < world) {
    st_release_sys(&p.done[threadIdx.x][rank], seq);
    if (!wait_flag(&p.done[rank][threadIdx.x], seq, limit_ns)) atomicCAS(status, 0, 2);
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // where the time of the exchanges goes (read by the host on request)
    clock[0] += t_arrived - t_begin;         // until every peer's buffer was ready
    clock[1] += t_moved - t_arrived;         // this rank's slice summed and stored everywhere
    clock[2] += global_timer_ns() - t_moved; // until every peer had stored its slice here
    clock[3] += 1;
  }
}

// element-wise maximum of n <= 4 words over the ranks; one warp
__global__ void peer_max_kernel(const PeerPointers p, const int rank, const int world, const int n,
                                unsigned *words, const u64 seq, int *status, const u64 limit_ns) {
  const int t = threadIdx.x;
  const int half = int(seq & 1) * world * 4;  // two sets of slots, used in turn
  if (t < world) {
    for (int j = 0; j < n; ++j) __stcg(&p.small[t][half + rank * 4 + j], words[j]);
    __threadfence_system();
    st_release_sys(&p.small_flag[t][rank], seq);
  }
  __syncwarp();
  bool ok = true;
  if (t < world) ok = wait_flag(&p.small_flag[rank][t], seq, limit_ns);
  if (!ok) atomicCAS(status, 0, 3);
  ok = __all_sync(0xffffffffu, ok);
  if (ok && t < n) {
    unsigned m = 0;
    for (int q = 0; q < world; ++q) m = max(m, __ldcg(&p.small[rank][half + q * 4 + t]));
    words[t] = m;
  }
}

__global__ void wait_probe_kernel(const u64 *flag, u64 limit_ns, int *timed_out) {
  *timed_out = wait_flag(flag, 1, limit_ns) ? 0 : 1;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct Layout {
  size_t send, recv, arrive, done, small, small_flag, counter, status, clock, total;
  Layout(size_t bytes, int world) {
    size_t at = 0;
    send = at, at += align256(bytes);
    recv = at, at += align256(bytes);
    arrive = at, at += align256(sizeof(u64) * world);
    done = at, at += align256(sizeof(u64) * world);
    small = at, at += align256(sizeof(unsigned) * 2 * world * 4);
    small_flag = at, at += align256(sizeof(u64) * world);
    counter = at, at += 256;
    status = at, at += 256;
    clock = at, at += 256;
    total = at;
  }
};

u64 wait_limit_ns() {  // ARBORETUM_PEER_WAIT_MS in the environment; 20 s by default
  const char *e = std::getenv("ARBORETUM_PEER_WAIT_MS");
  const double ms = e ? std::atof(e) : 20000.0;
  return u64((ms > 0 ? ms : 20000.0) * 1e6);
}

}  // namespace

PeerExchange *PeerExchange::Acquire(size_t bytes, const ShardInfo &sh, cudaStream_t s) {
  static PeerExchange *kept = nullptr;  // one per process, like its communicator
  if (kept && kept->rank_ == sh.rank && kept->world_ == sh.world && kept->bytes_ >= bytes) return kept;
  // (a smaller one that exists stays mapped: see the header)
  PeerExchange *x = Create(bytes, sh, s);
  if (x) kept = x;
  return x;
}

PeerExchange *PeerExchange::Create(size_t bytes, const ShardInfo &sh, cudaStream_t s) {
  if (!sh.allgather || sh.world < 2 || sh.world > kMaxPeers) return nullptr;
  const int world = sh.world;
  const Layout lay(bytes, world);
  PeerExchange *x = new PeerExchange();  // kept for the life of the process (or leaked with its
                                         // mappings when the set-up fails half way: rare, and
                                         // unmapping could not be agreed with the peers)
  x->rank_ = sh.rank;
  x->world_ = world;
  x->bytes_ = bytes;
  // what every rank contributes: its handle and whether it got this far
  struct Card {
    cudaIpcMemHandle_t handle;
    int ok;
    int pad[15];
  };
  static_assert(sizeof(Card) == 128, "one card per rank");
  Card mine;
  std::memset(&mine, 0, sizeof mine);
  bool ok = cudaMalloc(&x->region_, lay.total) == cudaSuccess;  // not from the pool: pool memory cannot be exported this way
  ok = ok && cudaMemset(x->region_, 0, lay.total) == cudaSuccess;
  ok = ok && cudaIpcGetMemHandle(&mine.handle, x->region_) == cudaSuccess;
  if (!ok) cudaGetLastError();
  mine.ok = ok ? 1 : 0;
  DevBuf d_cards;
  d_cards.alloc(sizeof(Card) * (world + 1));
  ARB_CUDA(cudaMemcpyAsync(d_cards.as<Card>() + world, &mine, sizeof mine, cudaMemcpyHostToDevice, s));
  if (sh.allgather(sh.ctx, d_cards.as<Card>() + world, d_cards.p, sizeof(Card), s) != 0)
    throw std::runtime_error("exchange of the peer-memory handles failed");
  std::vector<Card> cards(world);
  ARB_CUDA(cudaMemcpyAsync(cards.data(), d_cards.p, sizeof(Card) * world, cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaStreamSynchronize(s));
  for (const Card &c : cards) ok = ok && c.ok == 1;
  // second round: could everybody map everybody?  (a rank that cannot must not leave the
  // others waiting for it inside the first exchange)
  for (int q = 0; ok && q < world; ++q) {
    if (q == x->rank_) continue;
    if (cudaIpcOpenMemHandle(&x->peer_region_[q], cards[q].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      x->peer_region_[q] = nullptr;
      ok = false;
    }
  }
  mine.ok = ok ? 1 : 0;
  ARB_CUDA(cudaMemcpyAsync(d_cards.as<Card>() + world, &mine, sizeof mine, cudaMemcpyHostToDevice, s));
  if (sh.allgather(sh.ctx, d_cards.as<Card>() + world, d_cards.p, sizeof(Card), s) != 0)
    throw std::runtime_error("exchange of the peer-memory handles failed");
  ARB_CUDA(cudaMemcpyAsync(cards.data(), d_cards.p, sizeof(Card) * world, cudaMemcpyDeviceToHost, s));
  ARB_CUDA(cudaStreamSynchronize(s));
  for (const Card &c : cards) ok = ok && c.ok == 1;
  if (!ok) return nullptr;  // ~PeerExchange unmaps and frees what exists
  for (int q = 0; q < world; ++q) {
    char *base = static_cast<char *>(q == x->rank_ ? x->region_ : x->peer_region_[q]);
    x->ptrs_.send[q] = reinterpret_cast<long long *>(base + lay.send);
    x->ptrs_.recv[q] = reinterpret_cast<long long *>(base + lay.recv);
    x->ptrs_.arrive[q] = reinterpret_cast<u64 *>(base + lay.arrive);
    x->ptrs_.done[q] = reinterpret_cast<u64 *>(base + lay.done);
    x->ptrs_.small[q] = reinterpret_cast<unsigned *>(base + lay.small);
    x->ptrs_.small_flag[q] = reinterpret_cast<u64 *>(base + lay.small_flag);
  }
  for (int q = world; q < kMaxPeers; ++q) {
    x->ptrs_.send[q] = x->ptrs_.recv[q] = nullptr;
    x->ptrs_.arrive[q] = x->ptrs_.done[q] = x->ptrs_.small_flag[q] = nullptr;
    x->ptrs_.small[q] = nullptr;
  }
  x->d_counter_ = reinterpret_cast<unsigned *>(static_cast<char *>(x->region_) + lay.counter);
  x->d_status_ = reinterpret_cast<int *>(static_cast<char *>(x->region_) + lay.status);
  x->d_clock_ = reinterpret_cast<u64 *>(static_cast<char *>(x->region_) + lay.clock);
  return x;
}

void PeerExchange::AllReduce(size_t count, cudaStream_t s) {
  ARB_CHECK(count % 2 == 0 && count * sizeof(long long) <= bytes_, "exchange larger than its buffers");
  const size_t pairs = count / 2;
  const size_t slice = (pairs + world_ - 1) / world_;
  const int grid = int(std::max<size_t>(1, std::min<size_t>((slice + 255) / 256, size_t(device_sm_count()) * 4)));
  ++seq_;
  peer_allreduce_kernel<<<grid, 256, 0, s>>>(ptrs_, rank_, world_, pairs, seq_, d_counter_, d_status_, wait_limit_ns(),
                                             d_clock_);
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void PeerExchange::AllMax(unsigned *device_words, int n, cudaStream_t s) {
  ARB_CHECK(n >= 1 && n <= 4, "at most four words");
  ++small_seq_;
  peer_max_kernel<<<1, 32, 0, s>>>(ptrs_, rank_, world_, n, device_words, small_seq_, d_status_, wait_limit_ns());
  ARB_CUDA(cudaGetLastError());
  count_launch();
}

void PeerExchange::Clock(double ms[3], long long *exchanges, bool reset) {
  u64 v[4] = {0, 0, 0, 0};
  ARB_CUDA(cudaMemcpy(v, d_clock_, sizeof v, cudaMemcpyDeviceToHost));
  for (int i = 0; i < 3; ++i) ms[i] = double(v[i]) * 1e-6;
  *exchanges = (long long)v[3];
  if (reset) ARB_CUDA(cudaMemset(d_clock_, 0, sizeof v));
}

void peer_wait_probe(double limit_ms, int *timed_out, double *waited_ms) {
  DevBuf d;
  d.alloc(512);
  ARB_CUDA(cudaMemset(d.p, 0, 512));
  u64 *flag = d.as<u64>();
  int *out = reinterpret_cast<int *>(d.as<char>() + 256);
  cudaEvent_t e0, e1;
  ARB_CUDA(cudaEventCreate(&e0));
  ARB_CUDA(cudaEventCreate(&e1));
  ARB_CUDA(cudaEventRecord(e0, nullptr));
  wait_probe_kernel<<<1, 1>>>(flag, u64(limit_ms * 1e6), out);
  ARB_CUDA(cudaEventRecord(e1, nullptr));
  const cudaError_t e = cudaEventSynchronize(e1);
  float ms = 0.0f;
  if (e == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  ARB_CUDA(e);
  ARB_CUDA(cudaMemcpy(timed_out, out, sizeof(int), cudaMemcpyDeviceToHost));
  *waited_ms = ms;
}

int PeerExchange::Status() {
  int v = 0;
  ARB_CUDA(cudaMemcpy(&v, d_status_, sizeof v, cudaMemcpyDeviceToHost));
  return v;
}

}  // namespace arb
