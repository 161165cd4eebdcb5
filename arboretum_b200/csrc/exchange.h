// Exchange of the level histograms between row shards (one process per GPU of one box) over
// peer-mapped device memory: one kernel per level that signals, pulls this rank's slice of
// every peer's buffer through NVLink with plain loads, sums it and stores the sums into every
// peer's result buffer -- a reduce-scatter and an all-gather in one launch, without a
// library call on the level's critical path.  The reference has no multi-GPU path.  The
// messages are 128 KB to a few MB, where a collective library's launch and protocol latency
// dominates; ncclAllReduce remains the path when peer memory cannot be mapped (or with
// ARBORETUM_NO_PEER_EXCHANGE in the environment).  No multicast loads: every remote access is
// an ordinary ld / st on a pointer that cudaIpcOpenMemHandle returned.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <memory>
#include <vector>

#include "common.cuh"
#include "garden.h"

namespace arb {

constexpr int kMaxPeers = 8;

struct PeerPointers {  // by rank; entry `rank` is this rank's own memory
  long long *send[kMaxPeers];
  long long *recv[kMaxPeers];
  unsigned long long *arrive[kMaxPeers];  // [world] per rank: peer p's buffer is ready (sequence number)
  unsigned long long *done[kMaxPeers];    // [world] per rank: peer p has stored its slice here
  unsigned *small[kMaxPeers];             // [world][4] per rank: a few words to take the maximum of
  unsigned long long *small_flag[kMaxPeers];  // [world] per rank
};

class PeerExchange {
 public:
  // The process's exchange for this rank and world size, with room for `bytes` per buffer.
  // The first call (and any call that needs more room than there is) allocates this rank's
  // region (2 x `bytes` + flags), exchanges its handle with the other ranks through
  // `sh.allgather` and maps theirs; every rank must make the same calls.  Like the process's
  // communicator the exchange is kept until the process exits and never unmapped: freeing
  // memory that a peer still has mapped is undefined, and a rank must not wait for its peers
  // while it tears down.  Returns nullptr when any rank could not set it up (every rank then
  // returns nullptr: the decision itself is exchanged).
  static PeerExchange *Acquire(size_t bytes, const ShardInfo &sh, cudaStream_t s);
  long long *send_buffer() const { return ptrs_.send[rank_]; }
  const long long *result_buffer() const { return ptrs_.recv[rank_]; }
  size_t capacity_bytes() const { return bytes_; }
  // Sums `count` int64 words of every rank's send buffer into every rank's result buffer.
  void AllReduce(size_t count, cudaStream_t s);
  // Element-wise maximum over the ranks of up to 4 words at `device_words`, in place.
  void AllMax(unsigned *device_words, int n, cudaStream_t s);
  // 0 = fine; otherwise the step (1: a peer's buffer never became ready, 2: a peer never
  // finished its stores, 3: the few-words exchange) at which a wait ran into its time limit.
  // Reads a word of device memory: call it after the stream has been synchronised.
  int Status();
  const int *device_status() const { return d_status_; }
  // Device time of the AllReduce kernels since the last reset, in milliseconds: waiting for
  // the peers' buffers, moving this rank's slice, waiting for the peers' slices.
  void Clock(double ms[3], long long *exchanges, bool reset);

 private:
  PeerExchange() {}
  ~PeerExchange() {}
  static PeerExchange *Create(size_t bytes, const ShardInfo &sh, cudaStream_t s);
  int rank_ = 0, world_ = 1;
  size_t bytes_ = 0;
  void *region_ = nullptr;               // cudaMalloc'ed, exported
  void *peer_region_[kMaxPeers] = {};    // mapped peers (nullptr at rank_)
  PeerPointers ptrs_;
  unsigned *d_counter_ = nullptr;        // CTAs of the running exchange that have finished
  int *d_status_ = nullptr;
  unsigned long long *d_clock_ = nullptr;
  unsigned long long seq_ = 0, small_seq_ = 0;
};

// The bounded wait of the exchange kernels on a word that nothing ever sets: one thread waits
// `limit_ms`, gives up, and the kernel returns normally.  *timed_out = 1 when the wait ran
// into its limit (it must), *waited_ms = the kernel's device time.
void peer_wait_probe(double limit_ms, int *timed_out, double *waited_ms);

}  // namespace arb
