// One-shot push all-reduce of the centroid sums over NVLink peer memory.
//
// The reduction the reference stages through the host (src/gpu/kmeans/kmeans_impl.h:140-188)
// is a few tens of kilobytes per iteration (k * d int64 sums + k counts): latency, not
// bandwidth.  Instead of a library ring, every rank writes its vector straight into a slot
// of every peer's mailbox (plain peer stores), raises a flag there, waits for the flags of
// all ranks in its own mailbox and adds the slots in rank order - one kernel, one NVLink
// crossing.  Sums are integers, so the result is the same bits as any other reduction order.
//   mailbox[2][world][count]   two generations (sequence parity): a rank that runs ahead
//                              writes the next generation while a slower one still reads
//   flags[2][world]            sequence number of the generation a rank has delivered
// Peers are other devices of this process (peer access) or other processes (CUDA IPC
// handles, exchanged once through the NCCL communicator that exists anyway).  Every wait is
// bounded: after `spin_limit` polls (about two seconds by default, see wait_limits()) the kernel
// records an error word and returns, and the host reports KM_ETIMEOUT.  Plain peer loads/stores
// only - no multimem, no TMA.
// A second, single-generation mailbox carries the candidate records of the empty-cluster repair
// (gather_apply_kernel in km_finalize.cuh).
#pragma once

#include <vector>

#include "km_common.cuh"
#include "km_nccl.h"

namespace km {

constexpr int kPushCtas = 16;
constexpr int kPushThreads = 256;
constexpr size_t kPushMaxBytes = (size_t)1 << 20;   // larger vectors stay with NCCL

// Limits of the bounded device-side waits, process-wide.  Defaults: about two seconds for the
// peer-flag polls (40 ns sleep per poll) and about three seconds for the mbarrier waits of the
// tensor-core kernels (parked try_wait of at most 20 us each).  kmeans_set_wait_limits() changes them.
struct WaitLimits {
  unsigned int push_spins = 20000000u;
  unsigned int mbar_iters = 150000u;
};
inline WaitLimits& wait_limits() {
  static WaitLimits w;
  return w;
}

struct PushPeer {
  long long* mailbox = nullptr;    // [2][world][count] of the peer, mapped into this device
  unsigned int* flags = nullptr;   // [2][world] all-reduce flags, then [world] gather flags
  unsigned char* gmail = nullptr;  // [world][gslot] candidate records of the empty-cluster repair
  bool ipc_mailbox = false, ipc_flags = false, ipc_gmail = false;
};

struct PushState {
  bool ready = false;
  size_t count = 0;
  int world = 0;
  long long* mailbox = nullptr;        // this rank's own
  unsigned int* flags = nullptr;
  unsigned int* done = nullptr;        // CTAs of the current launch that finished pushing
  long long** d_peer_mailbox = nullptr;   // device arrays [world]
  unsigned int** d_peer_flags = nullptr;
  unsigned char* gmail = nullptr;         // this rank's gather mailbox
  size_t gslot = 0;                       // bytes of one rank's slot in it
  unsigned char* grec = nullptr;          // this rank's own record, before it is pushed
  unsigned char** d_peer_gmail = nullptr;
  unsigned int** d_peer_gflags = nullptr;
  std::vector<PushPeer> peers;
};

__global__ void __launch_bounds__(kPushThreads)
push_allreduce_kernel(const long long* __restrict__ src, long long* __restrict__ dst, size_t count, int rank, int world,
                      long long* const* __restrict__ peer_mailbox, unsigned int* const* __restrict__ peer_flags,
                      const long long* my_mailbox, const unsigned int* my_flags, unsigned int* done,
                      unsigned int seq, IterState* st, unsigned int spin_limit) {
  __shared__ int s_last, s_bad;
  const unsigned int buf = seq & 1u;
  const size_t total = (size_t)world * count;
  // 1. this rank's vector into slot `rank` of generation `buf` of every mailbox (its own included)
  for (size_t idx = (size_t)blockIdx.x * kPushThreads + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * kPushThreads) {
    const int p = (int)(idx / count);
    const size_t i = idx - (size_t)p * count;
    peer_mailbox[p][((size_t)buf * world + rank) * count + i] = src[i];
  }
  __threadfence_system();
  if (threadIdx.x == 0) { s_last = 0; s_bad = 0; }
  __syncthreads();
  // 2. the CTA that finishes last raises the flags
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(done, 1u);
    if (t == gridDim.x - 1) { s_last = 1; *done = 0; }
  }
  __syncthreads();
  if (s_last && threadIdx.x < world) {
    __threadfence_system();
    *reinterpret_cast<volatile unsigned int*>(peer_flags[threadIdx.x] + (size_t)buf * world + rank) = seq;
    __threadfence_system();
  }
  // 3. wait (bounded) for every rank's delivery into this mailbox
  if (threadIdx.x < world) {
    const volatile unsigned int* f = my_flags + (size_t)buf * world + threadIdx.x;
    unsigned int spins = 0;
    while (*f != seq) {
      if (++spins > spin_limit) { s_bad = 1; break; }
      __nanosleep(40);
    }
  }
  __syncthreads();
  if (s_bad) {
    if (threadIdx.x == 0) atomicMax(&st->error, 11);
    return;
  }
  __threadfence();
  // 4. add the slots in rank order (loads bypass L1: the addresses are reused every other iteration)
  for (size_t i = (size_t)blockIdx.x * kPushThreads + threadIdx.x; i < count; i += (size_t)gridDim.x * kPushThreads) {
    long long v = 0;
    for (int r = 0; r < world; ++r) v += __ldcv(my_mailbox + ((size_t)buf * world + r) * count + i);
    dst[i] = v;
  }
}

}  // namespace km
