// Arrival flags for the exchange fused into the pre-attention and attention kernels.
//
// Every rank owns one "sync block" of kSyncInts int32 in peer-mapped memory (zero at start).  All
// counters are epochs that advance by one per layer on every rank, kept on the device so that the
// kernels take no per-call argument and replay from a CUDA graph.
//
//   [0, 8]    barrier: one flag per peer, then the local barrier epoch (peer_barrier_kernel)
//   [16, 24)  in_flag[src]    src's q/k/v rows of layer e have landed here     (written by src)
//   [24]      in_epoch        layers this rank has scattered so far            (local)
//   [25]      scatter CTAs that have finished in the running launch           (local)
//   [32, 40)  out_flag[src]   src's output columns of layer e have landed here (written by src)
//   [40]      out_epoch       layers whose outputs this rank has sent          (local)
//   [41]      attention / merge CTAs that have finished in the running launch (local)
//   [42]      wait_epoch      layers whose outputs this rank has waited for    (local)
//   [48, 56)  q_flag[src]     src's QUERY rows of layer e have landed here     (written by src; push mode)
//   [56, 64)  push CTAs that have finished phase i of the running launch      (local; push mode)
//
// Push mode (the exchange overlapped with the attention itself): the pre-attention kernel stores the
// query rows straight into the peers' buffers and announces them (q_flag), but only stages the key
// and value rows for the peers in local memory; copy CTAs that run INSIDE the attention launch push
// those, in the order in which the receivers walk their keys (in_flag).
//
// Publishing uses the last-block pattern: every CTA orders its stores with a device-scope fence and
// bumps the local counter; the CTA that sees the full count issues ONE system-scope fence - which is
// cumulative over everything the counter chain made happen before it - and then writes the new
// epoch into each peer's flag slot with relaxed system-scope stores (fence + relaxed store is the
// release pattern; a release store per peer would wait for the previous peer's flag to be
// acknowledged before sending the next one - a serial chain of NVLink round trips).  (A system-scope fence in
// every CTA was measured to cost tens of microseconds per CTA while peer stores are in flight.)  Every wait is a
// bounded acquire poll that records status 5 and returns when its clock budget runs out.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace chitu {

constexpr int kSyncInts = 64;
constexpr int kSyncInFlag = 16, kSyncInEpoch = 24, kSyncScatterDone = 25;
constexpr int kSyncOutFlag = 32, kSyncOutEpoch = 40, kSyncAttnDone = 41, kSyncWaitEpoch = 42;
constexpr int kSyncQFlag = 48, kSyncPushDone = 56;

struct PeerSync {
  int* blocks[8];  // blocks[i]: rank i's sync block, mapped into this process; null entries past `world`
  int rank, world;
  long long timeout_cycles;
};

__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by ONE thread of every CTA of a launch after a CTA-wide barrier that follows the CTA's last
// peer store.  The CTA that completes the count advances `epoch_slot` and writes the new epoch to
// slot `flag_base + rank` of every peer's block (its own included).
__device__ __forceinline__ void publish_when_last(const PeerSync& ps, int done_slot, int epoch_slot, int flag_base,
                                                  unsigned total_ctas) {
  int* mine = ps.blocks[ps.rank];
  __threadfence();
  const unsigned prev = atomicAdd(reinterpret_cast<unsigned*>(mine + done_slot), 1u);
  if (prev + 1 == total_ctas) {
    __threadfence_system();
    mine[done_slot] = 0;
    const int epoch = mine[epoch_slot] + 1;
    mine[epoch_slot] = epoch;
    for (int i = 0; i < ps.world; ++i) st_relaxed_sys(ps.blocks[i] + flag_base + ps.rank, epoch);
  }
}

// One phase of the push CTAs: called by ONE thread of every push CTA after a CTA-wide barrier that
// follows the CTA's last store of the phase.  The CTA that completes the count tells the peers in the
// bit set `dests` that this rank's rows of the phase have landed.
__device__ __forceinline__ void push_phase_done(const PeerSync& ps, int phase, unsigned total_ctas, int flag_base,
                                                unsigned dests, int epoch) {
  int* mine = ps.blocks[ps.rank];
  __threadfence();
  const unsigned prev = atomicAdd(reinterpret_cast<unsigned*>(mine + kSyncPushDone + phase), 1u);
  if (prev + 1 == total_ctas) {
    __threadfence_system();
    mine[kSyncPushDone + phase] = 0;
    for (int i = 0; i < ps.world; ++i)
      if (i != ps.rank && ((dests >> i) & 1u)) st_relaxed_sys(ps.blocks[i] + flag_base + ps.rank, epoch);
  }
}

// Bounded wait until `*flag` has reached `epoch` (wrap-safe): system-scope acquire polls.  Returns false on
// timeout after recording status 5.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, long long timeout_cycles, int* status) {
  if (ld_acquire_sys(flag) - epoch < 0) {
    const long long t0 = clock64();
    unsigned spins = 0;
    while (ld_acquire_sys(flag) - epoch < 0) {
      if ((++spins & 0x3f) == 0 && clock64() - t0 > timeout_cycles) {
        if (status) atomicCAS(status, 0, 5);
        return false;
      }
    }
  }
  return true;
}

// Measurement aid: the GPU's nanosecond timer at the moment this launch ran.
__global__ void stamp_kernel(unsigned long long* slot) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *slot = t;
}

// One warp: lane i waits for peer i's output flag of the next layer, then the epoch advances.
__global__ void peer_wait_outputs_kernel(const PeerSync ps, int* status) {
  int* mine = ps.blocks[ps.rank];
  const int epoch = mine[kSyncWaitEpoch] + 1;
  __syncwarp();
  if (static_cast<int>(threadIdx.x) < ps.world)
    wait_flag(mine + kSyncOutFlag + threadIdx.x, epoch, ps.timeout_cycles, status);
  __syncwarp();
  if (threadIdx.x == 0) mine[kSyncWaitEpoch] = epoch;
}

}  // namespace chitu
