// Peer-memory helpers shared by the kernels that talk to other ranks through NVLink-mapped (symmetric) memory:
// system-scope loads / stores, the per-rank flag arrays (`flags[slot * world + rank] = sequence number`), a bounded wait
// for every rank's flag, and a "last block signals" epilogue.  Plain ld / st.global only: no multicast of any kind.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace dewb {
namespace peer {

constexpr int MAX_RANKS = 8;
constexpr int ERR_WAIT_PEER = 5;
constexpr int ERR_BAD_ARG = 6;

struct Peers {
  void* p[MAX_RANKS];
};

static inline Peers make_peers(const unsigned long long* ptrs, int world) {
  Peers r;
  for (int i = 0; i < MAX_RANKS; ++i) r.p[i] = (ptrs != nullptr && i < world) ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return r;
}

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_sys_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ int ld_sys_s32(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until flags[slot * world + r] >= seq for every rank r (sequence numbers only grow; the signed distance
// tolerates wrap-around).  Called by all threads of a block; bounded: after `limit_ns` it records ERR_WAIT_PEER and
// returns false for every thread.
static __device__ bool wait_all_peers(const uint32_t* my_flags, int slot, int world, uint32_t seq,
                                      unsigned long long limit_ns, int* err) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint32_t* f = my_flags + slot * world + threadIdx.x;
    const uint64_t t0 = now_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - seq) < 0) {
      if ((++spins & 63) == 0) {
        if (now_ns() - t0 > limit_ns) { ok_flag = 0; atomicCAS(err, 0, ERR_WAIT_PEER); break; }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// True (for the whole CTA) when an earlier launch has already reported an error: later launches leave at once.
static __device__ bool status_poisoned(const int* err) {
  __shared__ int poisoned;
  if (threadIdx.x == 0) poisoned = *reinterpret_cast<const volatile int*>(err);
  __syncthreads();
  return poisoned != 0;
}

// Called by every thread of every block once the block's peer stores / loads are issued: the block that arrives last at
// `counter` writes `seq` into slot[rank] of every peer's flag array (and resets the counter for the next launch).
static __device__ void last_block_signals(unsigned int* counter, Peers flags, int slot, int rank, int world, uint32_t seq) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int ticket = atomicAdd(counter, 1u);
    is_last = (ticket == gridDim.x - 1) ? 1 : 0;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + slot * world + rank, seq);
  }
}

}  // namespace peer
}  // namespace dewb
