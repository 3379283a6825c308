// Fused gradient reduce-scatter + sharded AdamW + parameter all-gather over NVLink peer memory, in ONE kernel.
//
// Every rank holds, per FSDP unit, a full fp32 gradient buffer and a full bf16 parameter buffer in symmetric
// (peer-mapped) memory, and owns one contiguous shard of the fp32 master weights and Adam moments. After a unit's
// backward, each rank launches this kernel, which
//   1. tells its peers "my gradients for this unit are complete" (release store of a sequence number into each
//      peer's flag array) and waits, with a time limit, for the same word from every peer;
//   2. for its own shard: pulls the W partial gradients straight from the peers' buffers with plain P2P loads,
//      sums them in fp32, applies the scale / clip coefficient and the AdamW update to master, m and v;
//   3. rounds the new weights to bf16 and pushes them into every rank's full parameter buffer (P2P stores), so no
//      separate all-gather follows;
//   4. when the last block finishes, tells the peers "my shard is pushed and I no longer read your gradients".
// Nothing here uses TMA or cluster multicast; peer access is ld/st.global through NVSwitch.
//
// Replaces, for the FSDP axis, the collectives XLA inserts around the optimizer in the reference
// (src/dew/mesh.py:101-146 leading-dim shards; src/dew/training/transaction.py:1292-1392 commit).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace dewb {
namespace comm {

constexpr int MAX_RANKS = 8;

struct Peers {
  void* p[MAX_RANKS];
};

enum : int { ERR_WAIT_PEER = 5 };

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
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

// Wait until flags[slot * world + r] >= seq for every rank r. Bounded: gives up after `limit_ns` and reports.
// Called by all threads of a block; returns false (for every thread) on time-out.
__device__ bool wait_all_peers(const uint32_t* my_flags, int slot, int world, uint32_t seq, unsigned long long limit_ns,
                               int* err) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint32_t* f = my_flags + slot * world + threadIdx.x;
    const uint64_t t0 = now_ns();
    uint32_t spins = 0;
    // sequence numbers only grow; signed distance tolerates wrap-around
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

// True (for the whole CTA) when an earlier launch has already reported a timed-out wait: later launches leave at once
// instead of each waiting out its own limit.
__device__ bool status_poisoned(const int* err) {
  __shared__ int poisoned;
  if (threadIdx.x == 0) poisoned = *reinterpret_cast<const volatile int*>(err);
  __syncthreads();
  return poisoned != 0;
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, ema_decay;
};

// mode 0: reduce + AdamW + push (fully fused)
// mode 1: reduce only -> reduced[shard_len] (fp32) and per-block sum of squares -> sumsq[gridDim.x]
// mode 2: AdamW from `reduced` (summed, not yet scaled: grad_scale is applied here) + push; `clip` gives
//         {sum sq, norm, coefficient} computed between the two phases
// mode 3: reduce and ADD into reduced[shard_len] (gradient accumulation over microbatches on the shard alone); like mode 0
//         it tells every peer at the end that this rank is done reading their buffers, so they may reuse them
__global__ void __launch_bounds__(512)
rs_adamw_ag_kernel(Peers grads, Peers params, Peers flags, float* __restrict__ master, float* __restrict__ m,
                   float* __restrict__ v, float* __restrict__ ema, float* __restrict__ reduced,
                   float* __restrict__ sumsq, const float* __restrict__ clip, long long shard_begin,
                   long long shard_len, long long decay_end, int rank, int world, AdamArgs a, uint32_t seq,
                   int slot_ready, int slot_done, unsigned int* __restrict__ block_counter,
                   unsigned long long limit_ns, int mode, int skip_nonfinite, int* __restrict__ err) {
  if (status_poisoned(err)) return;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(flags.p[rank]);
  if (mode != 2) {
    // 1. announce + wait: every peer's gradient buffer for this unit is final
    if (blockIdx.x == 0 && threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + slot_ready * world + rank, seq);
    }
    if (!wait_all_peers(my_flags, slot_ready, world, seq, limit_ns, err)) return;
  }
  float coef = a.grad_scale;
  bool skip = false;
  if (mode == 2 && clip != nullptr) {
    if (skip_nonfinite && !isfinite(clip[0])) skip = true;
    coef *= clip[2];
  }
  float local_sq = 0.f;
  const long long nvec = shard_len >> 3;   // 8 elements per thread-iteration; shard_len is a multiple of 8
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long off = i << 3;
    float g[8];
    if (mode == 2) {
      const float4 r0 = *reinterpret_cast<const float4*>(reduced + off);
      const float4 r1 = *reinterpret_cast<const float4*>(reduced + off + 4);
      g[0] = r0.x; g[1] = r0.y; g[2] = r0.z; g[3] = r0.w; g[4] = r1.x; g[5] = r1.y; g[6] = r1.z; g[7] = r1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.f;
      for (int r = 0; r < world; ++r) {
        const float* src = reinterpret_cast<const float*>(grads.p[r]) + shard_begin + off;
        const float4 x0 = ld_sys_f4(src), x1 = ld_sys_f4(src + 4);
        g[0] += x0.x; g[1] += x0.y; g[2] += x0.z; g[3] += x0.w; g[4] += x1.x; g[5] += x1.y; g[6] += x1.z; g[7] += x1.w;
      }
    }
    if (mode == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) local_sq += g[j] * g[j];
      *reinterpret_cast<float4*>(reduced + off) = make_float4(g[0], g[1], g[2], g[3]);
      *reinterpret_cast<float4*>(reduced + off + 4) = make_float4(g[4], g[5], g[6], g[7]);
      continue;
    }
    if (mode == 3) {
      float4 r0 = *reinterpret_cast<const float4*>(reduced + off), r1 = *reinterpret_cast<const float4*>(reduced + off + 4);
      r0.x += g[0]; r0.y += g[1]; r0.z += g[2]; r0.w += g[3]; r1.x += g[4]; r1.y += g[5]; r1.z += g[6]; r1.w += g[7];
      *reinterpret_cast<float4*>(reduced + off) = r0;
      *reinterpret_cast<float4*>(reduced + off + 4) = r1;
      continue;
    }
    float p[8], mm[8], vv[8];
    {
      const float4 p0 = *reinterpret_cast<const float4*>(master + off), p1 = *reinterpret_cast<const float4*>(master + off + 4);
      const float4 m0 = *reinterpret_cast<const float4*>(m + off), m1 = *reinterpret_cast<const float4*>(m + off + 4);
      const float4 v0 = *reinterpret_cast<const float4*>(v + off), v1 = *reinterpret_cast<const float4*>(v + off + 4);
      p[0] = p0.x; p[1] = p0.y; p[2] = p0.z; p[3] = p0.w; p[4] = p1.x; p[5] = p1.y; p[6] = p1.z; p[7] = p1.w;
      mm[0] = m0.x; mm[1] = m0.y; mm[2] = m0.z; mm[3] = m0.w; mm[4] = m1.x; mm[5] = m1.y; mm[6] = m1.z; mm[7] = m1.w;
      vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
    }
    if (!skip) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gi = g[j] * coef;
        mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gi;
        vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gi * gi;
        const float wd = (shard_begin + off + j) < decay_end ? a.wd : 0.f;
        p[j] = p[j] * (1.f - a.lr * wd) - a.lr * (mm[j] / a.bc1) / (sqrtf(vv[j] / a.bc2) + a.eps);
      }
      *reinterpret_cast<float4*>(master + off) = make_float4(p[0], p[1], p[2], p[3]);
      *reinterpret_cast<float4*>(master + off + 4) = make_float4(p[4], p[5], p[6], p[7]);
      *reinterpret_cast<float4*>(m + off) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(m + off + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
      *reinterpret_cast<float4*>(v + off) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(v + off + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
      if (ema != nullptr) {
        float4 e0 = *reinterpret_cast<const float4*>(ema + off), e1 = *reinterpret_cast<const float4*>(ema + off + 4);
        const float d = a.ema_decay, c = 1.f - a.ema_decay;
        e0.x = d * e0.x + c * p[0]; e0.y = d * e0.y + c * p[1]; e0.z = d * e0.z + c * p[2]; e0.w = d * e0.w + c * p[3];
        e1.x = d * e1.x + c * p[4]; e1.y = d * e1.y + c * p[5]; e1.z = d * e1.z + c * p[6]; e1.w = d * e1.w + c * p[7];
        *reinterpret_cast<float4*>(ema + off) = e0;
        *reinterpret_cast<float4*>(ema + off + 4) = e1;
      }
    }
    // 3. push the bf16 weights into every rank's full parameter buffer
    uint4 pk;
    pk.x = pack_bf16(p[0], p[1]); pk.y = pack_bf16(p[2], p[3]); pk.z = pack_bf16(p[4], p[5]); pk.w = pack_bf16(p[6], p[7]);
    for (int r = 0; r < world; ++r) {
      const int dst = (rank + r) % world;   // stagger destinations so ranks do not all hit the same peer at once
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[dst]) + shard_begin + off) = pk;
    }
  }
  if (mode == 1) {
    __shared__ float red[32];
    float s = local_sq;
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (threadIdx.x == 0) sumsq[blockIdx.x] = t;
    }
  }
  // 4. last block out tells every peer that this rank is done with the unit
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int ticket;
  if (threadIdx.x == 0) ticket = atomicAdd(block_counter, 1u);
  __syncthreads();
  if (ticket == gridDim.x - 1) {
    if (threadIdx.x == 0) *block_counter = 0;
    if (mode != 1 && threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + slot_done * world + rank, seq);
    }
  }
}

// Stand-alone bounded wait on one flag slot (used before a unit's forward: all peers have pushed its new weights).
__global__ void wait_flags_kernel(const uint32_t* my_flags, int slot, int world, uint32_t seq,
                                  unsigned long long limit_ns, int* err) {
  if (status_poisoned(err)) return;
  wait_all_peers(my_flags, slot, world, seq, limit_ns, err);
}

// Stand-alone signal: write seq into slot[rank] of every peer's flag array.
__global__ void signal_flags_kernel(Peers flags, int slot, int rank, int world, uint32_t seq) {
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + slot * world + rank, seq);
  }
}

// All-gather by pull: dst[r * shard_len + i] = peer r's src[i]  (bf16 or any 16-byte-multiple payload).
__global__ void allgather_pull_kernel(Peers src, uint4* __restrict__ dst, long long shard_vec, int world) {
  const long long total = shard_vec * world;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / shard_vec);
    const long long j = i - r * shard_vec;
    dst[i] = ld_sys_u4(reinterpret_cast<const uint4*>(src.p[r]) + j);
  }
}

// All-reduce (sum) of a small fp32 vector by pull: out[i] = sum_r peer r's src[i]
__global__ void allreduce_pull_f32_kernel(Peers src, float* __restrict__ out, int n, int world) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int r = 0; r < world; ++r) {
    float x;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(x) : "l"(reinterpret_cast<const float*>(src.p[r]) + i) : "memory");
    s += x;
  }
  out[i] = s;
}

}  // namespace comm
}  // namespace dewb

using namespace dewb::comm;

static Peers make_peers(const unsigned long long* ptrs, int world) {
  Peers p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

// hyper: {lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, ema_decay}
extern "C" int dewb_rs_adamw_ag(const unsigned long long* grad_ptrs, const unsigned long long* param_ptrs,
                                const unsigned long long* flag_ptrs, float* master, float* m, float* v, float* ema,
                                float* reduced, float* sumsq, const float* clip, long long shard_begin,
                                long long shard_len, long long decay_end, int rank, int world, const float* hyper,
                                unsigned int seq, int slot_ready, int slot_done, unsigned int* block_counter,
                                unsigned long long limit_ns, int mode, int skip_nonfinite, int blocks, int* err,
                                void* stream) {
  if (world < 1 || world > MAX_RANKS || (shard_len & 7) || (shard_begin & 7)) return -3;
  AdamArgs a{hyper[0], hyper[1], hyper[2], hyper[3], hyper[4], hyper[5], hyper[6], hyper[7], hyper[8]};
  if (blocks <= 0) blocks = 64;
  rs_adamw_ag_kernel<<<blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(grad_ptrs, world), make_peers(param_ptrs, world), make_peers(flag_ptrs, world), master, m, v, ema,
      reduced, sumsq, clip, shard_begin, shard_len, decay_end, rank, world, a, seq, slot_ready, slot_done,
      block_counter, limit_ns, mode, skip_nonfinite, err);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dewb_wait_flags(const void* my_flags, int slot, int world, unsigned int seq, unsigned long long limit_ns,
                               int* err, void* stream) {
  wait_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint32_t*>(my_flags),
                                                                          slot, world, seq, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dewb_signal_flags(const unsigned long long* flag_ptrs, int slot, int rank, int world, unsigned int seq,
                                 void* stream) {
  signal_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_peers(flag_ptrs, world), slot, rank,
                                                                            world, seq);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dewb_allgather_pull(const unsigned long long* src_ptrs, void* dst, long long shard_bytes, int world,
                                   int blocks, void* stream) {
  if (shard_bytes & 15) return -3;
  if (blocks <= 0) blocks = 64;
  allgather_pull_kernel<<<blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(src_ptrs, world), reinterpret_cast<uint4*>(dst), shard_bytes >> 4, world);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dewb_allreduce_pull_f32(const unsigned long long* src_ptrs, float* out, int n, int world, void* stream) {
  allreduce_pull_f32_kernel<<<(n + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(src_ptrs, world), out, n, world);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------
// One-shot all-reduce over peer memory with an optional fused "+ residual, RMSNorm" epilogue (tensor-parallel decode):
// every rank has written its partial [rows, d] (bf16) into its symmetric buffer; the kernel announces that, waits
// (bounded) for every peer, then each CTA sums one row across the W buffers in fp32, adds the residual stream, writes
// the new stream, and - in the same pass - normalises it for the next layer.
// Buffers alternate by sequence parity, so a rank may start writing the next partial as soon as this kernel returns.
namespace dewb {
namespace comm {

__global__ void __launch_bounds__(256)
allreduce_rows_kernel(Peers bufs, Peers flags, const __nv_bfloat16* __restrict__ partial,
                      const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ norm_w,
                      __nv_bfloat16* __restrict__ sum_out, __nv_bfloat16* __restrict__ norm_out, int rows, int d,
                      float eps, int rank, int world, uint32_t* __restrict__ seq_counter,
                      unsigned int* __restrict__ arrive_counter, long long half_stride, int slot,
                      unsigned long long limit_ns, int* __restrict__ err) {
  __shared__ float red[32];
  __shared__ unsigned int ticket;
  if (status_poisoned(err)) return;
  // The sequence number lives on the device (so a captured CUDA graph can replay this launch): every CTA reads it
  // before any CTA can have advanced it, because it is advanced by the last CTA to leave.
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(seq_counter) + 1;
  const long long half = (seq & 1) ? half_stride : 0;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(flags.p[rank]);
  const int nvec0 = d >> 3;
  // 1. stage this rank's partial rows into its symmetric buffer (the parity half of this sequence number)
  {
    uint4* mine = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[rank]) + half);
    for (int row = blockIdx.x; row < rows; row += gridDim.x)
      for (int i = threadIdx.x; i < nvec0; i += blockDim.x)
        mine[static_cast<long long>(row) * nvec0 + i] = reinterpret_cast<const uint4*>(partial + static_cast<long long>(row) * d)[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence_system(); ticket = atomicAdd(arrive_counter, 1u); }
  __syncthreads();
  if (ticket == gridDim.x - 1) {
    // the last CTA to finish staging announces the whole buffer to every rank (itself included)
    if (threadIdx.x == 0) *arrive_counter = 0;
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + slot * world + rank, seq);
    }
  }
  if (!wait_all_peers(my_flags, slot, world, seq, limit_ns, err)) return;
  const int nvec = d >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float ss = 0.f;
    // d <= 256 * 8 * 4 = 8192: each thread keeps up to 4 vectors of the row
    float acc[4][8];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = threadIdx.x + c * 256;
      if (i < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[c][j] = 0.f;
        // all peers' vectors are requested before any is used: one round trip over NVLink, not `world` of them
        uint4 pv[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < world)
            pv[r] = ld_sys_u4(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[(rank + r) % world]) + half + static_cast<long long>(row) * d) + i);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < world) {
            const uint4 v = pv[r];
            acc[c][0] += __uint_as_float(v.x << 16); acc[c][1] += __uint_as_float(v.x & 0xffff0000u);
            acc[c][2] += __uint_as_float(v.y << 16); acc[c][3] += __uint_as_float(v.y & 0xffff0000u);
            acc[c][4] += __uint_as_float(v.z << 16); acc[c][5] += __uint_as_float(v.z & 0xffff0000u);
            acc[c][6] += __uint_as_float(v.w << 16); acc[c][7] += __uint_as_float(v.w & 0xffff0000u);
          }
        if (residual != nullptr) {
          const uint4 v = reinterpret_cast<const uint4*>(residual + static_cast<long long>(row) * d)[i];
          acc[c][0] += __uint_as_float(v.x << 16); acc[c][1] += __uint_as_float(v.x & 0xffff0000u);
          acc[c][2] += __uint_as_float(v.y << 16); acc[c][3] += __uint_as_float(v.y & 0xffff0000u);
          acc[c][4] += __uint_as_float(v.z << 16); acc[c][5] += __uint_as_float(v.z & 0xffff0000u);
          acc[c][6] += __uint_as_float(v.w << 16); acc[c][7] += __uint_as_float(v.w & 0xffff0000u);
        }
        uint4 pk;
        pk.x = pack_bf16(acc[c][0], acc[c][1]); pk.y = pack_bf16(acc[c][2], acc[c][3]);
        pk.z = pack_bf16(acc[c][4], acc[c][5]); pk.w = pack_bf16(acc[c][6], acc[c][7]);
        if (sum_out != nullptr) reinterpret_cast<uint4*>(sum_out + static_cast<long long>(row) * d)[i] = pk;
        // normalise what was stored (bf16-rounded), as the stand-alone stream norm does
        acc[c][0] = __uint_as_float(pk.x << 16); acc[c][1] = __uint_as_float(pk.x & 0xffff0000u);
        acc[c][2] = __uint_as_float(pk.y << 16); acc[c][3] = __uint_as_float(pk.y & 0xffff0000u);
        acc[c][4] = __uint_as_float(pk.z << 16); acc[c][5] = __uint_as_float(pk.z & 0xffff0000u);
        acc[c][6] = __uint_as_float(pk.w << 16); acc[c][7] = __uint_as_float(pk.w & 0xffff0000u);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += acc[c][j] * acc[c][j];
      }
    }
    if (norm_out == nullptr) continue;   // (uniform over the block)
    // block sum
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = (threadIdx.x & 31) < 8 ? red[threadIdx.x & 31] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    const float rstd = rsqrtf(t / d + eps);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = threadIdx.x + c * 256;
      if (i < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(norm_w)[i];
        const float w[8] = {__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xffff0000u), __uint_as_float(wv.y << 16),
                            __uint_as_float(wv.y & 0xffff0000u), __uint_as_float(wv.z << 16), __uint_as_float(wv.z & 0xffff0000u),
                            __uint_as_float(wv.w << 16), __uint_as_float(wv.w & 0xffff0000u)};
        uint4 pk;
        pk.x = pack_bf16(acc[c][0] * rstd * w[0], acc[c][1] * rstd * w[1]); pk.y = pack_bf16(acc[c][2] * rstd * w[2], acc[c][3] * rstd * w[3]);
        pk.z = pack_bf16(acc[c][4] * rstd * w[4], acc[c][5] * rstd * w[5]); pk.w = pack_bf16(acc[c][6] * rstd * w[6], acc[c][7] * rstd * w[7]);
        reinterpret_cast<uint4*>(norm_out + static_cast<long long>(row) * d)[i] = pk;
      }
    }
  }
  // 3. the last CTA to leave advances the sequence number for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(arrive_counter + 1, 1u);
    if (t == gridDim.x - 1) { arrive_counter[1] = 0; __threadfence(); *seq_counter = seq; }
  }
}


// Two-shot form of the same operation, for the latency-bound decode step and the bandwidth-bound prefill alike:
//   1. every rank PUSHES each row of its partial into the slot [its rank] of the row's owner (rows are dealt to ranks in
//      contiguous blocks of R = ceil(rows / world)); when its last CTA has pushed, it tells every peer (flag phase 1);
//   2. the owner sums the `world` slots of each of its rows in fp32 (all slots requested before any is used), adds the
//      residual, rounds to bf16, normalises, and pushes the sum row and the normalised row into EVERY rank's output
//      regions; when its last reducing CTA is done, it tells every peer (flag phase 2);
//   3. that CTA waits for every peer's phase-2 word, so the kernel ends only when this rank's outputs are complete.
// Per rank 2 * (W - 1) / W of the tensor crosses NVLink once for the sum (and as much again for the normalised copy),
// where the one-shot form pulls (W - 1) whole tensors.  The outputs live in peer-visible memory: `sum_off` / `norm_off`
// (elements, same on every rank) are chosen by the host, which alternates regions from call to call.
__global__ void __launch_bounds__(512)
allreduce_rows_2shot_kernel(Peers bufs, Peers flags, const __nv_bfloat16* __restrict__ partial,
                            const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ norm_w,
                            int rows, int d, float eps, int rank, int world, uint32_t* __restrict__ counters,
                            long long slots_off, long long sum_off, long long norm_off, int flag_base,
                            unsigned long long limit_ns, int* __restrict__ err) {
  __shared__ float red[32];
  __shared__ unsigned int ticket;
  if (status_poisoned(err)) return;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(counters) + 1;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(flags.p[rank]) + flag_base;
  const int nvec = d >> 3;
  const int R = (rows + world - 1) / world;
  // 1. push every row of the partial to its owner
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int owner = row / R;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[owner]) + slots_off +
                                          (static_cast<long long>(rank) * R + (row - owner * R)) * d);
    const uint4* src = reinterpret_cast<const uint4*>(partial + static_cast<long long>(row) * d);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
  }
  // the block's stores are ordered before the barrier, and thread 0's system-scope fence after it is cumulative over them
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence_system(); ticket = atomicAdd(counters + 1, 1u); }
  __syncthreads();
  if (ticket == gridDim.x - 1) {
    if (threadIdx.x == 0) counters[1] = 0;
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + flag_base + rank, seq);
    }
  }
  // 2. the owner's CTAs reduce their rows and push the results to every rank
  int my_rows = rows - rank * R;
  my_rows = my_rows < 0 ? 0 : (my_rows > R ? R : my_rows);
  const int reducers = my_rows < 1 ? 1 : (my_rows < static_cast<int>(gridDim.x) ? my_rows : static_cast<int>(gridDim.x));
  if (static_cast<int>(blockIdx.x) >= reducers) return;
  if (!wait_all_peers(my_flags, 0, world, seq, limit_ns, err)) return;
  const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(bufs.p[rank]) + slots_off;
  for (int lr = blockIdx.x; lr < my_rows; lr += gridDim.x) {
    const long long row = static_cast<long long>(rank) * R + lr;
    float acc[2][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int i = threadIdx.x + c * 512;
      if (i < nvec) {
        uint4 pv[MAX_RANKS + 1];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < world) pv[r] = ld_sys_u4(reinterpret_cast<const uint4*>(slots + (static_cast<long long>(r) * R + lr) * d) + i);
        if (residual != nullptr) pv[MAX_RANKS] = ld_sys_u4(reinterpret_cast<const uint4*>(residual + row * d) + i);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[c][j] = 0.f;
#pragma unroll
        for (int r = 0; r <= MAX_RANKS; ++r)
          if (r < world || (r == MAX_RANKS && residual != nullptr)) {
            const uint4 v = pv[r];
            acc[c][0] += __uint_as_float(v.x << 16); acc[c][1] += __uint_as_float(v.x & 0xffff0000u);
            acc[c][2] += __uint_as_float(v.y << 16); acc[c][3] += __uint_as_float(v.y & 0xffff0000u);
            acc[c][4] += __uint_as_float(v.z << 16); acc[c][5] += __uint_as_float(v.z & 0xffff0000u);
            acc[c][6] += __uint_as_float(v.w << 16); acc[c][7] += __uint_as_float(v.w & 0xffff0000u);
          }
        uint4 pk;
        pk.x = pack_bf16(acc[c][0], acc[c][1]); pk.y = pack_bf16(acc[c][2], acc[c][3]);
        pk.z = pack_bf16(acc[c][4], acc[c][5]); pk.w = pack_bf16(acc[c][6], acc[c][7]);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < world)
            reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[(rank + r) % world]) + sum_off + row * d)[i] = pk;
        // the norm sees what was stored (bf16-rounded), as the stand-alone stream norm does
        acc[c][0] = __uint_as_float(pk.x << 16); acc[c][1] = __uint_as_float(pk.x & 0xffff0000u);
        acc[c][2] = __uint_as_float(pk.y << 16); acc[c][3] = __uint_as_float(pk.y & 0xffff0000u);
        acc[c][4] = __uint_as_float(pk.z << 16); acc[c][5] = __uint_as_float(pk.z & 0xffff0000u);
        acc[c][6] = __uint_as_float(pk.w << 16); acc[c][7] = __uint_as_float(pk.w & 0xffff0000u);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += acc[c][j] * acc[c][j];
      }
    }
    if (norm_w == nullptr) continue;   // (uniform over the block)
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = (threadIdx.x & 31) < 16 ? red[threadIdx.x & 31] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    const float rstd = rsqrtf(t / d + eps);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int i = threadIdx.x + c * 512;
      if (i < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(norm_w)[i];
        const float w[8] = {__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xffff0000u), __uint_as_float(wv.y << 16),
                            __uint_as_float(wv.y & 0xffff0000u), __uint_as_float(wv.z << 16), __uint_as_float(wv.z & 0xffff0000u),
                            __uint_as_float(wv.w << 16), __uint_as_float(wv.w & 0xffff0000u)};
        uint4 pk;
        pk.x = pack_bf16(acc[c][0] * rstd * w[0], acc[c][1] * rstd * w[1]); pk.y = pack_bf16(acc[c][2] * rstd * w[2], acc[c][3] * rstd * w[3]);
        pk.z = pack_bf16(acc[c][4] * rstd * w[4], acc[c][5] * rstd * w[5]); pk.w = pack_bf16(acc[c][6] * rstd * w[6], acc[c][7] * rstd * w[7]);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < world)
            reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[(rank + r) % world]) + norm_off + row * d)[i] = pk;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence_system(); ticket = atomicAdd(counters + 2, 1u); }
  __syncthreads();
  if (ticket != static_cast<unsigned int>(reducers) - 1) return;
  // 3. the last reducing CTA: tell every peer, wait for every peer, advance the sequence number
  if (threadIdx.x == 0) counters[2] = 0;
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + flag_base + world + rank, seq);
  }
  if (!wait_all_peers(my_flags + world, 0, world, seq, limit_ns, err)) return;
  if (threadIdx.x == 0) { __threadfence(); *reinterpret_cast<volatile uint32_t*>(counters) = seq; }
}


// ---------------------------------------------------------------------------------------------------------------------
// Low-latency form for the decode step (a few hundred rows): the same two shots, but every 16-byte store carries its own
// arrival flag - {2 bf16, seq, 2 bf16, seq} - so a receiver polls the data it needs and no fence, flag store or ticket sits
// between the phases (each 8-byte half of an aligned 16-byte store arrives whole).  Twice the bytes, a third of the latency.
//   1. every rank pushes each row of its partial, in that format, into slot [its rank] of the row's owner;
//   2. the owner polls the `world` slots of each of its rows, sums in fp32, adds the residual, rounds to bf16 and pushes the
//      sum row, in that format, to every rank (itself included);
//   3. every rank polls the sum rows, writes them to its own (ordinary) output and normalises them there.
// `seq` (device counter + 1, the same on every rank) is the flag value: whatever an earlier call left in a region carries
// another number.  The host alternates regions from call to call; a rank can run at most one call ahead of a peer (it needs
// that peer's next push to go further), so two regions suffice.  Polls are bounded: on time-out the error word is set and the
// kernel runs to its end on whatever it read.
struct LLine { uint32_t d0, f0, d1, f1; };

__device__ __forceinline__ void st_ll(void* p, uint32_t d0, uint32_t d1, uint32_t seq) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(seq), "r"(d1), "r"(seq) : "memory");
}
__device__ __forceinline__ LLine ld_ll(const void* p) {
  LLine v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.d0), "=r"(v.f0), "=r"(v.d1), "=r"(v.f1) : "l"(p) : "memory");
  return v;
}

template <int N>
__device__ __forceinline__ bool poll_lines(const uint8_t* const (&addr)[N], LLine (&out)[N], int n, uint32_t seq,
                                           unsigned long long limit_ns, int* err) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    bool all = true;
#pragma unroll
    for (int k = 0; k < N; ++k)
      if (k < n) {
        out[k] = ld_ll(addr[k]);
        all = all && out[k].f0 == seq && out[k].f1 == seq;
      }
    if (all) return true;
    if ((++spins & 31) == 0) {
      if (t0 == 0) t0 = now_ns();
      else if (now_ns() - t0 > limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); return false; }
    }
  }
}

__device__ __forceinline__ void add_bf16x2(float& a, float& b, uint32_t v) {
  a += __uint_as_float(v << 16);
  b += __uint_as_float(v & 0xffff0000u);
}

__global__ void __launch_bounds__(512)
allreduce_rows_ll_kernel(Peers bufs, const __nv_bfloat16* __restrict__ partial, const __nv_bfloat16* __restrict__ residual,
                         const __nv_bfloat16* __restrict__ norm_w, __nv_bfloat16* __restrict__ sum_out,
                         __nv_bfloat16* __restrict__ norm_out, int rows, int d, float eps, int rank, int world,
                         uint32_t* __restrict__ counters, long long slots_off, long long sums_off,
                         unsigned long long limit_ns, int* __restrict__ err) {
  __shared__ float red[32];
  if (status_poisoned(err)) return;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(counters) + 1;
  const int nvec = d >> 3;                       // 8 bf16 = two lines per vector
  const long long row_bytes = static_cast<long long>(d) * 4;     // a row in line format
  const int R = (rows + world - 1) / world;
  // 1. push the partial's rows to their owners
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int owner = row / R;
    uint8_t* dst = reinterpret_cast<uint8_t*>(bufs.p[owner]) + slots_off + (static_cast<long long>(rank) * R + (row - owner * R)) * row_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(partial + static_cast<long long>(row) * d);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 v = src[i];
      st_ll(dst + i * 32, v.x, v.y, seq);
      st_ll(dst + i * 32 + 16, v.z, v.w, seq);
    }
  }
  // 2. the owner's rows: poll the slots, reduce, push the sums to every rank
  int my_rows = rows - rank * R;
  my_rows = my_rows < 0 ? 0 : (my_rows > R ? R : my_rows);
  const uint8_t* slots = reinterpret_cast<const uint8_t*>(bufs.p[rank]) + slots_off;
  // The owned rows are few (rows / world): their vectors are dealt to ALL CTAs in warp-sized runs, so that the pushes to the
  // peers leave from every SM instead of from `my_rows` of them.
  const int total_vec = my_rows * nvec;
  const int lane = threadIdx.x & 31;
  for (int run = (threadIdx.x >> 5) * gridDim.x + blockIdx.x; run * 32 < total_vec; run += gridDim.x * (blockDim.x >> 5)) {
    const int v = run * 32 + lane;
    if (v < total_vec) {
      const int lr = v / nvec, i = v - lr * nvec;
      const long long row = static_cast<long long>(rank) * R + lr;
      const uint8_t* addr[2 * MAX_RANKS];
      LLine ln[2 * MAX_RANKS];
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        const uint8_t* base = slots + (static_cast<long long>(r < world ? r : 0) * R + lr) * row_bytes + i * 32;
        addr[2 * r] = base;
        addr[2 * r + 1] = base + 16;
      }
      poll_lines<2 * MAX_RANKS>(addr, ln, 2 * world, seq, limit_ns, err);
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < world) {
          add_bf16x2(a[0], a[1], ln[2 * r].d0); add_bf16x2(a[2], a[3], ln[2 * r].d1);
          add_bf16x2(a[4], a[5], ln[2 * r + 1].d0); add_bf16x2(a[6], a[7], ln[2 * r + 1].d1);
        }
      if (residual != nullptr) {
        const uint4 rv = reinterpret_cast<const uint4*>(residual + row * d)[i];
        add_bf16x2(a[0], a[1], rv.x); add_bf16x2(a[2], a[3], rv.y); add_bf16x2(a[4], a[5], rv.z); add_bf16x2(a[6], a[7], rv.w);
      }
      const uint32_t p0 = pack_bf16(a[0], a[1]), p1 = pack_bf16(a[2], a[3]), p2 = pack_bf16(a[4], a[5]), p3 = pack_bf16(a[6], a[7]);
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < world) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(bufs.p[(rank + r) % world]) + sums_off + row * row_bytes + i * 32;
          st_ll(dst, p0, p1, seq);
          st_ll(dst + 16, p2, p3, seq);
        }
    }
  }
  // 3. every rank: poll the sum rows, write them out, normalise
  const uint8_t* sums = reinterpret_cast<const uint8_t*>(bufs.p[rank]) + sums_off;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float acc[2][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int i = threadIdx.x + c * 512;
      if (i < nvec) {
        const uint8_t* addr[2] = {sums + row * row_bytes + i * 32, sums + row * row_bytes + i * 32 + 16};
        LLine ln[2];
        poll_lines<2>(addr, ln, 2, seq, limit_ns, err);
        uint4 pk;
        pk.x = ln[0].d0; pk.y = ln[0].d1; pk.z = ln[1].d0; pk.w = ln[1].d1;
        if (sum_out != nullptr) reinterpret_cast<uint4*>(sum_out + static_cast<long long>(row) * d)[i] = pk;
        acc[c][0] = __uint_as_float(pk.x << 16); acc[c][1] = __uint_as_float(pk.x & 0xffff0000u);
        acc[c][2] = __uint_as_float(pk.y << 16); acc[c][3] = __uint_as_float(pk.y & 0xffff0000u);
        acc[c][4] = __uint_as_float(pk.z << 16); acc[c][5] = __uint_as_float(pk.z & 0xffff0000u);
        acc[c][6] = __uint_as_float(pk.w << 16); acc[c][7] = __uint_as_float(pk.w & 0xffff0000u);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += acc[c][j] * acc[c][j];
      }
    }
    if (norm_out == nullptr) continue;   // (uniform over the block)
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = (threadIdx.x & 31) < 16 ? red[threadIdx.x & 31] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    const float rstd = rsqrtf(t / d + eps);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int i = threadIdx.x + c * 512;
      if (i < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(norm_w)[i];
        const float w[8] = {__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xffff0000u), __uint_as_float(wv.y << 16),
                            __uint_as_float(wv.y & 0xffff0000u), __uint_as_float(wv.z << 16), __uint_as_float(wv.z & 0xffff0000u),
                            __uint_as_float(wv.w << 16), __uint_as_float(wv.w & 0xffff0000u)};
        uint4 pk;
        pk.x = pack_bf16(acc[c][0] * rstd * w[0], acc[c][1] * rstd * w[1]); pk.y = pack_bf16(acc[c][2] * rstd * w[2], acc[c][3] * rstd * w[3]);
        pk.z = pack_bf16(acc[c][4] * rstd * w[4], acc[c][5] * rstd * w[5]); pk.w = pack_bf16(acc[c][6] * rstd * w[6], acc[c][7] * rstd * w[7]);
        reinterpret_cast<uint4*>(norm_out + static_cast<long long>(row) * d)[i] = pk;
      }
    }
  }
  // the last CTA to leave advances the sequence number for the next launch (every CTA read it before it could leave)
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(counters + 1, 1u);
    if (t == gridDim.x - 1) { counters[1] = 0; __threadfence(); *reinterpret_cast<volatile uint32_t*>(counters) = seq; }
  }
}

}  // namespace comm
}  // namespace dewb

// buf_ptrs: the W symmetric staging buffers (two halves of `half_stride` elements each, used alternately);
// `partial` is this rank's local [rows, d] partial sum; `counters`: device uint32[3] = {sequence, arrive, leave},
// zero-initialised once; out tensors are local.
extern "C" int dewb_allreduce_rows(const unsigned long long* buf_ptrs, const unsigned long long* flag_ptrs,
                                   const void* partial, const void* residual, const void* norm_w, void* sum_out,
                                   void* norm_out, int rows, int d, float eps, int rank, int world,
                                   unsigned int* counters, long long half_stride, int slot,
                                   unsigned long long limit_ns, int* err, void* stream) {
  if (d % 8 != 0 || d > 8192 || world < 1 || world > MAX_RANKS) return -3;
  if (rows <= 0) return 0;
  const int blocks = rows < 296 ? rows : 296;      // every CTA must be resident: they wait on one another's staging
  allreduce_rows_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(buf_ptrs, world), make_peers(flag_ptrs, world), reinterpret_cast<const __nv_bfloat16*>(partial),
      reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<const __nv_bfloat16*>(norm_w),
      reinterpret_cast<__nv_bfloat16*>(sum_out), reinterpret_cast<__nv_bfloat16*>(norm_out), rows, d, eps, rank, world,
      counters, counters + 1, half_stride, slot, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}

// Two-shot all-reduce + residual add + RMSNorm with the outputs in peer-visible memory (see the kernel's comment).
// Every rank's buffer holds, at the same element offsets, `slots` ([world][ceil(rows / world)][d]), `sum` ([rows][d]) and
// `norm` ([rows][d]); `counters`: device uint32[3] = {sequence, ticket 1, ticket 2}, zero-initialised once; flag words
// [flag_base, flag_base + 2 * world) of every rank's flag array belong to this call site.
extern "C" int dewb_allreduce_rows_2shot(const unsigned long long* buf_ptrs, const unsigned long long* flag_ptrs,
                                         const void* partial, const void* residual, const void* norm_w, int rows, int d,
                                         float eps, int rank, int world, unsigned int* counters, long long slots_off,
                                         long long sum_off, long long norm_off, int flag_base,
                                         unsigned long long limit_ns, int* err, void* stream) {
  using namespace dewb::comm;
  if (d % 8 != 0 || d > 8192 || world < 1 || world > MAX_RANKS) return -3;
  if ((slots_off | sum_off | norm_off) & 7) return -3;          // 16-byte vectors
  if (rows <= 0) return 0;
  const int blocks = rows < 148 ? rows : 148;                   // one resident CTA per SM at most
  allreduce_rows_2shot_kernel<<<blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(buf_ptrs, world), make_peers(flag_ptrs, world), reinterpret_cast<const __nv_bfloat16*>(partial),
      reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<const __nv_bfloat16*>(norm_w), rows, d, eps, rank,
      world, counters, slots_off, sum_off, norm_off, flag_base, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}

// Low-latency all-reduce + residual add + RMSNorm (see the kernel's comment).  Every rank's byte buffer holds, at the same
// byte offsets, `slots` ([world][ceil(rows / world)][d] in line format, 4 bytes per element) and `sums` ([rows][d], same
// format); `counters`: device uint32[2] = {sequence, leave ticket}, zero-initialised once; the outputs are ordinary local tensors.
extern "C" int dewb_allreduce_rows_ll(const unsigned long long* buf_ptrs, const void* partial, const void* residual,
                                      const void* norm_w, void* sum_out, void* norm_out, int rows, int d, float eps, int rank,
                                      int world, unsigned int* counters, long long slots_off, long long sums_off,
                                      unsigned long long limit_ns, int* err, void* stream) {
  using namespace dewb::comm;
  if (d % 8 != 0 || d > 8192 || world < 1 || world > MAX_RANKS) return -3;
  if ((slots_off | sums_off) & 15) return -3;
  if (rows <= 0) return 0;
  const int blocks = rows < 148 ? rows : 148;                   // every CTA must be resident: they poll what others push
  allreduce_rows_ll_kernel<<<blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(buf_ptrs, world), reinterpret_cast<const __nv_bfloat16*>(partial),
      reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<const __nv_bfloat16*>(norm_w),
      reinterpret_cast<__nv_bfloat16*>(sum_out), reinterpret_cast<__nv_bfloat16*>(norm_out), rows, d, eps, rank, world, counters,
      slots_off, sums_off, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}
