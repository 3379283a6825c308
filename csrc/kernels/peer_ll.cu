// Point-to-point and small all-to-all exchanges over NVLink peer memory with the arrival flag inside the data: every
// 16-byte store carries {4 bytes, tag, 4 bytes, tag}, so the receiver polls the bytes it needs and no fence, flag store or
// second kernel stands between "sent" and "received".  Two operations:
//
//   peer_exchange   this rank pushes `n` 16-byte vectors to rank `to` (or to nobody) and collects `n` vectors from rank `from`
//                   (or from nobody): the halo of a sequence-parallel convolution or banded attention, the hand-over of a
//                   recurrent state along the sequence axis, and their backward passes (the same call with the ranks swapped)
//   allreduce_small every rank pushes a short fp32 vector to every peer and reduces the `world` copies (sum or max): the row
//                   statistics of a vocabulary-parallel cross-entropy or of a norm over a feature axis split over ranks
//
// Every rank's receive buffer has one area per (region, sender).  Messages of a directed pair (sender -> receiver) are numbered
// by both ends (the k-th send meets the k-th receive); the number is the tag and selects the region.  A sender may not reuse an
// area before its receiver has read what the area held: the receiver's last CTA writes the tag it finished into the SENDER's
// acknowledgement word, and a sender that passes `need_ack` > 0 waits (bounded) for that word first.  (The reductions number
// their calls the same way: every rank takes part in every call.)  All polls are bounded: on time-out the error word is set and the kernel
// runs to its end on whatever it read.
//
// Replaces, over peer memory, the `ppermute` halos and state hand-offs of src/dew/nn/linear.py:696-781,
// src/dew/nn/local_attention.py:307, src/dew/nn/kernels/recurrence_algebra.py:367-370 and the `pmax` / `psum` of row statistics
// of src/dew/objectives/lm/chunked.py:1143-1228, src/dew/nn/norms.py:429.
#include <cstdint>
#include <cuda_runtime.h>

namespace dewb {
namespace peerll {

constexpr int MAX_RANKS = 8;
enum : int { ERR_WAIT_PEER = 5 };

struct Peers {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_line(void* p, uint32_t d0, uint32_t d1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(tag), "r"(d1), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Poll two lines (one 16-byte vector of payload) until both carry `tag`; false on time-out.
__device__ __forceinline__ bool poll_vector(const uint8_t* p, uint32_t tag, unsigned long long limit_ns, int* err, uint4& out) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    const uint4 a = ld_line(p), b = ld_line(p + 16);
    if (a.y == tag && a.w == tag && b.y == tag && b.w == tag) {
      out = make_uint4(a.x, a.z, b.x, b.z);
      return true;
    }
    if ((++spins & 31) == 0) {
      if (t0 == 0) t0 = now_ns();
      else if (now_ns() - t0 > limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); out = make_uint4(0, 0, 0, 0); return false; }
    }
  }
}

// One thread waits until acks[index] has reached `need` (signed distance, tags only grow); the block waits for it.
__device__ bool wait_ack(const uint32_t* word, uint32_t need, unsigned long long limit_ns, int* err) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint64_t t0 = now_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(word) - need) < 0) {
      if ((++spins & 63) == 0) {
        if (now_ns() - t0 > limit_ns) { ok = 0; atomicCAS(err, 0, ERR_WAIT_PEER); break; }
        __nanosleep(100);
      }
    }
  }
  __syncthreads();
  return ok != 0;
}

__device__ bool poisoned(const int* err) {
  __shared__ int bad;
  if (threadIdx.x == 0) bad = *reinterpret_cast<const volatile int*>(err);
  __syncthreads();
  return bad != 0;
}

// bufs: every rank's receive buffer (bytes); acks: every rank's acknowledgement words, acks[r][j] = the last tag rank j has read of
// what rank r sent it.  `send_off` / `recv_off`: byte offsets of the (region, sender) areas: the area of sender `rank` inside rank
// `to`'s buffer, and the area of sender `from` inside this rank's buffer.
__global__ void __launch_bounds__(256)
peer_exchange_kernel(Peers bufs, Peers acks, const uint4* __restrict__ src, uint4* __restrict__ dst, long long n, int rank, int to,
                     int from, uint32_t send_tag, uint32_t recv_tag, uint32_t need_ack, long long send_off, long long recv_off,
                     unsigned int* __restrict__ leave_counter, unsigned long long limit_ns, int* __restrict__ err) {
  if (poisoned(err)) return;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (to >= 0) {
    if (need_ack != 0 && !wait_ack(reinterpret_cast<const uint32_t*>(acks.p[rank]) + to, need_ack, limit_ns, err)) return;
    uint8_t* out = reinterpret_cast<uint8_t*>(bufs.p[to]) + send_off;
    for (long long v = first; v < n; v += stride) {
      const uint4 x = src[v];
      st_line(out + v * 32, x.x, x.y, send_tag);
      st_line(out + v * 32 + 16, x.z, x.w, send_tag);
    }
  }
  if (from >= 0) {
    const uint8_t* in = reinterpret_cast<const uint8_t*>(bufs.p[rank]) + recv_off;
    for (long long v = first; v < n; v += stride) {
      uint4 x;
      poll_vector(in + v * 32, recv_tag, limit_ns, err, x);
      dst[v] = x;
    }
    // the last block to finish reading tells the sender that the area is free again
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int t = atomicAdd(leave_counter, 1u);
      if (t == gridDim.x - 1) {
        *leave_counter = 0;
        st_release_sys(reinterpret_cast<uint32_t*>(acks.p[from]) + rank, recv_tag);
      }
    }
  }
}

// in / out: fp32 [n]; op 0 = sum, 1 = max.  Areas: [region][sender][n floats in line format = 8 bytes per float].
__global__ void __launch_bounds__(256)
allreduce_small_kernel(Peers bufs, Peers acks, const float* __restrict__ in, float* __restrict__ out, long long n, int rank, int world,
                       uint32_t tag, uint32_t need_ack, long long region_off, long long area_bytes, int op,
                       unsigned int* __restrict__ leave_counter, unsigned long long limit_ns, int* __restrict__ err) {
  if (poisoned(err)) return;
  __shared__ int ok_all;
  if (need_ack != 0) {
    // every peer must have read what this rank last wrote into the region
    if (threadIdx.x == 0) ok_all = 1;
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank) {
      const uint32_t* word = reinterpret_cast<const uint32_t*>(acks.p[rank]) + threadIdx.x;
      const uint64_t t0 = now_ns();
      uint32_t spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(word) - need_ack) < 0) {
        if ((++spins & 63) == 0) {
          if (now_ns() - t0 > limit_ns) { ok_all = 0; atomicCAS(err, 0, ERR_WAIT_PEER); break; }
          __nanosleep(100);
        }
      }
    }
    __syncthreads();
    if (!ok_all) return;
  }
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long pairs = (n + 1) / 2;                        // one line carries two floats
  for (long long v = first; v < pairs; v += stride) {
    const uint32_t a = __float_as_uint(in[2 * v]);
    const uint32_t b = 2 * v + 1 < n ? __float_as_uint(in[2 * v + 1]) : 0u;
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < world) {
        const int peer = (rank + r) % world;
        st_line(reinterpret_cast<uint8_t*>(bufs.p[peer]) + region_off + rank * area_bytes + v * 16, a, b, tag);
      }
  }
  const uint8_t* mine = reinterpret_cast<const uint8_t*>(bufs.p[rank]) + region_off;
  for (long long v = first; v < pairs; v += stride) {
    float s0 = op == 0 ? 0.f : -INFINITY, s1 = s0;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    uint4 ln[MAX_RANKS];
    while (true) {
      bool all = true;
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < world) {
          ln[r] = ld_line(mine + r * area_bytes + v * 16);
          all = all && ln[r].y == tag && ln[r].w == tag;
        }
      if (all) break;
      if ((++spins & 31) == 0) {
        if (t0 == 0) t0 = now_ns();
        else if (now_ns() - t0 > limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); break; }
      }
    }
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < world) {
        const float x0 = __uint_as_float(ln[r].x), x1 = __uint_as_float(ln[r].z);
        if (op == 0) { s0 += x0; s1 += x1; } else { s0 = fmaxf(s0, x0); s1 = fmaxf(s1, x1); }
      }
    out[2 * v] = s0;
    if (2 * v + 1 < n) out[2 * v + 1] = s1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(leave_counter, 1u);
    if (t == gridDim.x - 1) {
      *leave_counter = 0;
      for (int r = 0; r < world; ++r)
        if (r != rank) st_release_sys(reinterpret_cast<uint32_t*>(acks.p[r]) + rank, tag);
    }
  }
}

static Peers make_peers(const unsigned long long* ptrs, int world) {
  Peers p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

}  // namespace peerll
}  // namespace dewb

// src / dst: `n_bytes` (a multiple of 16) each; `to` / `from`: ranks or -1; the areas at `send_off` (in rank `to`'s buffer) and
// `recv_off` (in this rank's buffer) hold 2 * n_bytes each.  `leave_counter`: one zeroed device word per link.
extern "C" int dewb_peer_exchange(const unsigned long long* buf_ptrs, const unsigned long long* ack_ptrs, const void* src, void* dst,
                                  long long n_bytes, int rank, int world, int to, int from, unsigned int send_tag, unsigned int recv_tag,
                                  unsigned int need_ack,
                                  long long send_off, long long recv_off, unsigned int* leave_counter,
                                  unsigned long long limit_ns, int* err, void* stream) {
  using namespace dewb::peerll;
  if (n_bytes < 0 || (n_bytes & 15) || world < 1 || world > MAX_RANKS || to >= world || from >= world || ((send_off | recv_off) & 15))
    return -3;
  if (n_bytes == 0 || (to < 0 && from < 0)) return 0;
  const long long n = n_bytes / 16;
  long long blocks = (n + 255) / 256;
  if (blocks > 296) blocks = 296;                       // receivers poll what senders push: every CTA must be resident
  peer_exchange_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(buf_ptrs, world), make_peers(ack_ptrs, world), reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), n,
      rank, to, from, send_tag, recv_tag, need_ack, send_off, recv_off, leave_counter, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dewb_allreduce_small(const unsigned long long* buf_ptrs, const unsigned long long* ack_ptrs, const float* in, float* out,
                                    long long n, int rank, int world, unsigned int tag, unsigned int need_ack, long long region_off,
                                    long long area_bytes, int op, unsigned int* leave_counter, unsigned long long limit_ns,
                                    int* err, void* stream) {
  using namespace dewb::peerll;
  if (n < 0 || world < 1 || world > MAX_RANKS || (region_off & 15) || (area_bytes & 15) || area_bytes < (n + 1) / 2 * 16 || op < 0 || op > 1)
    return -3;
  if (n == 0) return 0;
  const long long pairs = (n + 1) / 2;
  long long blocks = (pairs + 255) / 256;
  if (blocks > 296) blocks = 296;
  allreduce_small_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_peers(buf_ptrs, world), make_peers(ack_ptrs, world), in, out, n, rank, world, tag, need_ack, region_off, area_bytes, op,
      leave_counter, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}
