// Token sampling for serving: greedy argmax and temperature / top-k / min-p / top-p sampling, one CTA per row of logits.
//
// No sort: every filter is a threshold on the (temperature-scaled) logit, found by a 4 x 8-bit radix descent over the
// order-preserving integer image of the floats -
//   top-k  : the k-th largest key, by counting histograms;
//   min-p  : logit >= max + log(min_p), closed form;
//   top-p  : the largest key t with  mass(keys > t) < top_p * Z,  by histograms of probability mass (Z and the masses are
//            taken over what top-k and min-p kept, as the reference applies the filters in that order);
// then the draw is the inverse CDF in token order at u * Z' (u in [0, 1) supplied per row by the caller, so the random
// stream stays on the host's keyed generators).  Equal logits at a threshold are all kept.
// Capability: src/dew/sampling/text.py (Sampling: temperature, top_k, top_p, min_p) and the serving draws
// (src/dew/inference/serving.py).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace dewb {
namespace sampling {

constexpr int THREADS = 1024;
constexpr uint32_t FULL = 0xffffffffu;

__device__ __forceinline__ uint32_t ordered(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* row, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int i) { return row[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* row, int i) { return __bfloat162float(row[i]); }

struct Shared {
  float red_f[32];
  int red_i[32];
  float hist_f[256];
  int hist_i[256];
  float bcast_f[4];
  uint32_t bcast_u[4];
};

__device__ float block_max(float v, Shared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
  if ((threadIdx.x & 31) == 0) sh.red_f[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh.red_f[threadIdx.x & 31];
  if ((threadIdx.x & 31) >= (blockDim.x >> 5)) r = -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(FULL, r, o));
  __syncthreads();
  return r;
}
__device__ float block_sum(float v, Shared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  if ((threadIdx.x & 31) == 0) sh.red_f[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh.red_f[threadIdx.x & 31] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(FULL, r, o);
  __syncthreads();
  return r;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
argmax_rows_kernel(const T* __restrict__ logits, long long row_stride, int V, long long* __restrict__ out) {
  __shared__ Shared sh;
  const T* row = logits + blockIdx.x * row_stride;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  // 16-byte loads over the aligned body of the row, four in flight per thread; scalar loads for the rest
  constexpr int PER = 16 / static_cast<int>(sizeof(T));
  int body = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    body = V / PER * PER;
    const uint4* rv = reinterpret_cast<const uint4*>(row);
    const int nvec = body / PER;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * blockDim.x) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vi = v0 + u * blockDim.x;
        raw[u] = vi < nvec ? rv[vi] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vi = v0 + u * blockDim.x;
        if (vi >= nvec) continue;
        const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
        for (int c = 0; c < PER; ++c) {
          const float x = load_logit(e, c);
          const int i = vi * PER + c;
          if (x > best || (x == best && i < idx)) { best = x; idx = i; }
        }
      }
    }
  }
  for (int i = body + threadIdx.x; i < V; i += blockDim.x) {
    const float x = load_logit(row, i);
    if (x > best || (x == best && i < idx)) { best = x; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(FULL, best, o);
    const int oi = __shfl_xor_sync(FULL, idx, o);
    if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sh.red_f[threadIdx.x >> 5] = best; sh.red_i[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? sh.red_f[threadIdx.x] : -INFINITY;
    idx = threadIdx.x < (blockDim.x >> 5) ? sh.red_i[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(FULL, best, o);
      const int oi = __shfl_xor_sync(FULL, idx, o);
      if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
sample_rows_kernel(const T* __restrict__ logits, long long row_stride, int V, const float* __restrict__ uniform,
                   float inv_temperature, int top_k, float top_p, float min_p, long long* __restrict__ out,
                   int* __restrict__ kept_out) {
  __shared__ Shared sh;
  const T* row = logits + blockIdx.x * row_stride;
  const int tid = threadIdx.x;
  // row maximum of the scaled logits
  float mx = -INFINITY;
  for (int i = tid; i < V; i += THREADS) mx = fmaxf(mx, load_logit(row, i) * inv_temperature);
  mx = block_max(mx, sh);
  uint32_t thr = 0;                         // keep keys >= thr
  if (min_p > 0.f) thr = ordered(mx + __logf(min_p));
  if (top_k > 0 && top_k < V) {
    uint32_t prefix = 0;
    int remaining = top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) sh.hist_i[tid] = 0;
      __syncthreads();
      const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < V; i += THREADS) {
        const uint32_t key = ordered(load_logit(row, i) * inv_temperature);
        if ((key & mask) == prefix) atomicAdd(&sh.hist_i[(key >> shift) & 255], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, b = 255;
        for (; b > 0; --b) { if (cum + sh.hist_i[b] >= remaining) break; cum += sh.hist_i[b]; }
        sh.bcast_u[0] = static_cast<uint32_t>(b);
        sh.bcast_u[1] = static_cast<uint32_t>(remaining - cum);
      }
      __syncthreads();
      prefix |= sh.bcast_u[0] << shift;
      remaining = static_cast<int>(sh.bcast_u[1]);
      __syncthreads();
    }
    thr = max(thr, prefix);
  }
  // mass of what top-k and min-p keep
  float z = 0.f;
  for (int i = tid; i < V; i += THREADS) {
    const float x = load_logit(row, i) * inv_temperature;
    if (ordered(x) >= thr) z += __expf(x - mx);
  }
  z = block_sum(z, sh);
  if (top_p < 1.f) {
    const float target = top_p * z;
    uint32_t prefix = 0;
    float above = 0.f;                      // mass of keys greater than every key that matches the prefix so far
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) sh.hist_f[tid] = 0.f;
      __syncthreads();
      const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < V; i += THREADS) {
        const float x = load_logit(row, i) * inv_temperature;
        const uint32_t key = ordered(x);
        if (key >= thr && (key & mask) == prefix) atomicAdd(&sh.hist_f[(key >> shift) & 255], __expf(x - mx));
      }
      __syncthreads();
      if (tid == 0) {
        float cum = above;
        int b = 255;
        for (; b > 0; --b) { if (cum + sh.hist_f[b] >= target) break; cum += sh.hist_f[b]; }
        sh.bcast_u[0] = static_cast<uint32_t>(b);
        sh.bcast_f[0] = cum;
      }
      __syncthreads();
      prefix |= sh.bcast_u[0] << shift;
      above = sh.bcast_f[0];
      __syncthreads();
    }
    thr = max(thr, prefix);
  }
  // inverse CDF in token order over the kept set: every thread owns a contiguous span of tokens
  const int span = (V + THREADS - 1) / THREADS;
  const int lo = min(tid * span, V), hi = min(lo + span, V);
  float part = 0.f;
  int kept = 0;
  for (int i = lo; i < hi; ++i) {
    const float x = load_logit(row, i) * inv_temperature;
    if (ordered(x) >= thr) { part += __expf(x - mx); ++kept; }
  }
  // exclusive prefix of the per-thread masses (warp scan, then the warp totals)
  float incl = part;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(FULL, incl, o);
    if ((tid & 31) >= o) incl += up;
  }
  if ((tid & 31) == 31) sh.red_f[tid >> 5] = incl;
  int kept_w = kept;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) kept_w += __shfl_xor_sync(FULL, kept_w, o);
  if ((tid & 31) == 0) sh.red_i[tid >> 5] = kept_w;
  __syncthreads();
  float warp_off = 0.f, total = 0.f;
  for (int w = 0; w < THREADS / 32; ++w) { if (w < (tid >> 5)) warp_off += sh.red_f[w]; total += sh.red_f[w]; }
  const float excl = warp_off + incl - part;
  const float target = fminf(uniform[blockIdx.x], 0.99999994f) * total;
  if (tid == 0) {
    sh.bcast_u[2] = 0xffffffffu;
    int kt = 0;
    for (int w = 0; w < THREADS / 32; ++w) kt += sh.red_i[w];
    if (kept_out != nullptr) kept_out[blockIdx.x] = kt;
  }
  __syncthreads();
  if (part > 0.f && target >= excl && target < excl + part) {
    float run = excl;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      const float x = load_logit(row, i) * inv_temperature;
      if (ordered(x) >= thr) {
        pick = i;                                   // the last kept token of the span if rounding leaves the target beyond it
        run += __expf(x - mx);
        if (target < run) break;
      }
    }
    atomicMin(&sh.bcast_u[2], static_cast<uint32_t>(pick));
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t pick = sh.bcast_u[2];
    if (pick == 0xffffffffu) {
      // rounding put the target past the last span's end: take the last kept token
      pick = 0;
      for (int i = V - 1; i >= 0; --i) {
        if (ordered(load_logit(row, i) * inv_temperature) >= thr) { pick = static_cast<uint32_t>(i); break; }
      }
    }
    out[blockIdx.x] = static_cast<long long>(pick);
  }
}

}  // namespace sampling
}  // namespace dewb

// logits [rows, V] (fp32: dtype 0, bf16: dtype 1) with `row_stride` elements between rows -> out [rows] int64.
extern "C" int dewb_argmax_rows(const void* logits, int dtype, long long rows, long long row_stride, int V, long long* out,
                                void* stream) {
  using namespace dewb::sampling;
  if (V <= 0) return -3;
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0) argmax_rows_kernel<float><<<static_cast<unsigned>(rows), THREADS, 0, s>>>(reinterpret_cast<const float*>(logits), row_stride, V, out);
  else argmax_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), THREADS, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), row_stride, V, out);
  return static_cast<int>(cudaGetLastError());
}

// One draw per row: temperature > 0; top_k <= 0 or >= V: off; top_p >= 1: off; min_p <= 0: off.  uniform [rows] fp32 in
// [0, 1).  kept [rows] int32 (may be null) receives the size of each row's filtered set.
extern "C" int dewb_sample_rows(const void* logits, int dtype, long long rows, long long row_stride, int V,
                                const float* uniform, float temperature, int top_k, float top_p, float min_p,
                                long long* out, int* kept, void* stream) {
  using namespace dewb::sampling;
  if (V <= 0 || !(temperature > 0.f)) return -3;
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float inv_t = 1.f / temperature;
  if (dtype == 0)
    sample_rows_kernel<float><<<static_cast<unsigned>(rows), THREADS, 0, s>>>(reinterpret_cast<const float*>(logits), row_stride, V, uniform,
                                                                              inv_t, top_k, top_p, min_p, out, kept);
  else
    sample_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), THREADS, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), row_stride,
                                                                                      V, uniform, inv_t, top_k, top_p, min_p, out, kept);
  return static_cast<int>(cudaGetLastError());
}
