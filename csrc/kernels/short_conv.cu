// Short causal depthwise convolution (kernel size <= 4) with optional SiLU, forward and backward, bf16 [B, T, C].
//   y[b,t,c] = act( sum_j w[c,j] * x[b, t - (K-1) + j, c] + bias[c] )
// One thread owns 8 channels (one 16-byte vector) and walks a run of time steps keeping the last K-1 inputs in
// registers, so every input is read from HBM once. The backward recomputes the pre-activation, walks time in reverse
// for dx, and accumulates dw / dbias per thread before a block-level atomic fold into fp32 outputs.
// Capability parity: src/dew/nn/kernels/short_conv.py (conv :159, forward :138, backward :146).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace dewb {
namespace sconv {

constexpr int TCHUNK = 64;     // time steps per thread-run

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pk(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pk(f[0], f[1]), pk(f[2], f[3]), pk(f[4], f[5]), pk(f[6], f[7]));
}

template <int K>
__global__ void __launch_bounds__(128)
short_conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                      __nv_bfloat16* __restrict__ y, int T, int C, int act) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;       // channel vector
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * TCHUNK;
  if (cv * 8 >= C) return;
  float wr[8][K], br[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(cv * 8 + i) * K + j];
    br[i] = bias != nullptr ? bias[cv * 8 + i] : 0.f;
  }
  const long long base = static_cast<long long>(b) * T * C + cv * 8;
  float hist[K > 1 ? K - 1 : 1][8];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int t = t0 - (K - 1) + j;
    if (t >= 0) unpack8(*reinterpret_cast<const uint4*>(x + base + static_cast<long long>(t) * C), hist[j]);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) hist[j][i] = 0.f;
    }
  }
  const int t1 = min(T, t0 + TCHUNK);
  for (int t = t0; t < t1; ++t) {
    float cur[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(x + base + static_cast<long long>(t) * C), cur);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s = br[i] + wr[i][K - 1] * cur[i];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) s += wr[i][j] * hist[j][i];
      o[i] = act ? s / (1.f + __expf(-s)) : s;
    }
    *reinterpret_cast<uint4*>(y + base + static_cast<long long>(t) * C) = pack8(o);
#pragma unroll
    for (int j = 0; j + 1 < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) hist[j][i] = hist[j + 1][i];
    if (K > 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) hist[K - 2][i] = cur[i];
    }
  }
}

// dx[t] = sum_j w[j] * g[t + (K-1) - j],  g = dy * act'(pre);  dw[j] += sum_t g[t] * x[t - (K-1) + j]; dbias += sum g
template <int K>
__global__ void __launch_bounds__(128)
short_conv_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                      const float* __restrict__ w, const float* __restrict__ bias, __nv_bfloat16* __restrict__ dx,
                      float* __restrict__ dw, float* __restrict__ dbias, int T, int C, int act) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * TCHUNK;
  if (cv * 8 >= C) return;
  float wr[8][K], br[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(cv * 8 + i) * K + j];
    br[i] = bias != nullptr ? bias[cv * 8 + i] : 0.f;
  }
  const long long base = static_cast<long long>(b) * T * C + cv * 8;
  auto load_x = [&](int t, float (&f)[8]) {
    if (t >= 0 && t < T) unpack8(*reinterpret_cast<const uint4*>(x + base + static_cast<long long>(t) * C), f);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
  };
  // g at time t (0 outside [0, T)); needs x[t-K+1 .. t]
  auto grad_at = [&](int t, float (&g)[8]) {
    if (t < 0 || t >= T) {
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = 0.f;
      return;
    }
    float d[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + base + static_cast<long long>(t) * C), d);
    if (!act) {
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = d[i];
      return;
    }
    float pre[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = br[i];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      float xv[8];
      load_x(t - (K - 1) + j, xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) pre[i] += wr[i][j] * xv[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-pre[i]));
      g[i] = d[i] * sg * (1.f + pre[i] * (1.f - sg));
    }
  };
  float dwacc[8][K], dbacc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    dbacc[i] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) dwacc[i][j] = 0.f;
  }
  const int t1 = min(T, t0 + TCHUNK);
  for (int t = t0; t < t1; ++t) {
    float g[8];
    grad_at(t, g);
    // weight / bias gradients from this time step
#pragma unroll
    for (int j = 0; j < K; ++j) {
      float xv[8];
      load_x(t - (K - 1) + j, xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) dwacc[i][j] += g[i] * xv[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) dbacc[i] += g[i];
    // input gradient at this time step gathers g from t .. t + K - 1
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = wr[i][K - 1] * g[i];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      float gn[8];
      grad_at(t + (K - 1) - j, gn);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += wr[i][j] * gn[i];
    }
    *reinterpret_cast<uint4*>(dx + base + static_cast<long long>(t) * C) = pack8(o);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < K; ++j) atomicAdd(dw + (cv * 8 + i) * K + j, dwacc[i][j]);
    if (dbias != nullptr) atomicAdd(dbias + cv * 8 + i, dbacc[i]);
  }
}

}  // namespace sconv
}  // namespace dewb

using namespace dewb::sconv;

// x, y [B, T, C] bf16 (C % 8 == 0); w [C, K] fp32; bias [C] fp32 or null.
extern "C" int dewb_short_conv_fwd(const void* x, const float* w, const float* bias, void* y, int B, int T, int C, int K,
                                   int act, void* stream) {
  if (C % 8 != 0 || K < 2 || K > 4) return -3;
  if (B <= 0 || T <= 0) return 0;
  dim3 grid((C / 8 + 127) / 128, (T + TCHUNK - 1) / TCHUNK, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(y);
  switch (K) {
    case 2: short_conv_fwd_kernel<2><<<grid, 128, 0, s>>>(xp, w, bias, yp, T, C, act); break;
    case 3: short_conv_fwd_kernel<3><<<grid, 128, 0, s>>>(xp, w, bias, yp, T, C, act); break;
    default: short_conv_fwd_kernel<4><<<grid, 128, 0, s>>>(xp, w, bias, yp, T, C, act); break;
  }
  return static_cast<int>(cudaGetLastError());
}

// dw [C, K] and dbias [C] (fp32) must be zeroed by the caller; they are accumulated with atomics.
extern "C" int dewb_short_conv_bwd(const void* x, const void* dy, const float* w, const float* bias, void* dx, float* dw,
                                   float* dbias, int B, int T, int C, int K, int act, void* stream) {
  if (C % 8 != 0 || K < 2 || K > 4) return -3;
  if (B <= 0 || T <= 0) return 0;
  dim3 grid((C / 8 + 127) / 128, (T + TCHUNK - 1) / TCHUNK, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *xp = reinterpret_cast<const __nv_bfloat16*>(x), *dp = reinterpret_cast<const __nv_bfloat16*>(dy);
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(dx);
  switch (K) {
    case 2: short_conv_bwd_kernel<2><<<grid, 128, 0, s>>>(xp, dp, w, bias, op, dw, dbias, T, C, act); break;
    case 3: short_conv_bwd_kernel<3><<<grid, 128, 0, s>>>(xp, dp, w, bias, op, dw, dbias, T, C, act); break;
    default: short_conv_bwd_kernel<4><<<grid, 128, 0, s>>>(xp, dp, w, bias, op, dw, dbias, T, C, act); break;
  }
  return static_cast<int>(cudaGetLastError());
}
