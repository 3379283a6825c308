// Bandwidth-bound row kernels for sm_100a: RMSNorm family, SwiGLU, RoPE, cross-entropy rows, AdamW, casts.
// Each is a single pass over its operands with 16-byte vector accesses and fp32 math; the roofline for all of
// them is HBM bandwidth, so the only design rule is "touch every byte once".
//
// Capability parity: src/dew/nn/kernels/norm_swiglu.py (rms_norm :1242, stream_rms_norm :1204, gated_rms_norm
// :1266, swiglu :1456, packed_swiglu :1467), src/dew/nn/rope.py, src/dew/optim.py (_adamw :1114),
// src/dew/averaging.py:116-139 (ema_update).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

namespace dewb {
namespace ew {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = lo(v.x); f[1] = hi(v.x); f[2] = lo(v.y); f[3] = hi(v.y);
  f[4] = lo(v.z); f[5] = hi(v.z); f[6] = lo(v.w); f[7] = hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack(f[0], f[1]); v.y = pack(f[2], f[3]); v.z = pack(f[4], f[5]); v.w = pack(f[6], f[7]);
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; `red` is shared scratch of >= 32 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_CACHE = 4;   // uint4 vectors cached per thread: rows up to 256*4*8 = 8192 wide stay in registers

// ---------------------------------------------------------------------------------------------------------
// RMSNorm forward. MODE 0: y = norm(x) * w.  MODE 1 (stream): h = x + branch, writes h and y = norm(h) * w.
// MODE 2 (gated): y = norm(x) * w * silu(z).   d must be a multiple of 8; one block per row.
template <int MODE>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ other, const bf16* __restrict__ w,
                   bf16* __restrict__ y, bf16* __restrict__ h_out, float* __restrict__ rstd_out, int d, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  const uint4* orow = MODE != 0 ? reinterpret_cast<const uint4*>(other + row * d) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 cache[NORM_CACHE];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_CACHE; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (i < nvec) {
      uint4 v = xr[i];
      float f[8]; unpack8(v, f);
      if (MODE == 1) {
        float g[8]; unpack8(orow[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        v = pack8(f);
        unpack8(v, f);  // the stream is stored in bf16, so normalise what is stored
        reinterpret_cast<uint4*>(h_out + row * d)[i] = v;
      }
      cache[c] = v;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  for (int i = threadIdx.x + NORM_CACHE * NORM_THREADS; i < nvec; i += NORM_THREADS) {
    uint4 v = xr[i];
    float f[8]; unpack8(v, f);
    if (MODE == 1) {
      float g[8]; unpack8(orow[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      v = pack8(f); unpack8(v, f);
      reinterpret_cast<uint4*>(h_out + row * d)[i] = v;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  uint4* yr = reinterpret_cast<uint4*>(y + row * d);
  const uint4* src = MODE == 1 ? reinterpret_cast<const uint4*>(h_out + row * d) : xr;
#pragma unroll
  for (int c = 0; c < NORM_CACHE; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (i < nvec) {
      float f[8], g[8]; unpack8(cache[c], f); unpack8(wr[i], g);
      if (MODE == 2) {
        float z[8]; unpack8(orow[i], z);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j] * (z[j] / (1.f + __expf(-z[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
      }
      yr[i] = pack8(f);
    }
  }
  for (int i = threadIdx.x + NORM_CACHE * NORM_THREADS; i < nvec; i += NORM_THREADS) {
    float f[8], g[8]; unpack8(src[i], f); unpack8(wr[i], g);
    if (MODE == 2) {
      float z[8]; unpack8(orow[i], z);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j] * (z[j] / (1.f + __expf(-z[j])));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
    }
    yr[i] = pack8(f);
  }
}

// ---------------------------------------------------------------------------------------------------------
// RMSNorm backward. A persistent grid walks rows; each block keeps its share of dw in registers and writes one
// partial row of `dw_partial[gridDim.x, d]` (fp32 scratch) that `colsum_kernel` then folds into dw.
//   dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w (* silu(z) when gated),  xhat = x * rstd
//   dres (optional): gradient arriving on the residual stream, added into dx (stream norm).
//   gated: also writes dz = dy * w * xhat * silu'(z).
// d <= NORM_THREADS * 8 * BWD_COLS.
constexpr int BWD_COLS = 4;
template <bool GATED>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                   const float* __restrict__ rstd, const bf16* __restrict__ dres, const bf16* __restrict__ z,
                   bf16* __restrict__ dx, bf16* __restrict__ dz, float* __restrict__ dw_partial, long long rows, int d) {
  __shared__ float red[32];
  const int nvec = d >> 3;
  float dwacc[BWD_COLS][8];
#pragma unroll
  for (int c = 0; c < BWD_COLS; ++c)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[c][j] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * d);
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
    const float rs = rstd[row];
    float gx[BWD_COLS][8], xh[BWD_COLS][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < BWD_COLS; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        float a[8], b[8], ww[8];
        unpack8(dyr[i], a); unpack8(xr[i], b); unpack8(wr[i], ww);
        float zz[8];
        if (GATED) unpack8(reinterpret_cast<const uint4*>(z + row * d)[i], zz);
        float dzv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = b[j] * rs;
          float dyj = a[j];
          if (GATED) {
            const float sg = 1.f / (1.f + __expf(-zz[j]));
            const float silu = zz[j] * sg;
            dzv[j] = dyj * ww[j] * xhat * (sg * (1.f + zz[j] * (1.f - sg)));
            dyj *= silu;
          }
          xh[c][j] = xhat;
          gx[c][j] = dyj * ww[j];
          dwacc[c][j] += dyj * xhat;
          dot += gx[c][j] * xhat;
        }
        if (GATED) reinterpret_cast<uint4*>(dz + row * d)[i] = pack8(dzv);
      }
    }
    dot = block_sum(dot, red) / d;
#pragma unroll
    for (int c = 0; c < BWD_COLS; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (gx[c][j] - xh[c][j] * dot);
        if (dres != nullptr) {
          float r[8]; unpack8(reinterpret_cast<const uint4*>(dres + row * d)[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        reinterpret_cast<uint4*>(dx + row * d)[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < BWD_COLS; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (i < nvec) {
      float4* out = reinterpret_cast<float4*>(dw_partial + static_cast<long long>(blockIdx.x) * d + i * 8);
      out[0] = make_float4(dwacc[c][0], dwacc[c][1], dwacc[c][2], dwacc[c][3]);
      out[1] = make_float4(dwacc[c][4], dwacc[c][5], dwacc[c][6], dwacc[c][7]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Row-group kernels for d <= 4096: a row is owned by G lanes of one warp (G a power of two <= 32), each lane keeps
// its VPL 16-byte vectors of the row in registers, reductions are shuffles only (no shared memory, no block barrier),
// and a block of 8 warps covers 8 * 32 / G rows. These are the fast paths; the block-per-row kernels above remain for
// wider rows.
template <int G_>
__device__ __forceinline__ float group_sum(float v, int G) {
  for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int MODE, int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ other, const bf16* __restrict__ w,
                        bf16* __restrict__ y, bf16* __restrict__ h_out, float* __restrict__ rstd_out, long long rows,
                        int d, float eps, int G) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gpw = 32 / G;
  const long long row = (static_cast<long long>(blockIdx.x) * 8 + warp) * gpw + lane / G;
  const int gl = lane % G;
  const bool live = row < rows;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  const uint4* orow = reinterpret_cast<const uint4*>(other + row * d);
  uint4 cache[VPL];
  uint4 oth[MODE == 2 ? VPL : 1];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < VPL; ++c) {
    const int i = gl + c * G;
    if (live && i < nvec) {
      cache[c] = xr[i];
      if (MODE != 0) oth[MODE == 2 ? c : 0] = orow[i];
      if (MODE == 1) {
        float f[8], g[8]; unpack8(cache[c], f); unpack8(oth[0], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        cache[c] = pack8(f);
        reinterpret_cast<uint4*>(h_out + row * d)[i] = cache[c];
      }
      float f[8]; unpack8(cache[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  ss = group_sum<0>(ss, G);
  const float rstd = rsqrtf(ss / d + eps);
  if (live && gl == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int c = 0; c < VPL; ++c) {
    const int i = gl + c * G;
    if (live && i < nvec) {
      float f[8], g[8]; unpack8(cache[c], f); unpack8(wr[i], g);
      if (MODE == 2) {
        float z[8]; unpack8(oth[c], z);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j] * (z[j] / (1.f + __expf(-z[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
      }
      reinterpret_cast<uint4*>(y + row * d)[i] = pack8(f);
    }
  }
}

// Wide rows (1024 <= d <= 8192): one 128-thread block per row, VPT 16-byte vectors per thread, every load of the row
// issued before the first use. Low register count keeps 12+ blocks resident per SM, which is what hides DRAM latency.
__device__ __forceinline__ float block128_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) red[warp] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

template <int MODE, int VPT>
__global__ void __launch_bounds__(128)
rmsnorm_fwd_block_kernel(const bf16* __restrict__ x, const bf16* __restrict__ other, const bf16* __restrict__ w,
                         bf16* __restrict__ y, bf16* __restrict__ h_out, float* __restrict__ rstd_out, int d, float eps) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  const uint4* orow = reinterpret_cast<const uint4*>(other + row * d);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 cache[VPT], oth[MODE != 0 ? VPT : 1], wv[VPT];
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int i = threadIdx.x + c * 128;
    if (i < nvec) {
      cache[c] = xr[i];
      if (MODE != 0) oth[c] = orow[i];
      wv[c] = wr[i];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int i = threadIdx.x + c * 128;
    if (i < nvec) {
      float f[8]; unpack8(cache[c], f);
      if (MODE == 1) {
        float g[8]; unpack8(oth[c], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        cache[c] = pack8(f);
        reinterpret_cast<uint4*>(h_out + row * d)[i] = cache[c];
        unpack8(cache[c], f);            // the statistics see the rounded sum, as every later reader does
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  ss = block128_sum(ss, red);
  const float rstd = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int i = threadIdx.x + c * 128;
    if (i < nvec) {
      float f[8], g[8]; unpack8(cache[c], f); unpack8(wv[c], g);
      if (MODE == 2) {
        float z[8]; unpack8(oth[c], z);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j] * (z[j] / (1.f + __expf(-z[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
      }
      reinterpret_cast<uint4*>(y + row * d)[i] = pack8(f);
    }
  }
}

template <bool GATED, int VPT>
__global__ void __launch_bounds__(128)
rmsnorm_bwd_dx_block_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                            const float* __restrict__ rstd, const bf16* __restrict__ dres, const bf16* __restrict__ z,
                            bf16* __restrict__ dx, bf16* __restrict__ dz, int d) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const float rs = rstd[row];
  uint4 gv[VPT], xv[VPT], wv[VPT], rv[VPT], zv[GATED ? VPT : 1];
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int i = threadIdx.x + c * 128;
    if (i < nvec) {
      gv[c] = reinterpret_cast<const uint4*>(dy + row * d)[i];
      xv[c] = reinterpret_cast<const uint4*>(x + row * d)[i];
      wv[c] = wr[i];
      if (dres != nullptr) rv[c] = reinterpret_cast<const uint4*>(dres + row * d)[i];
      if (GATED) zv[c] = reinterpret_cast<const uint4*>(z + row * d)[i];
    }
  }
  float dot = 0.f;
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int i = threadIdx.x + c * 128;
    if (i < nvec) {
      float a[8], b[8], ww[8]; unpack8(gv[c], a); unpack8(xv[c], b); unpack8(wv[c], ww);
      if (GATED) {
        float zz[8], dzv[8]; unpack8(zv[c], zz);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sg = 1.f / (1.f + __expf(-zz[j]));
          dzv[j] = a[j] * ww[j] * (b[j] * rs) * (sg * (1.f + zz[j] * (1.f - sg)));
          a[j] *= zz[j] * sg;
        }
        reinterpret_cast<uint4*>(dz + row * d)[i] = pack8(dzv);
        gv[c] = pack8(a);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * ww[j] * (b[j] * rs);
    }
  }
  dot = block128_sum(dot, red) / d;
#pragma unroll
  for (int c = 0; c < VPT; ++c) {
    const int i = threadIdx.x + c * 128;
    if (i < nvec) {
      float a[8], b[8], ww[8], o[8]; unpack8(gv[c], a); unpack8(xv[c], b); unpack8(wv[c], ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (a[j] * ww[j] - (b[j] * rs) * dot);
      if (dres != nullptr) {
        float r[8]; unpack8(rv[c], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      reinterpret_cast<uint4*>(dx + row * d)[i] = pack8(o);
    }
  }
}

// dx (and dz when gated) for one row per lane group; dw is a separate column reduction (rmsnorm_dw_kernel).
template <bool GATED, int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dx_rows_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                           const float* __restrict__ rstd, const bf16* __restrict__ dres, const bf16* __restrict__ z,
                           bf16* __restrict__ dx, bf16* __restrict__ dz, long long rows, int d, int G) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gpw = 32 / G;
  const long long row = (static_cast<long long>(blockIdx.x) * 8 + warp) * gpw + lane / G;
  const int gl = lane % G;
  const bool live = row < rows;
  const int nvec = d >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const float rs = live ? rstd[row] : 0.f;
  uint4 gxp[VPL], xhp[VPL];     // g = dy * w (* silu z) and xhat, kept packed in bf16 pairs? no: fp32 needs 2x; keep inputs
  float dot = 0.f;
#pragma unroll
  for (int c = 0; c < VPL; ++c) {
    const int i = gl + c * G;
    if (live && i < nvec) {
      gxp[c] = reinterpret_cast<const uint4*>(dy + row * d)[i];
      xhp[c] = reinterpret_cast<const uint4*>(x + row * d)[i];
      float a[8], b[8], ww[8]; unpack8(gxp[c], a); unpack8(xhp[c], b); unpack8(wr[i], ww);
      if (GATED) {
        float zz[8], dzv[8]; unpack8(reinterpret_cast<const uint4*>(z + row * d)[i], zz);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sg = 1.f / (1.f + __expf(-zz[j]));
          dzv[j] = a[j] * ww[j] * (b[j] * rs) * (sg * (1.f + zz[j] * (1.f - sg)));
          a[j] *= zz[j] * sg;
        }
        reinterpret_cast<uint4*>(dz + row * d)[i] = pack8(dzv);
        gxp[c] = pack8(a);   // dy * silu(z), rounded to bf16 like every other stored intermediate
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * ww[j] * (b[j] * rs);
    }
  }
  dot = group_sum<0>(dot, G) / d;
#pragma unroll
  for (int c = 0; c < VPL; ++c) {
    const int i = gl + c * G;
    if (live && i < nvec) {
      float a[8], b[8], ww[8], o[8]; unpack8(gxp[c], a); unpack8(xhp[c], b); unpack8(wr[i], ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (a[j] * ww[j] - (b[j] * rs) * dot);
      if (dres != nullptr) {
        float r[8]; unpack8(reinterpret_cast<const uint4*>(dres + row * d)[i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      reinterpret_cast<uint4*>(dx + row * d)[i] = pack8(o);
    }
  }
}

// dw partials: block (32, 8); thread (tx, ty) owns vector column blockIdx.x * 32 + tx and walks rows
// blockIdx.y * 8 + ty, + gridDim.y * 8, ...; the 8 row-threads fold through shared memory into
// partial[blockIdx.y, d].
template <bool GATED>
__global__ void __launch_bounds__(256)
rmsnorm_dw_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ rstd,
                  const bf16* __restrict__ z, float* __restrict__ partial, long long rows, int d) {
  __shared__ float red[8][32][9];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int vec = blockIdx.x * 32 + tx;
  const int nvec = d >> 3;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (vec < nvec) {
    for (long long r = static_cast<long long>(blockIdx.y) * 8 + ty; r < rows; r += static_cast<long long>(gridDim.y) * 8) {
      float a[8], b[8];
      unpack8(reinterpret_cast<const uint4*>(dy + r * d)[vec], a);
      unpack8(reinterpret_cast<const uint4*>(x + r * d)[vec], b);
      const float rs = rstd[r];
      if (GATED) {
        float zz[8]; unpack8(reinterpret_cast<const uint4*>(z + r * d)[vec], zz);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] *= zz[j] / (1.f + __expf(-zz[j]));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += a[j] * b[j] * rs;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[ty][tx][j] = acc[j];
  __syncthreads();
  if (ty == 0 && vec < nvec) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += red[k][tx][j];
      acc[j] = s;
    }
    float4* out = reinterpret_cast<float4*>(partial + static_cast<long long>(blockIdx.y) * d + vec * 8);
    out[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    out[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// out[col] (+)= sum_r partial[r, col]; one thread per column, coalesced over columns
__global__ void colsum_kernel(const float* __restrict__ partial, int nrows, int d, float* __restrict__ out_f32,
                              bf16* __restrict__ out_bf16, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= d) return;
  float s = 0.f;
  for (int r = 0; r < nrows; ++r) s += partial[static_cast<long long>(r) * d + col];
  if (out_f32 != nullptr) out_f32[col] = accumulate ? out_f32[col] + s : s;
  if (out_bf16 != nullptr) out_bf16[col] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[col]) + s : s);
}

// ---------------------------------------------------------------------------------------------------------
// SwiGLU on a packed [rows, 2F] tensor (gate = columns [0,F), up = columns [F,2F)) or on two tensors.
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up, bf16* __restrict__ out,
                                  long long rows, int F, long long in_stride) {
  const long long nvec = rows * (F >> 3);
  const int fv = F >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += 4 * stride) {
    uint4 gv[4], uv[4];
    long long rr[4]; int cc[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {           // issue every load of the iteration before any math
      const long long i = i0 + k * stride;
      if (i < nvec) {
        rr[k] = i / fv; cc[k] = static_cast<int>(i - rr[k] * fv);
        gv[k] = __ldcs(reinterpret_cast<const uint4*>(gate + rr[k] * in_stride) + cc[k]);
        uv[k] = __ldcs(reinterpret_cast<const uint4*>(up + rr[k] * in_stride) + cc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (i0 + k * stride < nvec) {
        float g[8], u[8]; unpack8(gv[k], g); unpack8(uv[k], u);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
        reinterpret_cast<uint4*>(out + rr[k] * F)[cc[k]] = pack8(g);
      }
    }
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ gate, const bf16* __restrict__ up,
                                  bf16* __restrict__ dgate, bf16* __restrict__ dup, long long rows, int F,
                                  long long in_stride) {
  const long long nvec = rows * (F >> 3);
  const int fv = F >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += 2 * stride) {
    uint4 gv[2], uv[2], dv[2];
    long long rr[2]; int cc[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const long long i = i0 + k * stride;
      if (i < nvec) {
        rr[k] = i / fv; cc[k] = static_cast<int>(i - rr[k] * fv);
        gv[k] = __ldcs(reinterpret_cast<const uint4*>(gate + rr[k] * in_stride) + cc[k]);
        uv[k] = __ldcs(reinterpret_cast<const uint4*>(up + rr[k] * in_stride) + cc[k]);
        dv[k] = __ldcs(reinterpret_cast<const uint4*>(dy + rr[k] * F) + cc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (i0 + k * stride < nvec) {
        float g[8], u[8], d[8], dg[8], du[8];
        unpack8(gv[k], g); unpack8(uv[k], u); unpack8(dv[k], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sg = 1.f / (1.f + __expf(-g[j]));
          du[j] = d[j] * g[j] * sg;
          dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
        }
        reinterpret_cast<uint4*>(dgate + rr[k] * in_stride)[cc[k]] = pack8(dg);
        reinterpret_cast<uint4*>(dup + rr[k] * in_stride)[cc[k]] = pack8(du);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// RoPE (rotate-half convention) applied in place to the first `rot_heads` heads of a packed
// [tokens, heads, D] tensor; positions[t] indexes cos/sin [table_rows, D/2] (fp32). sign = -1 gives the backward.
__global__ void rope_kernel(bf16* __restrict__ x, const float* __restrict__ cosb, const float* __restrict__ sinb,
                            const int* __restrict__ positions, long long tokens, int heads, int rot_heads, int D,
                            int table_rows, float sign) {
  const int half = D >> 1;
  const int hv = half >> 3;  // uint4 vectors per half
  const long long total = tokens * rot_heads * hv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % hv);
    const long long th = i / hv;
    const int h = static_cast<int>(th % rot_heads);
    const long long t = th / rot_heads;
    int pos = positions != nullptr ? positions[t] : static_cast<int>(t);
    pos = min(max(pos, 0), table_rows - 1);     // a position past the tables reads their last row, never outside them
    bf16* base = x + (t * heads + h) * D;
    uint4* p1 = reinterpret_cast<uint4*>(base) + c;
    uint4* p2 = reinterpret_cast<uint4*>(base + half) + c;
    float a[8], b[8];
    unpack8(*p1, a); unpack8(*p2, b);
    const float4* cp = reinterpret_cast<const float4*>(cosb + static_cast<long long>(pos) * half + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sinb + static_cast<long long>(pos) * half + c * 8);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float o1[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sn[j] * sign;
      o1[j] = a[j] * cs[j] - b[j] * s;
      o2[j] = b[j] * cs[j] + a[j] * s;
    }
    *p1 = pack8(o1); *p2 = pack8(o2);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Cross-entropy over one chunk of logits [rows, V] (bf16, row stride ld). One block per row:
//   pass 1: online (max, sum exp) and the target logit; loss = lse - z_t (+ z_loss * lse^2); rows with
//           target == ignore_index contribute nothing;
//   pass 2: logits <- (softmax - onehot) * scale * (1 + 2 z_loss lse)   in place (gradient of the summed loss)
// loss_out[row] is written (fp32); lse_out optional.
__global__ void __launch_bounds__(512)
ce_rows_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss_out,
               float* __restrict__ lse_out, int V, long long ld, int ignore_index, float grad_scale, float z_loss,
               float softcap, int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const long long tgt = targets[row];
  const bool live = tgt != ignore_index && tgt >= 0 && tgt < V;
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8]; unpack8(reinterpret_cast<const uint4*>(lr)[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 0; j < 8; ++j) { if (softcap > 0.f) f[j] = softcap * tanhf(f[j] / softcap); lm = fmaxf(lm, f[j]); }
    if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += blockDim.x) {
    float f = __bfloat162float(lr[i]);
    if (softcap > 0.f) f = softcap * tanhf(f / softcap);
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  const float gm = block_max(m, red);
  s = block_sum(s * __expf(m - gm), red);
  const float lse = gm + __logf(s);
  if (threadIdx.x == 0) {
    float zt = 0.f;
    if (live) { zt = __bfloat162float(lr[tgt]); if (softcap > 0.f) zt = softcap * tanhf(zt / softcap); }
    loss_out[row] = live ? (lse - zt + z_loss * lse * lse) : 0.f;
    if (lse_out != nullptr) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();
  const float gs = live ? grad_scale * (1.f + 2.f * z_loss * lse) : 0.f;
  const float gs1 = live ? grad_scale : 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8]; unpack8(reinterpret_cast<const uint4*>(lr)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float dcap = 1.f;
      float v = f[j];
      if (softcap > 0.f) { const float th = tanhf(v / softcap); v = softcap * th; dcap = 1.f - th * th; }
      float g = __expf(v - lse) * gs;
      if (static_cast<long long>(i) * 8 + j == tgt) g -= gs1;
      f[j] = g * dcap;
    }
    reinterpret_cast<uint4*>(lr)[i] = pack8(f);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += blockDim.x) {
    float v = __bfloat162float(lr[i]);
    float dcap = 1.f;
    if (softcap > 0.f) { const float th = tanhf(v / softcap); v = softcap * th; dcap = 1.f - th * th; }
    float g = __expf(v - lse) * gs;
    if (i == tgt) g -= gs1;
    lr[i] = __float2bfloat16(g * dcap);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Sum of squares of a flat bf16/fp32 buffer into partial[gridDim.x]; finalize computes the clip coefficient.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = static_cast<float>(g[i]);
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] = total sum of squares (+= when accumulate), out[1] = norm, out[2] = clip coefficient min(1, max_norm/norm)
__global__ void clip_coef_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, float max_norm,
                                 int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    if (accumulate) s += out[0];
    out[0] = s;
    const float norm = sqrtf(s);
    out[1] = norm;
    out[2] = (max_norm > 0.f && norm > max_norm) ? max_norm / (norm + 1e-6f) : 1.f;
  }
}

// ---------------------------------------------------------------------------------------------------------
// AdamW over a flat shard: fp32 master weights, fp32 moments, gradient in bf16 or fp32; writes the bf16 compute
// copy and (optionally) an EMA of the master in the same pass.
//   g' = g * grad_scale * clip[2]  (clip may be null);  p <- p (1 - lr wd) - lr m_hat / (sqrt(v_hat) + eps)
//   a non-finite total norm (clip[0]) skips the update when skip_nonfinite is set.
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ g, bf16* __restrict__ p_bf16, float* __restrict__ ema,
                             long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                             float bc2, float grad_scale, const float* __restrict__ clip, float ema_decay,
                             int skip_nonfinite) {
  float coef = grad_scale;
  if (clip != nullptr) {
    if (skip_nonfinite && !isfinite(clip[0])) return;
    coef *= clip[2];
  }
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gi = static_cast<float>(g[i]) * coef;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi; v[i] = vi;
    float pi = p[i];
    pi = pi * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    p[i] = pi;
    if (p_bf16 != nullptr) p_bf16[i] = __float2bfloat16(pi);
    if (ema != nullptr) ema[i] = ema_decay * ema[i] + (1.f - ema_decay) * pi;
  }
}

__global__ void ema_kernel(float* __restrict__ ema, const float* __restrict__ live, long long n, float decay) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    ema[i] = decay * ema[i] + (1.f - decay) * live[i];
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

// Row-wise fp8 quantisation: scale[row] = absmax(row) / 448; q = e4m3(x / scale). One warp per row.
__global__ void quantize_rows_fp8_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                                         long long rows, int d) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  const int nvec = d >> 3;
  float mx = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float f[8]; unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(f[j]));
  }
  mx = warp_max(mx);
  const float sc = mx > 0.f ? mx / 448.f : 1.f;
  if (lane == 0) scale[row] = sc;
  const float inv = 1.f / sc;
  for (int i = lane; i < nvec; i += 32) {
    float f[8]; unpack8(xr[i], f);
    uint32_t lo4 = 0, hi4 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo4 |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
      hi4 |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f[4 + j] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
    }
    reinterpret_cast<uint2*>(q + row * d)[i] = make_uint2(lo4, hi4);
  }
}

static inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace ew
}  // namespace dewb

using namespace dewb::ew;

#define STREAM(p) reinterpret_cast<cudaStream_t>(p)
#define LAST_ERR() static_cast<int>(cudaGetLastError())

// Select the device for this library's CUDA runtime on the calling thread.
extern "C" int dewb_set_device(int device) {
  // cudaSetDevice binds (and, the first time, creates) the device's primary context on the calling thread; it is not
  // a stream operation, so it is legal while another thread's stream is being captured into a graph.
  return static_cast<int>(cudaSetDevice(device));
}

extern "C" int dewb_rmsnorm_fwd(const void* x, const void* other, const void* w, void* y, void* h_out, float* rstd,
                                long long rows, int d, float eps, int mode, void* stream) {
  if (d % 8 != 0 || rows <= 0) return rows == 0 ? 0 : -3;
  const bf16 *xp = (const bf16*)x, *op = (const bf16*)other, *wp = (const bf16*)w;
  bf16 *yp = (bf16*)y, *hp = (bf16*)h_out;
  if (d <= 4096) {
    const int nvec = d >> 3;
    int G = 32;
    while (G > 1 && (G >> 1) >= nvec) G >>= 1;
    const int need = (nvec + G - 1) / G;
    const long long rows_per_block = 8LL * (32 / G);
    const unsigned blocks = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
    if (nvec >= 128) {
      const int vpt = (nvec + 127) / 128;
      const unsigned nb = static_cast<unsigned>(rows);
#define DEWB_FWD_BLOCK(MODE, VPT) rmsnorm_fwd_block_kernel<MODE, VPT><<<nb, 128, 0, STREAM(stream)>>>(xp, op, wp, yp, hp, rstd, d, eps)
#define DEWB_FWD_BMODE(VPT) do { if (mode == 0) DEWB_FWD_BLOCK(0, VPT); else if (mode == 1) DEWB_FWD_BLOCK(1, VPT); else DEWB_FWD_BLOCK(2, VPT); } while (0)
      if (vpt <= 1) DEWB_FWD_BMODE(1); else if (vpt <= 2) DEWB_FWD_BMODE(2); else DEWB_FWD_BMODE(4);
#undef DEWB_FWD_BMODE
#undef DEWB_FWD_BLOCK
      return LAST_ERR();
    }
#define DEWB_FWD_ROWS(MODE, VPL) rmsnorm_fwd_rows_kernel<MODE, VPL><<<blocks, 256, 0, STREAM(stream)>>>(xp, op, wp, yp, hp, rstd, rows, d, eps, G)
#define DEWB_FWD_MODE(VPL) do { if (mode == 0) DEWB_FWD_ROWS(0, VPL); else if (mode == 1) DEWB_FWD_ROWS(1, VPL); else DEWB_FWD_ROWS(2, VPL); } while (0)
    if (need <= 1) DEWB_FWD_MODE(1); else if (need <= 2) DEWB_FWD_MODE(2); else if (need <= 4) DEWB_FWD_MODE(4);
    else if (need <= 8) DEWB_FWD_MODE(8); else DEWB_FWD_MODE(16);
#undef DEWB_FWD_MODE
#undef DEWB_FWD_ROWS
    return LAST_ERR();
  }
  dim3 grid(static_cast<unsigned>(rows));
  if (mode == 0) rmsnorm_fwd_kernel<0><<<grid, NORM_THREADS, 0, STREAM(stream)>>>(xp, op, wp, yp, hp, rstd, d, eps);
  else if (mode == 1) rmsnorm_fwd_kernel<1><<<grid, NORM_THREADS, 0, STREAM(stream)>>>(xp, op, wp, yp, hp, rstd, d, eps);
  else rmsnorm_fwd_kernel<2><<<grid, NORM_THREADS, 0, STREAM(stream)>>>(xp, op, wp, yp, hp, rstd, d, eps);
  return LAST_ERR();
}

// Rows of scratch `dw_partial` the backward needs: one per block of its persistent grid.
extern "C" int dewb_rmsnorm_bwd_blocks(long long rows) {
  const long long cap = 148 * 2;
  return static_cast<int>(rows < cap ? rows : cap);
}

// dw_partial: fp32 scratch [dewb_rmsnorm_bwd_blocks(rows), d]. dw_f32 / dw_bf16: either may be null.
extern "C" int dewb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                const void* z, void* dx, void* dz, float* dw_partial, float* dw_f32, void* dw_bf16,
                                int accumulate, long long rows, int d, void* stream) {
  if (d % 8 != 0 || d > NORM_THREADS * 8 * BWD_COLS) return -3;
  if (rows <= 0) return 0;
  const int blocks = dewb_rmsnorm_bwd_blocks(rows);
  if (d <= 4096) {
    const int nvec = d >> 3;
    int G = 32;
    while (G > 1 && (G >> 1) >= nvec) G >>= 1;
    const int need = (nvec + G - 1) / G;
    const long long rows_per_block = 8LL * (32 / G);
    const unsigned nb = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
#define DEWB_BWD_ROWS(GATED, VPL) rmsnorm_bwd_dx_rows_kernel<GATED, VPL><<<nb, 256, 0, STREAM(stream)>>>( \
      (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, (const bf16*)z, (bf16*)dx, (bf16*)dz, rows, d, G)
#define DEWB_BWD_G(VPL) do { if (z != nullptr) DEWB_BWD_ROWS(true, VPL); else DEWB_BWD_ROWS(false, VPL); } while (0)
#define DEWB_BWD_BLOCK(GATED, VPT) rmsnorm_bwd_dx_block_kernel<GATED, VPT><<<static_cast<unsigned>(rows), 128, 0, STREAM(stream)>>>( \
      (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, (const bf16*)z, (bf16*)dx, (bf16*)dz, d)
#define DEWB_BWD_B(VPT) do { if (z != nullptr) DEWB_BWD_BLOCK(true, VPT); else DEWB_BWD_BLOCK(false, VPT); } while (0)
    if (nvec >= 128) {
      const int vpt = (nvec + 127) / 128;
      if (vpt <= 1) DEWB_BWD_B(1); else if (vpt <= 2) DEWB_BWD_B(2); else DEWB_BWD_B(4);
    }
    else if (need <= 1) DEWB_BWD_G(1); else if (need <= 2) DEWB_BWD_G(2); else if (need <= 4) DEWB_BWD_G(4);
    else if (need <= 8) DEWB_BWD_G(8); else DEWB_BWD_G(16);
#undef DEWB_BWD_B
#undef DEWB_BWD_BLOCK
#undef DEWB_BWD_G
#undef DEWB_BWD_ROWS
    // dw: column reduction with `blocks` row splits, folded by colsum_kernel
    int splits = blocks < 1 ? 1 : blocks;
    const long long max_useful = (rows + 7) / 8;
    if (splits > max_useful) splits = static_cast<int>(max_useful);
    dim3 g((nvec + 31) / 32, splits);
    if (z != nullptr) rmsnorm_dw_kernel<true><<<g, 256, 0, STREAM(stream)>>>((const bf16*)dy, (const bf16*)x, rstd, (const bf16*)z, dw_partial, rows, d);
    else rmsnorm_dw_kernel<false><<<g, 256, 0, STREAM(stream)>>>((const bf16*)dy, (const bf16*)x, rstd, nullptr, dw_partial, rows, d);
    colsum_kernel<<<(d + 255) / 256, 256, 0, STREAM(stream)>>>(dw_partial, splits, d, dw_f32, (bf16*)dw_bf16, accumulate);
    return LAST_ERR();
  }
  if (z != nullptr)
    rmsnorm_bwd_kernel<true><<<blocks, NORM_THREADS, 0, STREAM(stream)>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, (const bf16*)z, (bf16*)dx, (bf16*)dz,
        dw_partial, rows, d);
  else
    rmsnorm_bwd_kernel<false><<<blocks, NORM_THREADS, 0, STREAM(stream)>>>(
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, nullptr, (bf16*)dx, nullptr,
        dw_partial, rows, d);
  colsum_kernel<<<(d + 255) / 256, 256, 0, STREAM(stream)>>>(dw_partial, blocks, d, dw_f32, (bf16*)dw_bf16, accumulate);
  return LAST_ERR();
}

extern "C" int dewb_swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int F, long long in_stride,
                               void* stream) {
  if (F % 8 != 0 || in_stride % 8 != 0) return -3;
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(rows * (F >> 3), 256), 256, 0, STREAM(stream)>>>((const bf16*)gate, (const bf16*)up,
                                                                                (bf16*)out, rows, F, in_stride);
  return LAST_ERR();
}
extern "C" int dewb_swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup, long long rows,
                               int F, long long in_stride, void* stream) {
  if (F % 8 != 0 || in_stride % 8 != 0) return -3;
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(rows * (F >> 3), 256), 256, 0, STREAM(stream)>>>(
      (const bf16*)dy, (const bf16*)gate, (const bf16*)up, (bf16*)dgate, (bf16*)dup, rows, F, in_stride);
  return LAST_ERR();
}

extern "C" int dewb_rope(void* x, const float* cosb, const float* sinb, const int* positions, long long tokens,
                         int heads, int rot_heads, int D, int table_rows, float sign, void* stream) {
  if (D % 16 != 0 || table_rows <= 0) return -3;
  if (tokens <= 0 || rot_heads <= 0) return 0;
  rope_kernel<<<grid_for(tokens * rot_heads * (D >> 4), 256), 256, 0, STREAM(stream)>>>(
      (bf16*)x, cosb, sinb, positions, tokens, heads, rot_heads, D, table_rows, sign);
  return LAST_ERR();
}

extern "C" int dewb_ce_rows(void* logits, const long long* targets, float* loss, float* lse, long long rows, int V,
                            long long ld, int ignore_index, float grad_scale, float z_loss, float softcap,
                            int write_grad, void* stream) {
  if (ld % 8 != 0) return -3;
  if (rows <= 0) return 0;
  ce_rows_kernel<<<static_cast<unsigned>(rows), 512, 0, STREAM(stream)>>>((bf16*)logits, targets, loss, lse, V, ld,
                                                                          ignore_index, grad_scale, z_loss, softcap,
                                                                          write_grad);
  return LAST_ERR();
}

// partial: fp32 scratch of at least 1024 floats; out: 3 floats {sum sq, norm, clip coefficient}
extern "C" int dewb_grad_norm(const void* g, long long n, int is_bf16, float* partial, float* out, float max_norm,
                              int accumulate, void* stream) {
  const int blocks = grid_for(n, 512, 1024);
  if (is_bf16) sumsq_kernel<bf16><<<blocks, 512, 0, STREAM(stream)>>>((const bf16*)g, n, partial);
  else sumsq_kernel<float><<<blocks, 512, 0, STREAM(stream)>>>((const float*)g, n, partial);
  clip_coef_kernel<<<1, 256, 0, STREAM(stream)>>>(partial, blocks, out, max_norm, accumulate);
  return LAST_ERR();
}

extern "C" int dewb_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p_bf16, float* ema,
                          long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                          float grad_scale, const float* clip, float ema_decay, int skip_nonfinite, void* stream) {
  if (n <= 0) return 0;
  const int blocks = grid_for(n, 256);
  if (g_is_bf16)
    adamw_kernel<bf16><<<blocks, 256, 0, STREAM(stream)>>>(p, m, v, (const bf16*)g, (bf16*)p_bf16, ema, n, lr, beta1,
                                                           beta2, eps, wd, bc1, bc2, grad_scale, clip, ema_decay,
                                                           skip_nonfinite);
  else
    adamw_kernel<float><<<blocks, 256, 0, STREAM(stream)>>>(p, m, v, (const float*)g, (bf16*)p_bf16, ema, n, lr, beta1,
                                                            beta2, eps, wd, bc1, bc2, grad_scale, clip, ema_decay,
                                                            skip_nonfinite);
  return LAST_ERR();
}

// x [rows, d] bf16 (d % 8 == 0) -> q [rows, d] e4m3 bytes and scale [rows] fp32.
extern "C" int dewb_quantize_rows_fp8(const void* x, void* q, float* scale, long long rows, int d, void* stream) {
  if (d % 8 != 0) return -3;
  if (rows <= 0) return 0;
  quantize_rows_fp8_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, STREAM(stream)>>>(
      (const bf16*)x, (uint8_t*)q, scale, rows, d);
  return LAST_ERR();
}

extern "C" int dewb_ema(float* ema, const float* live, long long n, float decay, void* stream) {
  if (n <= 0) return 0;
  ema_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(ema, live, n, decay);
  return LAST_ERR();
}

extern "C" int dewb_cast_f32_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(src, (bf16*)dst, n);
  return LAST_ERR();
}

// ---------------------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that cannot allocate (declaration and rules of use: csrc/include/dewb_noalloc.h).
// The weight-gradient partial sums live in this file-scope device array instead of a caller-provided buffer.
#include "../include/dewb_noalloc.h"

static __device__ __align__(256) float g_noalloc_dw_partial[DEWB_NOALLOC_MAX_SPLITS * DEWB_NOALLOC_MAX_D];

// Device address of the array, per device. In host code the array's name is only a handle for the runtime's symbol
// table; the address a kernel can use comes from cudaGetSymbolAddress, asked for once with that device current.
static float* g_noalloc_ptr[64];

namespace {
// Makes `device` the current device for the lifetime of the object and puts the caller's device back afterwards, on
// every return path: the address looked up below and the kernels launched with it must belong to the same device.
struct NoallocDeviceScope {
  int prev = -1;
  int target;
  cudaError_t err = cudaSuccess;
  explicit NoallocDeviceScope(int device) : target(device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != target) err = cudaSetDevice(target);
  }
  ~NoallocDeviceScope() {
    if (prev >= 0 && prev != target) cudaSetDevice(prev);
  }
};
}  // namespace

static int noalloc_body(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                        float* dw_f32, void* dw_bf16, int accumulate, long long rows, int d, int device, void* stream) {
  if (g_noalloc_ptr[device] == nullptr) {
    // one-time set-up for this device (not to be done under stream capture); `device` is current here
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dw_partial);
    if (e != cudaSuccess || p == nullptr) return e != cudaSuccess ? static_cast<int>(e) : DEWB_NOALLOC_ERR_SYMBOL;
    // concurrent first calls from several host threads all store the same value: the race is harmless
    g_noalloc_ptr[device] = p;
  }
  float* partial = g_noalloc_ptr[device];
  const int nvec = d >> 3;
  int G = 32;
  while (G > 1 && (G >> 1) >= nvec) G >>= 1;
  const int need = (nvec + G - 1) / G;
  const long long rows_per_block = 8LL * (32 / G);
  const unsigned nb = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
#define DEWB_NA_ROWS(VPL) rmsnorm_bwd_dx_rows_kernel<false, VPL><<<nb, 256, 0, STREAM(stream)>>>( \
    (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, nullptr, (bf16*)dx, nullptr, rows, d, G)
#define DEWB_NA_BLOCK(VPT) rmsnorm_bwd_dx_block_kernel<false, VPT><<<static_cast<unsigned>(rows), 128, 0, STREAM(stream)>>>( \
    (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, nullptr, (bf16*)dx, nullptr, d)
  // the same kernel choice as dewb_rmsnorm_bwd, so both entries perform the same arithmetic
  if (nvec >= 128) {
    const int vpt = (nvec + 127) / 128;
    if (vpt <= 1) DEWB_NA_BLOCK(1); else if (vpt <= 2) DEWB_NA_BLOCK(2); else DEWB_NA_BLOCK(4);
  }
  else if (need <= 1) DEWB_NA_ROWS(1); else if (need <= 2) DEWB_NA_ROWS(2); else if (need <= 4) DEWB_NA_ROWS(4);
  else if (need <= 8) DEWB_NA_ROWS(8); else DEWB_NA_ROWS(16);
#undef DEWB_NA_BLOCK
#undef DEWB_NA_ROWS
  // every split row of the array that colsum reads below is written here first: stale contents never leak
  int splits = DEWB_NOALLOC_MAX_SPLITS;
  const long long max_useful = (rows + 7) / 8;
  if (splits > max_useful) splits = static_cast<int>(max_useful);
  dim3 g((nvec + 31) / 32, splits);
  rmsnorm_dw_kernel<false><<<g, 256, 0, STREAM(stream)>>>((const bf16*)dy, (const bf16*)x, rstd, nullptr, partial, rows, d);
  colsum_kernel<<<(d + 255) / 256, 256, 0, STREAM(stream)>>>(partial, splits, d, dw_f32, (bf16*)dw_bf16, accumulate);
  return LAST_ERR();
}

extern "C" int dewb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                        const void* dres, void* dx, float* dw_f32, void* dw_bf16, int accumulate,
                                        long long rows, int d, int device, void* stream) {
  if (d <= 0 || d % 8 != 0) return -3;
  if (d > DEWB_NOALLOC_MAX_D) return DEWB_NOALLOC_ERR_TOO_LARGE;
  if (device < 0 || device >= 64) return -3;
  if (rows <= 0) return 0;
  // `device` stays current from the address look-up to the last launch, whatever device the caller had current;
  // `stream` must be a stream of `device` (or null for its default stream)
  NoallocDeviceScope scope(device);
  if (scope.err != cudaSuccess) return static_cast<int>(scope.err);
  return noalloc_body(dy, x, w, rstd, dres, dx, dw_f32, dw_bf16, accumulate, rows, d, device, stream);
}
