// Row-wise l2 normalisation (the q / k normalisation in front of the gated delta rule), forward and backward.
//   y = x / max(||x||, eps)             one warp per row, fp32 arithmetic, bf16 in and out
//   dx = (dy - y <y, dy>) / max(||x||, eps)
// The input rows may be strided views (a head slice of a wider projection): row r = (token, head) starts at
// token * token_stride + head * head_stride elements.  Outputs are contiguous [rows, D].
// Capability: the l2-normalised q and k of src/dew/nn/linear.py:1107-1408 (GatedDeltaNet).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace dewb {
namespace l2n {

constexpr uint32_t FULL = 0xffffffffu;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}

// D <= 1024, D % 8 == 0: each lane holds up to 4 pieces of 8 values
__global__ void __launch_bounds__(256)
l2norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ rnorm,
                  long long rows, int heads, long long token_stride, long long head_stride, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int nvec = D >> 3;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const long long tok = r / heads;
    const int hd = static_cast<int>(r - tok * heads);
    const uint4* xr = reinterpret_cast<const uint4*>(x + tok * token_stride + hd * head_stride);
    float f[4][8];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = lane + 32 * u;
      if (i < nvec) {
        unpack8(xr[i], f[u]);
#pragma unroll
        for (int c = 0; c < 8; ++c) ss = fmaf(f[u][c], f[u][c], ss);
      }
    }
    ss = warp_sum(ss);
    const float inv = 1.f / fmaxf(sqrtf(ss), eps);
    if (lane == 0 && rnorm != nullptr) rnorm[r] = inv;
    uint4* yr = reinterpret_cast<uint4*>(y + r * D);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = lane + 32 * u;
      if (i < nvec)
        yr[i] = make_uint4(pack2(f[u][0] * inv, f[u][1] * inv), pack2(f[u][2] * inv, f[u][3] * inv),
                           pack2(f[u][4] * inv, f[u][5] * inv), pack2(f[u][6] * inv, f[u][7] * inv));
    }
  }
}

__global__ void __launch_bounds__(256)
l2norm_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rnorm,
                  __nv_bfloat16* __restrict__ dx, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int nvec = D >> 3;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const uint4* yr = reinterpret_cast<const uint4*>(y + r * D);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + r * D);
    float fy[4][8], fg[4][8];
    float dot = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = lane + 32 * u;
      if (i < nvec) {
        unpack8(yr[i], fy[u]);
        unpack8(gr[i], fg[u]);
#pragma unroll
        for (int c = 0; c < 8; ++c) dot = fmaf(fy[u][c], fg[u][c], dot);
      }
    }
    dot = warp_sum(dot);
    const float inv = rnorm[r];
    uint4* xr = reinterpret_cast<uint4*>(dx + r * D);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = lane + 32 * u;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) o[c] = (fg[u][c] - fy[u][c] * dot) * inv;
        xr[i] = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
      }
    }
  }
}

static inline int grid_for_rows(long long rows) {
  long long b = (rows * 32 + 255) / 256;
  if (b < 1) b = 1;
  return static_cast<int>(b < 148 * 16 ? b : 148 * 16);
}

}  // namespace l2n
}  // namespace dewb

// x: bf16 rows of D values, row r = (token r / heads, head r % heads) at token * token_stride + head * head_stride elements
// (strides multiples of 8); y bf16 [rows, D]; rnorm fp32 [rows] (may be null) = 1 / max(||x||, eps).
extern "C" int dewb_l2norm_fwd(const void* x, void* y, float* rnorm, long long rows, int heads, long long token_stride,
                               long long head_stride, int D, float eps, void* stream) {
  using namespace dewb::l2n;
  if (D <= 0 || D > 1024 || D % 8 != 0 || heads <= 0 || token_stride % 8 != 0 || head_stride % 8 != 0) return -3;
  if (rows <= 0) return 0;
  l2norm_fwd_kernel<<<grid_for_rows(rows), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y), rnorm, rows, heads, token_stride,
      head_stride, D, eps);
  return static_cast<int>(cudaGetLastError());
}

// y, dy: bf16 [rows, D] contiguous; dx bf16 [rows, D].
extern "C" int dewb_l2norm_bwd(const void* y, const void* dy, const float* rnorm, void* dx, long long rows, int D,
                               void* stream) {
  using namespace dewb::l2n;
  if (D <= 0 || D > 1024 || D % 8 != 0) return -3;
  if (rows <= 0) return 0;
  l2norm_bwd_kernel<<<grid_for_rows(rows), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), reinterpret_cast<const __nv_bfloat16*>(dy), rnorm,
      reinterpret_cast<__nv_bfloat16*>(dx), rows, D);
  return static_cast<int>(cudaGetLastError());
}
