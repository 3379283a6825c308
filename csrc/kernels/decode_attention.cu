// Paged decode attention (flash-decoding) for sm_100a: one new query token per row against that row's cached keys.
//
// grid = (row, kv head, key split). A CTA handles the G = Hq / Hkv query heads that share its KV head, so every cached
// key and value is read from HBM exactly once per row. Each of its 4 warps walks 32-key blocks of the split:
//   scores : lane = key      - each lane reads one key row (16-byte loads) and dots it with the G queries in smem
//   values : lane = d-slice  - the block's probabilities are broadcast by shuffle; value rows are read coalesced
// Online softmax per warp in fp32 (log2 domain); warps, then splits, are merged with the usual (max, sum, acc) algebra.
// The cache is paged: pool [pages, page_size, Hkv, D] for keys and for values, page_table [rows, max_pages] (int32),
// lengths [rows]. Optional per-token-per-head fp32 scales dequantise int8 / fp8-e4m3 pools.
// The kernel is bandwidth-bound by design (arithmetic intensity G FLOP/byte); tensor cores would not help at G <= 8.
//
// Capability parity: src/dew/nn/kernels/decode_attention.py (attend_paged: BLOCK 32 keys, key splits combined in
// fp32), src/dew/nn/kv_cache.py:1297-1320 (pool layout), :411-446 (int8 / fp8 KV quantisation).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

namespace dewb {
namespace decode {

constexpr int WARPS = 4;
constexpr int MAX_G = 8;

__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// KV element kinds
enum : int { KV_BF16 = 0, KV_INT8 = 1, KV_FP8 = 2 };

template <int KIND>
__device__ __forceinline__ void load8(const void* base, long long elem_off, float (&f)[8]) {
  if (KIND == KV_BF16) {
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_off);
    f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
    f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
  } else if (KIND == KV_INT8) {
    const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(base) + elem_off);
    const int8_t* b = reinterpret_cast<const int8_t*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(b[i]);
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(base) + elem_off);
    const __nv_fp8_e4m3* b = reinterpret_cast<const __nv_fp8_e4m3*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(b[i]);
  }
}

// partial results per (row, q head, split): m (log2 domain), l, acc[D]
// GT: the number of query heads per KV head when it is 1, 2, 4 or 8 (arrays and loops sized for it, no predicates);
// 0 = any count up to MAX_G, checked at run time.
template <int D, int KIND, int GT>
__global__ void __launch_bounds__(WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const void* __restrict__ kpool, const void* __restrict__ vpool,
                    const float* __restrict__ kscale, const float* __restrict__ vscale,
                    const int* __restrict__ page_table, const int* __restrict__ lengths, float* __restrict__ part_m,
                    float* __restrict__ part_l, float* __restrict__ part_acc, int Hq, int Hkv, int page_size,
                    int max_pages, int splits, float scale_log2, int window) {
  constexpr int DV = D / 32;                 // value elements per lane
  const int row = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  constexpr int GM = GT ? GT : MAX_G;          // compile-time bound of every per-head array and loop
  const int G = GT ? GT : Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ __align__(16) float sq[GM][D];
  __shared__ float sm_m[WARPS][GM], sm_l[WARPS][GM];
  __shared__ float sm_acc[WARPS][GM][D];
  __shared__ __align__(16) float sp[WARPS][32][GM];      // the current block's probabilities, [key][head]: one broadcast read per key
  __shared__ int stok[WARPS][32];                         // and the pool token index of each of its keys
  const int len = lengths[row];
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    sq[g][d] = __bfloat162float(q[(static_cast<long long>(row) * Hq + hk * G + g) * D + d]) * scale_log2;
  }
  __syncthreads();
  // keys of this split: [k_begin, k_end) in 32-key blocks, interleaved across the CTA's warps
  const int first = (window > 0 && len > window) ? len - window : 0;
  const int span = len - first;
  const int per_split = ((span + splits - 1) / splits + 31) / 32 * 32;
  const int k_begin = first + split * per_split;
  const int k_end = min(len, k_begin + per_split);
  float m[GM], l[GM], acc[GM][DV];
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DV; ++i) acc[g][i] = 0.f;
  }
  const int* table = page_table + static_cast<long long>(row) * max_pages;
  for (int kb = k_begin + warp * 32; kb < k_end; kb += WARPS * 32) {
    const int key = kb + lane;
    const bool live = key < k_end;
    float s[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) s[g] = -INFINITY;
    long long tok = 0;      // (page * page_size + slot) of this lane's key
    if (live) {
      const int page = table[key / page_size];
      tok = static_cast<long long>(page) * page_size + (key % page_size);
      const long long base = (tok * Hkv + hk) * D;
      float dot[GM];
#pragma unroll
      for (int g = 0; g < GM; ++g) dot[g] = 0.f;
      // the key row in halves of 64 values: all eight loads of a half are in flight before the first is used, and the
      // queries come from shared memory as float4 broadcasts
#pragma unroll
      for (int h0 = 0; h0 < D; h0 += 64) {
        float kf[8][8];
#pragma unroll
        for (int c = 0; c < 8; ++c) load8<KIND>(kpool, base + h0 + c * 8, kf[c]);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
#pragma unroll
          for (int g = 0; g < GM; ++g)
            if (GT != 0 || g < G) {
              const float4 qa = *reinterpret_cast<const float4*>(&sq[g][h0 + c * 8]);
              const float4 qb = *reinterpret_cast<const float4*>(&sq[g][h0 + c * 8 + 4]);
              dot[g] += kf[c][0] * qa.x + kf[c][1] * qa.y + kf[c][2] * qa.z + kf[c][3] * qa.w + kf[c][4] * qb.x + kf[c][5] * qb.y +
                        kf[c][6] * qb.z + kf[c][7] * qb.w;
            }
        }
      }
      const float ks = KIND == KV_BF16 ? 1.f : kscale[tok * Hkv + hk];
#pragma unroll
      for (int g = 0; g < GM; ++g) if (GT != 0 || g < G) s[g] = dot[g] * ks;
    }
    // online softmax update (per query head), block maximum by warp reduction
    float p[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
      if (GT != 0 || g < G) {
        float bm = s[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
        const float mn = fmaxf(m[g], bm);
        const float alpha = m[g] == -INFINITY ? 0.f : exp2f(m[g] - mn);
        p[g] = live ? exp2f(s[g] - mn) : 0.f;
        float ps = p[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l[g] = l[g] * alpha + ps;
        m[g] = mn;
#pragma unroll
        for (int i = 0; i < DV; ++i) acc[g][i] *= alpha;
      }
    }
    // values: lane owns columns [lane * DV, lane * DV + DV); walk the block's keys
    // eight keys at a time: their addresses, then their eight loads (all in flight together), then the products; keys
    // past the end of the block carry zero probability and re-read a valid row
    const int nkeys = min(32, k_end - kb);
    __syncwarp();
#pragma unroll
    for (int g = 0; g < GM; ++g) sp[warp][lane][g] = (GT != 0 || g < G) ? p[g] : 0.f;
    stok[warp][lane] = static_cast<int>(tok);
    __syncwarp();
    for (int j0 = 0; j0 < nkeys; j0 += 8) {
      long long tj[8];
      float vf[8][DV];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) tj[jj] = stok[warp][min(j0 + jj, nkeys - 1)];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const long long vb = (tj[jj] * Hkv + hk) * D + lane * DV;
        if (KIND == KV_BF16) {
          const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(vpool) + vb;
          if (DV == 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(vp);
            vf[jj][0] = bf_lo(v.x); vf[jj][1] = bf_hi(v.x); vf[jj][2] = bf_lo(v.y); vf[jj][3] = bf_hi(v.y);
          } else {
#pragma unroll
            for (int i = 0; i < DV; ++i) vf[jj][i] = __bfloat162float(vp[i]);
          }
        } else if (KIND == KV_INT8) {
          const int8_t* vp = reinterpret_cast<const int8_t*>(vpool) + vb;
#pragma unroll
          for (int i = 0; i < DV; ++i) vf[jj][i] = static_cast<float>(vp[i]);
        } else {
          const __nv_fp8_e4m3* vp = reinterpret_cast<const __nv_fp8_e4m3*>(vpool) + vb;
#pragma unroll
          for (int i = 0; i < DV; ++i) vf[jj][i] = static_cast<float>(vp[i]);
        }
      }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int j = min(j0 + jj, 31);
        const bool on = j0 + jj < nkeys;
        const float vs = KIND == KV_BF16 ? 1.f : vscale[tj[jj] * Hkv + hk];
        float pk[GM];
        if (GM % 4 == 0) {
#pragma unroll
          for (int g4 = 0; g4 < GM / 4; ++g4) {
            const float4 t4 = *reinterpret_cast<const float4*>(&sp[warp][j][g4 * 4]);
            pk[g4 * 4] = t4.x; pk[g4 * 4 + 1] = t4.y; pk[g4 * 4 + 2] = t4.z; pk[g4 * 4 + 3] = t4.w;
          }
        } else {
#pragma unroll
          for (int g = 0; g < GM; ++g) pk[g] = sp[warp][j][g];
        }
#pragma unroll
        for (int g = 0; g < GM; ++g) {
          if (GT != 0 || g < G) {
            const float pj = on ? pk[g] * vs : 0.f;
#pragma unroll
            for (int i = 0; i < DV; ++i) acc[g][i] += pj * vf[jj][i];
          }
        }
      }
    }
  }
  // merge the CTA's warps
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    if (GT != 0 || g < G) {
      if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
      for (int i = 0; i < DV; ++i) sm_acc[warp][g][lane * DV + i] = acc[g][i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = sm_m[w][g] == -INFINITY ? 0.f : exp2f(sm_m[w][g] - mm);
      ll += sm_l[w][g] * f;
      a += sm_acc[w][g][d] * f;
    }
    const long long o = (static_cast<long long>(row) * Hq + hk * G + g) * splits + split;
    part_acc[o * D + d] = a;
    if (d == 0) { part_m[o] = mm; part_l[o] = ll; }
  }
}

// out[row, h, :] = sum_s acc_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M); optional attention sink per head
template <int D>
__global__ void decode_combine_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                      const float* __restrict__ part_acc, const float* __restrict__ sinks,
                                      __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int Hq, int splits) {
  const long long rh = blockIdx.x;          // row * Hq + h
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_m[rh * splits + s]);
  float L = 0.f, a = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_m[rh * splits + s];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
    L += part_l[rh * splits + s] * f;
    a += part_acc[(rh * splits + s) * D + d] * f;
  }
  if (sinks != nullptr && M > -INFINITY) {
    const float sk = sinks[rh % Hq] * 1.4426950408889634f;      // the sink is a logit in natural units
    const float Mn = fmaxf(M, sk);
    const float f = exp2f(M - Mn);
    L = L * f + exp2f(sk - Mn);
    a *= f;
    M = Mn;
  }
  if (d < D) out[rh * D + d] = __float2bfloat16(L > 0.f ? a / L : 0.f);
  if (d == 0 && lse != nullptr) lse[rh] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
}

// Append one token per row to the paged pools: k_new / v_new [rows, Hkv, D] -> pool slot lengths[row] of the row.
// KIND 1 / 2 quantise per token per head: scale = absmax / limit (127 for int8, 448 for fp8-e4m3).
template <int KIND>
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                 void* __restrict__ kpool, void* __restrict__ vpool, float* __restrict__ kscale,
                                 float* __restrict__ vscale, const int* __restrict__ page_table,
                                 const int* __restrict__ positions, int Hkv, int D, int page_size, int max_pages) {
  const int row = blockIdx.x, hk = blockIdx.y, which = blockIdx.z;     // which: 0 keys, 1 values
  const int pos = positions[row];
  if (pos < 0) return;
  const int page = page_table[static_cast<long long>(row) * max_pages + pos / page_size];
  const long long tok = static_cast<long long>(page) * page_size + pos % page_size;
  const __nv_bfloat16* src = (which ? v_new : k_new) + (static_cast<long long>(row) * Hkv + hk) * D;
  void* pool = which ? vpool : kpool;
  const long long dst = (tok * Hkv + hk) * D;
  if (KIND == KV_BF16) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) reinterpret_cast<__nv_bfloat16*>(pool)[dst + d] = src[d];
    return;
  }
  __shared__ float red[32];
  float mx = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) mx = fmaxf(mx, fabsf(__bfloat162float(src[d])));
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = 0.f;
  for (int w = 0; w < (blockDim.x + 31) / 32; ++w) mx = fmaxf(mx, red[w]);
  const float limit = KIND == KV_INT8 ? 127.f : 448.f;
  const float sc = mx > 0.f ? mx / limit : 1.f;
  if (threadIdx.x == 0) (which ? vscale : kscale)[tok * Hkv + hk] = sc;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float x = __bfloat162float(src[d]) / sc;
    if (KIND == KV_INT8) reinterpret_cast<int8_t*>(pool)[dst + d] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(x))));
    else reinterpret_cast<__nv_fp8_e4m3*>(pool)[dst + d] = __nv_fp8_e4m3(x);
  }
}

}  // namespace decode
}  // namespace dewb

using namespace dewb::decode;

// Scratch (caller-provided fp32): part_m, part_l [rows * Hq * splits], part_acc [rows * Hq * splits * D].
extern "C" int dewb_paged_decode(const void* q, const void* kpool, const void* vpool, const float* kscale,
                                 const float* vscale, const int* page_table, const int* lengths, const float* sinks,
                                 void* out, float* lse, float* part_m, float* part_l, float* part_acc, int rows, int Hq,
                                 int Hkv, int D, int page_size, int max_pages, int splits, float scale, int window,
                                 int kv_kind, void* stream_ptr) {
  if (rows <= 0) return 0;
  if ((D != 64 && D != 128 && D != 256) || Hq % Hkv != 0 || Hq / Hkv > MAX_G || splits < 1) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(rows, Hkv, splits);
  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(q);
  const int Gq = Hq / Hkv;
#define DEWB_DECODE_G(DD, KK, GG) paged_decode_kernel<DD, KK, GG><<<grid, WARPS * 32, 0, stream>>>( \
    qp, kpool, vpool, kscale, vscale, page_table, lengths, part_m, part_l, part_acc, Hq, Hkv, page_size, max_pages, splits, scale_log2, window)
#define DEWB_DECODE(DD, KK) do { if (Gq == 4) DEWB_DECODE_G(DD, KK, 4); else if (Gq == 8) DEWB_DECODE_G(DD, KK, 8); \
    else if (Gq == 1) DEWB_DECODE_G(DD, KK, 1); else if (Gq == 2) DEWB_DECODE_G(DD, KK, 2); else DEWB_DECODE_G(DD, KK, 0); } while (0)
#define DEWB_DECODE_D(KK) do { if (D == 64) DEWB_DECODE(64, KK); else if (D == 128) DEWB_DECODE(128, KK); else DEWB_DECODE(256, KK); } while (0)
  if (kv_kind == KV_BF16) DEWB_DECODE_D(KV_BF16); else if (kv_kind == KV_INT8) DEWB_DECODE_D(KV_INT8); else DEWB_DECODE_D(KV_FP8);
#undef DEWB_DECODE_D
#undef DEWB_DECODE
#undef DEWB_DECODE_G
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 64) decode_combine_kernel<64><<<rows * Hq, 64, 0, stream>>>(part_m, part_l, part_acc, sinks, op, lse, Hq, splits);
  else if (D == 128) decode_combine_kernel<128><<<rows * Hq, 128, 0, stream>>>(part_m, part_l, part_acc, sinks, op, lse, Hq, splits);
  else decode_combine_kernel<256><<<rows * Hq, 256, 0, stream>>>(part_m, part_l, part_acc, sinks, op, lse, Hq, splits);
  return static_cast<int>(cudaGetLastError());
}

// One decode step's packed projection output qkv [rows, Hq + 2 Hkv, D] (bf16): rotate the query and key heads in place
// (rotate-half RoPE at positions[row]; cos / sin [table_rows, D / 2] fp32, null = no rotation) and write the row's rotated key
// heads and its value heads into the paged bf16 cache at slot positions[row].  One launch where a rotation kernel, an append
// kernel and four copies of strided slices ran.  Rows with positions[row] < 0 are left alone.
__global__ void rope_append_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosb, const float* __restrict__ sinb,
                                   const int* __restrict__ positions, int Hq, int Hkv, int D, int table_rows,
                                   __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool,
                                   const int* __restrict__ page_table, int page_size, int max_pages) {
  const int row = blockIdx.x, head = blockIdx.y;
  const int pos = positions[row];
  if (pos < 0) return;
  const int half = D >> 1;
  const int c = threadIdx.x;                                   // uint4 chunk within a half
  if (c >= (half >> 3)) return;
  __nv_bfloat16* base = qkv + (static_cast<long long>(row) * (Hq + 2 * Hkv) + head) * D;
  uint4 lo = *(reinterpret_cast<const uint4*>(base) + c);
  uint4 hi = *(reinterpret_cast<const uint4*>(base + half) + c);
  const bool is_v = head >= Hq + Hkv;
  if (!is_v && cosb != nullptr) {
    const int tp = min(pos, table_rows - 1);
    const float4* cp = reinterpret_cast<const float4*>(cosb + static_cast<long long>(tp) * half + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sinb + static_cast<long long>(tp) * half + c * 8);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t a[4] = {lo.x, lo.y, lo.z, lo.w}, b[4] = {hi.x, hi.y, hi.z, hi.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a0 = __uint_as_float(a[j] << 16), a1 = __uint_as_float(a[j] & 0xffff0000u);
      const float b0 = __uint_as_float(b[j] << 16), b1 = __uint_as_float(b[j] & 0xffff0000u);
      const float x0 = a0 * cs[2 * j] - b0 * sn[2 * j], x1 = a1 * cs[2 * j + 1] - b1 * sn[2 * j + 1];
      const float y0 = b0 * cs[2 * j] + a0 * sn[2 * j], y1 = b1 * cs[2 * j + 1] + a1 * sn[2 * j + 1];
      __nv_bfloat162 p = __floats2bfloat162_rn(x0, x1), q2 = __floats2bfloat162_rn(y0, y1);
      o1[j] = *reinterpret_cast<uint32_t*>(&p);
      o2[j] = *reinterpret_cast<uint32_t*>(&q2);
    }
    lo = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    hi = make_uint4(o2[0], o2[1], o2[2], o2[3]);
    *(reinterpret_cast<uint4*>(base) + c) = lo;
    *(reinterpret_cast<uint4*>(base + half) + c) = hi;
  }
  if (head >= Hq) {
    const int hk = is_v ? head - Hq - Hkv : head - Hq;
    const int page = page_table[static_cast<long long>(row) * max_pages + pos / page_size];
    const long long tok = static_cast<long long>(page) * page_size + pos % page_size;
    __nv_bfloat16* dst = (is_v ? vpool : kpool) + (tok * Hkv + hk) * D;
    *(reinterpret_cast<uint4*>(dst) + c) = lo;
    *(reinterpret_cast<uint4*>(dst + half) + c) = hi;
  }
}

extern "C" int dewb_rope_append(void* qkv, const float* cosb, const float* sinb, const int* positions, int rows, int Hq, int Hkv,
                                int D, int table_rows, void* kpool, void* vpool, const int* page_table, int page_size,
                                int max_pages, void* stream_ptr) {
  if (rows <= 0) return 0;
  if (D % 16 != 0 || D > 512 || (cosb != nullptr && table_rows <= 0)) return -3;
  dim3 grid(rows, Hq + 2 * Hkv);
  rope_append_kernel<<<grid, 32, 0, reinterpret_cast<cudaStream_t>(stream_ptr)>>>(
      reinterpret_cast<__nv_bfloat16*>(qkv), cosb, sinb, positions, Hq, Hkv, D, table_rows, reinterpret_cast<__nv_bfloat16*>(kpool),
      reinterpret_cast<__nv_bfloat16*>(vpool), page_table, page_size, max_pages);
  return static_cast<int>(cudaGetLastError());
}

// positions[row] = slot to write (the row's current length), or < 0 to skip the row.
extern "C" int dewb_kv_append(const void* k_new, const void* v_new, void* kpool, void* vpool, float* kscale,
                              float* vscale, const int* page_table, const int* positions, int rows, int Hkv, int D,
                              int page_size, int max_pages, int kv_kind, void* stream_ptr) {
  if (rows <= 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  dim3 grid(rows, Hkv, 2);
  const __nv_bfloat16 *kp = reinterpret_cast<const __nv_bfloat16*>(k_new), *vp = reinterpret_cast<const __nv_bfloat16*>(v_new);
  if (kv_kind == KV_BF16) kv_append_kernel<KV_BF16><<<grid, 128, 0, stream>>>(kp, vp, kpool, vpool, kscale, vscale, page_table, positions, Hkv, D, page_size, max_pages);
  else if (kv_kind == KV_INT8) kv_append_kernel<KV_INT8><<<grid, 128, 0, stream>>>(kp, vp, kpool, vpool, kscale, vscale, page_table, positions, Hkv, D, page_size, max_pages);
  else kv_append_kernel<KV_FP8><<<grid, 128, 0, stream>>>(kp, vp, kpool, vpool, kscale, vscale, page_table, positions, Hkv, D, page_size, max_pages);
  return static_cast<int>(cudaGetLastError());
}

// The second stage alone: out [rows, Hq, D] bf16 from the per-split partials (used after dewb_paged_decode_stream).
extern "C" int dewb_decode_combine(const float* part_m, const float* part_l, const float* part_acc, const float* sinks,
                                   void* out, float* lse, int rows, int Hq, int D, int splits, void* stream_ptr) {
  if (rows <= 0) return 0;
  if (D != 64 && D != 128 && D != 256) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 64) decode_combine_kernel<64><<<rows * Hq, 64, 0, stream>>>(part_m, part_l, part_acc, sinks, op, lse, Hq, splits);
  else if (D == 128) decode_combine_kernel<128><<<rows * Hq, 128, 0, stream>>>(part_m, part_l, part_acc, sinks, op, lse, Hq, splits);
  else decode_combine_kernel<256><<<rows * Hq, 256, 0, stream>>>(part_m, part_l, part_acc, sinks, op, lse, Hq, splits);
  return static_cast<int>(cudaGetLastError());
}
