// Mamba-2 SSD forward scan for sm_100a (chunk 64, state dimension N = 128, head dimension P = 64).
//
// One CTA walks the chunks of one (batch, pair of heads): two heads of the same B / C group share every key / query
// operand, so their 64-wide value rows are stacked into the 128 rows (TMEM lanes) of one accumulator.  With a the
// per-step log decay dt * A of a head, g its running sum inside the chunk, X~ = x dt:
//     y_i  = e^{g_i} C_i S0 + sum_{j <= i} (C_i . B_j) e^{g_i - g_j} X~_j
//     S1   = e^{g_L} S0 + sum_j e^{g_L - g_j} X~_j (x) B_j
// computed transposed (rows = value index p of the two heads):
//     o1 = S^T C^T ;  o2 = X~^T P_h^T (one product per head, the other head's rows of the operand are zero) ;
//     dS = (X~ e^{g_L - g})^T B ;  y^T = e^{g} o1 + o2 ;  S^T <- e^{g_L} S^T + dS
// P_h = (C B^T) o e^{g_i - g_j} (lower triangle) and g arrive from the caller per head.  Same roles and bounded waits
// as the gated-delta-rule scan: warps 0..3 math (thread = TMEM lane), warp 4 TMA producer, warp 5 MMA issuer.
//
// Replaces the reference's ported SSD forward kernels ChunkState / StatePassing / ChunkScan
// (src/dew/nn/kernels/mamba_ssd.py:421-660).
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace dewb {
namespace ssd {

constexpr int ND = 128;           // state dimension (rows of B and C)
constexpr int PD = 64;            // head dimension
constexpr int CH = 64;
constexpr uint32_t FULL = 0xffffffffu;
constexpr int THREADS = 192;
constexpr int TMA_WARP = 4, MMA_WARP = 5;
constexpr int T16 = CH * 128 * 2;                      // [64 x 128] bf16 tile (two 64-column sub-tiles)
constexpr int T8 = CH * CH * 2;                        // [64 x 64] bf16 tile
constexpr int STAGE = 3 * T16 + 2 * T8;                // X~ pair, C, B, P of both heads
constexpr int OFF_STATE = 2 * STAGE;                   // [128 x 128] bf16 state tile
constexpr int OFF_VN0 = OFF_STATE + 2 * T16;           // X~^T of head 0 (rows 64..127 zero)
constexpr int OFF_VN1 = OFF_VN0 + T16;                 // X~^T of head 1 (rows 0..63 zero)
constexpr int OFF_VD = OFF_VN1 + T16;                  // decayed X~^T of both heads
constexpr int OFF_G = OFF_VD + T16;                    // g: [stage][head][64]
constexpr int OFF_BARS = OFF_G + 2 * 2 * CH * 4;
constexpr int SMEM = OFF_BARS + 256;
constexpr int F_X = 0, F_C = T16, F_B = 2 * T16, F_P0 = 3 * T16, F_P1 = 3 * T16 + T8;
static_assert(SMEM <= 232448, "ssd scan exceeds the shared memory of an SM");

struct Bars {
  uint64_t in_full[2], in_empty[2], s_ready, vn_ready, out_full;
  uint32_t tmem_base;
  int abort_flag, poisoned;
};
static_assert(sizeof(Bars) <= 256, "Bars must fit its slot");

__device__ __forceinline__ uint32_t swz(int r, int c16) { return static_cast<uint32_t>(r * 128 + ((c16 ^ (r & 7)) << 4)); }

__device__ __forceinline__ void write_state_row(uint8_t* tile, int v, const float (&S)[ND]) {
#pragma unroll
  for (int c16 = 0; c16 < 16; ++c16) {
    uint4 pk;
    pk.x = pack_bf16(S[c16 * 8 + 0], S[c16 * 8 + 1]); pk.y = pack_bf16(S[c16 * 8 + 2], S[c16 * 8 + 3]);
    pk.z = pack_bf16(S[c16 * 8 + 4], S[c16 * 8 + 5]); pk.w = pack_bf16(S[c16 * 8 + 6], S[c16 * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + (c16 >> 3) * (128 * 128) + swz(v, c16 & 7)) = pk;
  }
}

__global__ void __launch_bounds__(THREADS, 1)
ssd_scan_fwd_kernel(const __grid_constant__ CUtensorMap tx, const __grid_constant__ CUtensorMap tc,
                    const __grid_constant__ CUtensorMap tb, const __grid_constant__ CUtensorMap tp,
                    const float* __restrict__ gc, const float* __restrict__ initial, __nv_bfloat16* __restrict__ out,
                    float* __restrict__ final_state, int T, int H, int G, int Tp, int N, int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    return;
  }
  Bars* bars = reinterpret_cast<Bars*>(smem + OFF_BARS);
  if (threadIdx.x == 0) bars->poisoned = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (bars->poisoned != 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hp = H / 2;
  const int x = blockIdx.x, b = x / Hp, hp = x % Hp;
  const int h0 = 2 * hp;
  const int grp = h0 / (H / G);
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->in_full[i], 1); mbar_init(&bars->in_empty[i], 4); }
    mbar_init(&bars->s_ready, 4);
    mbar_init(&bars->vn_ready, 4);
    mbar_init(&bars->out_full, 1);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == MMA_WARP) { tmem_alloc(&bars->tmem_base, 256); tmem_relinquish(); }
  // the halves of the two X~^T operand tiles that belong to the other head stay zero for the whole kernel
  for (int i = tid; i < 2 * T16 / 16; i += THREADS) reinterpret_cast<uint4*>(smem + OFF_VN0)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  uint8_t* sState = smem + OFF_STATE;
  uint8_t* sVn0 = smem + OFF_VN0;
  uint8_t* sVn1 = smem + OFF_VN1;
  uint8_t* sVd = smem + OFF_VD;
  float* sG = reinterpret_cast<float*>(smem + OFF_G);
  constexpr int TM_O1 = 0, TM_O2 = 64, TM_DS = 128;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      tma_prefetch_desc(&tx); tma_prefetch_desc(&tc); tma_prefetch_desc(&tb); tma_prefetch_desc(&tp);
      for (int n = 0; n < N; ++n) {
        const int s = n & 1; const uint32_t ph = (n >> 1) & 1;
        if (!mbar_wait(&bars->in_empty[s], ph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); break; }
        uint8_t* st = smem + s * STAGE;
        uint64_t* bar = &bars->in_full[s];
        mbar_expect_tx(bar, STAGE + 2 * CH * 4);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          tma_load_4d(st + F_X + t * (CH * 128), &tx, bar, t * 64, hp, n * CH, b);
          tma_load_4d(st + F_C + t * (CH * 128), &tc, bar, t * 64, grp, n * CH, b);
          tma_load_4d(st + F_B + t * (CH * 128), &tb, bar, t * 64, grp, n * CH, b);
        }
        const long long r0 = (static_cast<long long>(b) * H + h0) * Tp + n * CH;
        tma_load_2d(st + F_P0, &tp, bar, 0, static_cast<int>(r0));
        tma_load_2d(st + F_P1, &tp, bar, 0, static_cast<int>(r0 + Tp));
        bulk_load_1d(sG + (s * 2 + 0) * CH, gc + r0, CH * 4, bar);
        bulk_load_1d(sG + (s * 2 + 1) * CH, gc + r0 + Tp, CH * 4, bar);
      }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_n64 = make_idesc(128, 64, 1, 1, 0, 0);
      constexpr uint32_t idesc_ds = make_idesc(128, 128, 1, 1, 0, 1);
      const uint32_t sa = smem_u32(sState), v0a = smem_u32(sVn0), v1a = smem_u32(sVn1), vda = smem_u32(sVd);
      for (int n = 0; n < N; ++n) {
        const int s = n & 1; const uint32_t ph = (n >> 1) & 1;
        const uint32_t st = smem_u32(smem + s * STAGE);
        if (!mbar_wait(&bars->in_full[s], ph, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); break; }
        if (!mbar_wait(&bars->s_ready, n & 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_OTHER); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < ND / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (128 * 128) + (kk & 3) * 32, boff = (kk >> 2) * (CH * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem + TM_O1, make_sdesc_sw128(sa + aoff, 16, 1024), make_sdesc_sw128(st + F_C + boff, 16, 1024),
                       idesc_n64, kk > 0 ? 1u : 0u);
        }
        if (!mbar_wait(&bars->vn_ready, n & 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_OTHER); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)
          umma_bf16_ss(tmem + TM_O2, make_sdesc_sw128(v0a + kk * 32, 16, 1024), make_sdesc_sw128(st + F_P0 + kk * 32, 16, 1024),
                       idesc_n64, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)
          umma_bf16_ss(tmem + TM_O2, make_sdesc_sw128(v1a + kk * 32, 16, 1024), make_sdesc_sw128(st + F_P1 + kk * 32, 16, 1024),
                       idesc_n64, 1u);
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)
          umma_bf16_ss(tmem + TM_DS, make_sdesc_sw128(vda + kk * 32, 16, 1024),
                       make_sdesc_sw128(st + F_B + kk * 2048, CH * 128, 1024), idesc_ds, kk > 0 ? 1u : 0u);
        umma_commit(&bars->out_full);
      }
    }
  } else {
    const int v = tid;                                   // rows 0..63: head h0, rows 64..127: head h0 + 1
    const int hh = v >> 6;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float S[ND];
    if (initial != nullptr) {
      // initial / final state: [B, H, P, N] fp32; this thread's row is (head h0 + hh, p = v & 63)
      const float* src = initial + ((static_cast<long long>(b) * H + h0 + hh) * PD + (v & 63)) * ND;
#pragma unroll
      for (int d = 0; d < ND; d += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(src + d);
        S[d] = q4.x; S[d + 1] = q4.y; S[d + 2] = q4.z; S[d + 3] = q4.w;
      }
    } else {
#pragma unroll
      for (int d = 0; d < ND; ++d) S[d] = 0.f;
    }
    write_state_row(sState, v, S);
    fence_proxy_async();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars->s_ready);
    uint8_t* my_vn = hh ? sVn1 : sVn0;
    bool ok = true;
    for (int n = 0; n < N && ok; ++n) {
      const int s = n & 1; const uint32_t ph = (n >> 1) & 1;
      const uint8_t* st = smem + s * STAGE;
      const float* gs = sG + (s * 2 + hh) * CH;
      {
        const bool got = mbar_wait(&bars->in_full[s], ph, abort_flag);
        if (!__all_sync(FULL, got)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
      }
      const float gl = gs[CH - 1];
      const uint8_t* xcol = st + F_X + (v >> 6) * (CH * 128) + (v & 7) * 2;
      const int xc16 = (v & 63) >> 3;
#pragma unroll
      for (int j8 = 0; j8 < 8; ++j8) {
        float vn[8], vd[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = j8 * 8 + jj;
          vn[jj] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(xcol + swz(j, xc16)));
          vd[jj] = vn[jj] * __expf(gl - gs[j]);
        }
        uint4 p0, p1;
        p0.x = pack_bf16(vn[0], vn[1]); p0.y = pack_bf16(vn[2], vn[3]); p0.z = pack_bf16(vn[4], vn[5]); p0.w = pack_bf16(vn[6], vn[7]);
        p1.x = pack_bf16(vd[0], vd[1]); p1.y = pack_bf16(vd[2], vd[3]); p1.z = pack_bf16(vd[4], vd[5]); p1.w = pack_bf16(vd[6], vd[7]);
        *reinterpret_cast<uint4*>(my_vn + swz(v, j8)) = p0;
        *reinterpret_cast<uint4*>(sVd + swz(v, j8)) = p1;
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->vn_ready);
      {
        const bool got = mbar_wait(&bars->out_full, n & 1, abort_flag);
        if (!__all_sync(FULL, got)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; break; }
      }
      tc_fence_after();
      // y^T row: out is [B, T, H, P] = [B, T, H / 2, 128] with this thread's column v of pair hp
      __nv_bfloat16* orow = out + ((static_cast<long long>(b) * T + n * CH) * Hp + hp) * 128 + v;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t o1[32], o2[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_O1 + half * 32, o1);
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_O2 + half * 32, o2);
        tmem_ld_wait();
#pragma unroll
        for (int ii = 0; ii < 32; ++ii) {
          const int i = half * 32 + ii;
          const float o = __expf(gs[i]) * __uint_as_float(o1[ii]) + __uint_as_float(o2[ii]);
          if (n * CH + i < T) orow[static_cast<long long>(i) * Hp * 128] = __float2bfloat16(o);
        }
      }
      const float dl = __expf(gl);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t d[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DS + q * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) S[q * 32 + i] = fmaf(S[q * 32 + i], dl, __uint_as_float(d[i]));
      }
      write_state_row(sState, v, S);
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&bars->s_ready); mbar_arrive(&bars->in_empty[s]); }
    }
    if (ok && final_state != nullptr) {
      float* dst = final_state + ((static_cast<long long>(b) * H + h0 + hh) * PD + (v & 63)) * ND;
#pragma unroll
      for (int d = 0; d < ND; d += 4) *reinterpret_cast<float4*>(dst + d) = make_float4(S[d], S[d + 1], S[d + 2], S[d + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

static int make_map4(CUtensorMap* m, const void* base, int B, int T, int H, int D, int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(H) * D * 2, static_cast<uint64_t>(T) * H * D * 2};
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return make_tmap_nd(m, base, 4, dims, strides, box, 2, true);
}

}  // namespace ssd
}  // namespace dewb

// xdt bf16 [B, T, H, 64] (x * dt), Bm / Cm bf16 [B, T, G, 128], P bf16 [B * H, Tp, 64] (per head, lower triangle of
// (C B^T) e^{g_i - g_j}), gc fp32 [B * H, Tp] (running sum of dt * A inside each chunk of 64; zero past T), all contiguous;
// H even, two consecutive heads in one group.  initial / final_state fp32 [B, H, 64, 128] (initial may be null);
// out bf16 [B, T, H, 64].
extern "C" int dewb_ssd_scan_fwd(const void* xdt, const void* Bm, const void* Cm, const void* P, const float* gc,
                                 const float* initial, void* out, float* final_state, int B, int T, int H, int G, int Tp,
                                 int* err, void* stream_ptr) {
  using namespace dewb::ssd;
  if (B <= 0 || T <= 0 || H <= 0 || (H & 1) || G <= 0 || H % G != 0 || ((H / G) & 1) || Tp % CH != 0 || Tp < T) return -3;
  const int N = (T + CH - 1) / CH;
  CUtensorMap tx, tc, tb, tp;
  int r;
  if ((r = make_map4(&tx, xdt, B, T, H / 2, 128, CH))) return 1000 + r;
  if ((r = make_map4(&tc, Cm, B, T, G, ND, CH))) return 2000 + r;
  if ((r = make_map4(&tb, Bm, B, T, G, ND, CH))) return 3000 + r;
  if ((r = dewb::make_tmap_2d(&tp, P, static_cast<uint64_t>(B) * H * Tp, CH, CH, CH, 64, 2, true))) return 4000 + r;
  cudaError_t e = cudaFuncSetAttribute(ssd_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  ssd_scan_fwd_kernel<<<B * (H / 2), THREADS, SMEM, reinterpret_cast<cudaStream_t>(stream_ptr)>>>(
      tx, tc, tb, tp, gc, initial, reinterpret_cast<__nv_bfloat16*>(out), final_state, T, H, G, Tp, N, err);
  return static_cast<int>(cudaGetLastError());
}
