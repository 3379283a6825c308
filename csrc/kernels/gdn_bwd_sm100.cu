// Gated delta rule, chunk-local part of the backward (chunk 64, 128-wide keys and values) for sm_100a.
//
// Once the two scans have left every chunk's entry state S0, exit-state gradient dS1, corrected values Vn and their
// gradient dVn in memory, the remaining gradients are local to a chunk.  With gc the cumulative log decay inside the
// chunk, D_ij = e^{gc_i - gc_j}, A = strict(beta_i (k_i . k_j) D_ij), W / U the solutions of (I + A) [W | U] =
// [beta e^gc K | beta V], P = scale (q_i . k_j) D_ij (lower triangle):
//
//   gdn_bwd_state_kernel  (one CTA per 128 tokens = two chunks; per chunk, rows of the accumulators = feature index)
//       X1^T  = S0 dO^T            -> dq_part = scale e^{gc} X1
//       dWn^T = S0 dVn^T           -> right-hand side -dWn of the transposed solve
//       dKd^T = dS1 Vn^T           -> dk_part = e^{g_L - gc} dKd + beta e^{gc} dKt
//       (I + A^T) [dKt | dVt] = [-dWn | dVn]   back substitution in fp32, one column per thread;  dv = beta dVt
//       and the per-token sums that feed d gc and d beta.
//   gdn_bwd_pair_kernel   (one CTA per 128 tokens; 128x128 products whose two 64x64 diagonal blocks are used)
//       dP = dO Vn^T,  dA = -(dKt W^T + dVt U^T),  K K^T again for A itself
//       Gt = scale dP o D (lower),  Bt = dA o (beta_i D_ij) (strictly lower)
//       dq = dq_part + Gt K ;  dk = dk_part + Gt^T Q + Bt K + Bt^T K   (computed transposed: rows = feature index)
//       d gc from the row and column sums of dP o P and dA o A, d g by the reverse running sum inside the chunk, d beta.
//
// Every wait is bounded (status word + abort flag, as in the other kernels of this library).
// Replaces the reference's ChunkBwdDvLocal / ChunkBwdDqkwg / PrepareWyReprBwd kernels (src/dew/nn/kernels/fla_gdn.py:650-1080).
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace dewb {
namespace gdnb {

constexpr int HD = 128;
constexpr int CH = 64;
constexpr int PT = 128;
constexpr uint32_t FULL = 0xffffffffu;
constexpr int THREADS = 256;
constexpr int T32 = PT * HD * 2;     // [128 x 128] bf16 tile: two 64-column sub-tiles of 16 KiB
constexpr int T16 = CH * HD * 2;     // [64 x 128] bf16 tile: two 64-column sub-tiles of 8 KiB

__device__ __forceinline__ uint32_t swz(int r, int c16) { return static_cast<uint32_t>(r * 128 + ((c16 ^ (r & 7)) << 4)); }

// bf16 element (row r, column c) of a tile stored as 64-column sub-tiles of `rows` rows (128-byte swizzle)
__device__ __forceinline__ float tile_get(const uint8_t* tile, int rows, int r, int c) {
  const uint8_t* p = tile + (c >> 6) * (rows * 128) + swz(r, (c & 63) >> 3) + (c & 7) * 2;
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
}
__device__ __forceinline__ void tile_put(uint8_t* tile, int rows, int r, int c, float v) {
  uint8_t* p = tile + (c >> 6) * (rows * 128) + swz(r, (c & 63) >> 3) + (c & 7) * 2;
  *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}

// v[k] holds this lane's term for token k (32 tokens); on return lane l holds the sum over the warp of token l's terms.
// 31 shuffles for 32 sums (a butterfly that halves the token set at every step) instead of 5 per sum.
__device__ __forceinline__ float reduce_scatter32(float (&v)[32], int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int k = 0; k < o; ++k) {
      const float send = upper ? v[k] : v[k + o];
      const float keep = upper ? v[k + o] : v[k];
      v[k] = keep + __shfl_xor_sync(FULL, send, o);
    }
  }
  return v[0];
}

struct Tail {
  float g[PT], beta[PT], eg[PT];
  // state kernel: per-token sums over the feature index.  Each of the four warps that share a token keeps its own slot and
  // the reader adds the slots in a fixed order, so the gradients of g and beta are bitwise repeatable (no shared atomics).
  float sum_q[4][PT], sum_k[4][PT], sum_kd[4][PT], sum_v[4][PT];
  float dss[2][4];                                           // <dS1, S0> per chunk, one slot per warp
  float red[8];
  uint64_t bar[6];
  uint32_t tmem_base;
  int poisoned, abort_flag;
};

// ------------------------------------------------------------------------------------------------------------------
// state kernel

constexpr int S_OFF_K = 0, S_OFF_S = T32, S_OFF_G = 2 * T32, S_OFF_DO = 3 * T32, S_OFF_DVN = 3 * T32 + T16,
              S_OFF_VN = 3 * T32 + 2 * T16, S_OFF_V = 3 * T32 + 3 * T16, S_OFF_Q = 3 * T32 + 4 * T16,
              S_OFF_AT = 3 * T32 + 5 * T16, S_OFF_TAIL = S_OFF_AT + 2 * CH * CH * 4;
constexpr int TAIL_BYTES = 10240;
constexpr int STATE_SMEM = S_OFF_TAIL + TAIL_BYTES;
static_assert(sizeof(Tail) <= TAIL_BYTES, "Tail must fit its slot");
static_assert(STATE_SMEM <= 232448, "state kernel exceeds the shared memory of an SM");

__global__ void __launch_bounds__(THREADS, 1)
gdn_bwd_state_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tq,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const __grid_constant__ CUtensorMap tvn, const __grid_constant__ CUtensorMap tdvn,
                     const __grid_constant__ CUtensorMap tst, const __grid_constant__ CUtensorMap tds,
                     const float* __restrict__ gc, const float* __restrict__ beta, __nv_bfloat16* __restrict__ dKt,
                     __nv_bfloat16* __restrict__ dVt, __nv_bfloat16* __restrict__ dv, float* __restrict__ dq_part,
                     float* __restrict__ dk_part, float* __restrict__ gpart, float* __restrict__ bpart, int T, int H, int rep,
                     int Tp, int N, float scale, int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    return;
  }
  Tail* tail = reinterpret_cast<Tail*>(smem + S_OFF_TAIL);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) tail->poisoned = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (tail->poisoned != 0) return;
  const int x = blockIdx.y, b = x / H, h = x % H;
  const int t0 = blockIdx.x * PT;
  uint8_t* sK = smem + S_OFF_K;
  uint8_t* sS = smem + S_OFF_S;
  uint8_t* sG = smem + S_OFF_G;
  uint8_t* sdO = smem + S_OFF_DO;
  uint8_t* sdVn = smem + S_OFF_DVN;
  uint8_t* sVn = smem + S_OFF_VN;
  uint8_t* sV = smem + S_OFF_V;
  uint8_t* sQ = smem + S_OFF_Q;
  float* sAT = reinterpret_cast<float*>(smem + S_OFF_AT);
  uint64_t* bar_k = &tail->bar[0];
  uint64_t* bar_kk = &tail->bar[1];
  uint64_t* bar_in = &tail->bar[2];
  uint64_t* bar_mma = &tail->bar[3];
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(&tail->bar[i], 1);
    tail->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) { tmem_alloc(&tail->tmem_base, 512); tmem_relinquish(); }
  if (tid < PT) {
    const int t = t0 + tid;
    const float gi = gc[static_cast<long long>(x) * Tp + t];
    tail->g[tid] = gi;
    tail->eg[tid] = __expf(gi);
    tail->beta[tid] = t < T ? beta[(static_cast<long long>(b) * T + t) * H + h] : 0.f;
#pragma unroll
    for (int w4 = 0; w4 < 4; ++w4) { tail->sum_q[w4][tid] = 0.f; tail->sum_k[w4][tid] = 0.f; tail->sum_kd[w4][tid] = 0.f; tail->sum_v[w4][tid] = 0.f; }
  }
  if (tid < 8) tail->dss[tid >> 2][tid & 3] = 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  constexpr int TM_KK = 0, TM_X1 = 128, TM_DW = 192, TM_DKD = 256;

  if (tid == 0) {
    mbar_expect_tx(bar_k, T32);
    tma_load_4d(sK, &tk, bar_k, 0, h / rep, t0, b);                       // `rep` value heads share a key head
    tma_load_4d(sK + PT * 128, &tk, bar_k, 64, h / rep, t0, b);
    if (!mbar_wait(bar_k, 0, abort_flag)) atomicCAS(err, 0, ERR_WAIT_FULL);
    else {
      tc_fence_after();
      constexpr uint32_t idesc = make_idesc(128, 128, 1, 1, 0, 0);
      const uint32_t ka = smem_u32(sK);
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
        umma_bf16_ss(tmem + TM_KK, make_sdesc_sw128(ka + off, 16, 1024), make_sdesc_sw128(ka + off, 16, 1024), idesc, kk > 0 ? 1u : 0u);
      }
      umma_commit(bar_kk);
    }
  }
  if (warp == 0) __syncwarp();      // the issuing thread's warp-mates park here instead of spinning beside it
  if (warp < 4) {
    // token row i: A[i][j] = beta_i (k_i . k_j) e^{g_i - g_j} (j < i), stored transposed: sAT[c][j][i], each row of the
    // transpose rotated by four floats per row so that the solve's broadcast float4 reads stay aligned and these
    // column-wise stores stay free of bank conflicts
    const int i = tid, c = i >> 6, il = i & 63;
    const bool got = mbar_wait(bar_kk, 0, abort_flag);
    if (__all_sync(FULL, got)) {
      tc_fence_after();
      uint32_t v0[32], v1[32];
      const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
      tmem_ld_32x32b_x32(tmem + lane_addr + TM_KK + c * 64, v0);
      tmem_ld_32x32b_x32(tmem + lane_addr + TM_KK + c * 64 + 32, v1);
      tmem_ld_wait();
      const float gi = tail->g[i], bi = tail->beta[i];
      float* at = sAT + c * (CH * CH);
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const float s = __uint_as_float(j < 32 ? v0[j & 31] : v1[j & 31]);
        const float a = (j < il) ? bi * s * __expf(gi - tail->g[c * 64 + j]) : 0.f;
        at[j * CH + ((il + 4 * j) & 63)] = a;
      }
      tc_fence_before();
    } else if (lane == 0) {
      atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
    }
  }
  __syncthreads();

  for (int c = 0; c < 2; ++c) {
    const int n = blockIdx.x * 2 + c;
    if (n >= N || tail->abort_flag != 0) break;
    if (tid == 0) {
      mbar_expect_tx(bar_in, 2 * T32 + 5 * T16);
      const int srow = (x * N + n) * HD;
      const int trow = x * Tp + n * CH;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        tma_load_2d(sS + s * (PT * 128), &tst, bar_in, s * 64, srow);
        tma_load_2d(sG + s * (PT * 128), &tds, bar_in, s * 64, srow);
        tma_load_4d(sdO + s * (CH * 128), &tdo, bar_in, s * 64, h, n * CH, b);
        tma_load_2d(sdVn + s * (CH * 128), &tdvn, bar_in, s * 64, trow);
        tma_load_2d(sVn + s * (CH * 128), &tvn, bar_in, s * 64, trow);
        tma_load_4d(sV + s * (CH * 128), &tv, bar_in, s * 64, h, n * CH, b);
        tma_load_4d(sQ + s * (CH * 128), &tq, bar_in, s * 64, h / rep, n * CH, b);
      }
      if (!mbar_wait(bar_in, c & 1, abort_flag)) atomicCAS(err, 0, ERR_WAIT_FULL);
      else {
        tc_fence_after();
        // S0 is stored transposed ([value][key]): as the A operand [M = key, K = value] it is MN-major
        constexpr uint32_t idesc_s = make_idesc(128, 64, 1, 1, 1, 0);
        constexpr uint32_t idesc_g = make_idesc(128, 64, 1, 1, 0, 0);
        const uint32_t sa = smem_u32(sS), ga = smem_u32(sG), doa = smem_u32(sdO), dvna = smem_u32(sdVn), vna = smem_u32(sVn);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t boff = (kk >> 2) * (CH * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem + TM_X1, make_sdesc_sw128(sa + kk * 2048, PT * 128, 1024), make_sdesc_sw128(doa + boff, 16, 1024),
                       idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t boff = (kk >> 2) * (CH * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem + TM_DW, make_sdesc_sw128(sa + kk * 2048, PT * 128, 1024), make_sdesc_sw128(dvna + boff, 16, 1024),
                       idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (PT * 128) + (kk & 3) * 32, boff = (kk >> 2) * (CH * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem + TM_DKD, make_sdesc_sw128(ga + aoff, 16, 1024), make_sdesc_sw128(vna + boff, 16, 1024),
                       idesc_g, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar_mma);
      }
    }
    if (warp == 0) __syncwarp();
    // everybody: the tiles have landed (the per-thread wait gives the acquire) and the products are complete
    bool ok = mbar_wait(bar_in, c & 1, abort_flag);
    ok = mbar_wait(bar_mma, c & 1, abort_flag) && ok;
    ok = __all_sync(FULL, ok);
    if (!ok && lane == 0) atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const float* at = sAT + c * (CH * CH);
      const int f = tid & 127;                             // feature index: key index (threads 0..127) or value index
      const long long trow = static_cast<long long>(x) * Tp + n * CH;
      float xs[CH];
      if (tid < 128) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DW, v0);
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DW + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; ++j) xs[j] = -__uint_as_float(j < 32 ? v0[j & 31] : v1[j & 31]);
      } else {
#pragma unroll
        for (int j = 0; j < CH; ++j) xs[j] = tile_get(sdVn, CH, j, f);
      }
      // back substitution: x_i = r_i - sum_{j > i} A[j][i] x_j  (xs holds r, then x)
#pragma unroll
      for (int i = CH - 2; i >= 0; --i) {
        float acc = xs[i], acc1 = 0.f;                     // two chains: half the dependent latency per row
        const float4* arow = reinterpret_cast<const float4*>(at + i * CH);
#pragma unroll
        for (int j4 = (i + 1) >> 2; j4 < 16; ++j4) {
          const float4 av = arow[(j4 + i) & 15];
          if (j4 * 4 + 0 > i) acc = fmaf(-av.x, xs[j4 * 4 + 0], acc);
          if (j4 * 4 + 1 > i) acc1 = fmaf(-av.y, xs[j4 * 4 + 1], acc1);
          if (j4 * 4 + 2 > i) acc = fmaf(-av.z, xs[j4 * 4 + 2], acc);
          if (j4 * 4 + 3 > i) acc1 = fmaf(-av.w, xs[j4 * 4 + 3], acc1);
        }
        xs[i] = acc + acc1;
      }
      if (tid < 128) {
        // dKt column; dk_part = e^{g_L - g} dKd + beta e^g dKt; sums over the key index
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DKD, v0);
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DKD + 32, v1);
        tmem_ld_wait();
        const float gl = tail->g[c * 64 + 63];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float p1[32], p2[32];
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int j = half * 32 + jj, r = c * 64 + j;
            const float kv = tile_get(sK, PT, r, f);
            const float dkd = __expf(gl - tail->g[r]) * __uint_as_float(half == 0 ? v0[jj] : v1[jj]);
            dKt[(trow + j) * HD + f] = __float2bfloat16(xs[j]);
            const int t = n * CH + j;
            if (t < T) dk_part[((static_cast<long long>(b) * T + t) * H + h) * HD + f] = dkd + tail->beta[r] * tail->eg[r] * xs[j];
            p1[jj] = xs[j] * kv;
            p2[jj] = dkd * kv;
          }
          const float s1 = reduce_scatter32(p1, lane), s2 = reduce_scatter32(p2, lane);
          tail->sum_k[warp & 3][c * 64 + half * 32 + lane] = s1;
          tail->sum_kd[warp & 3][c * 64 + half * 32 + lane] = s2;
        }
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_X1, v0);
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_X1 + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float p1[32];
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int j = half * 32 + jj, r = c * 64 + j;
            const float dq1 = scale * tail->eg[r] * __uint_as_float(half == 0 ? v0[jj] : v1[jj]);
            const int t = n * CH + j;
            if (t < T) dq_part[((static_cast<long long>(b) * T + t) * H + h) * HD + f] = dq1;
            p1[jj] = dq1 * tile_get(sQ, CH, j, f);
          }
          const float s = reduce_scatter32(p1, lane);
          tail->sum_q[warp & 3][c * 64 + half * 32 + lane] = s;
        }
        // <dS1, S0>: row f of dS1 against column f of the transposed state tile
        float acc = 0.f;
#pragma unroll 8
        for (int v = 0; v < HD; ++v) acc = fmaf(tile_get(sG, PT, f, v), tile_get(sS, PT, v, f), acc);
        acc = warp_sum(acc);
        if (lane == 0) tail->dss[c][warp & 3] = acc;
      } else {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float p1[32];
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int j = half * 32 + jj, r = c * 64 + j;
            dVt[(trow + j) * HD + f] = __float2bfloat16(xs[j]);
            const int t = n * CH + j;
            if (t < T) dv[((static_cast<long long>(b) * T + t) * H + h) * HD + f] = __float2bfloat16(tail->beta[r] * xs[j]);
            p1[jj] = xs[j] * tile_get(sV, CH, j, f);
          }
          const float s = reduce_scatter32(p1, lane);
          tail->sum_v[warp & 3][c * 64 + half * 32 + lane] = s;
        }
      }
      tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
  }
  // per-token partial gradients of gc and beta
  if (tid < PT && tail->abort_flag == 0) {
    const int i = tid, c = i >> 6;
    auto four = [](const float (*a)[PT], int j) { return (a[0][j] + a[1][j]) + (a[2][j] + a[3][j]); };
    const float sq = four(tail->sum_q, i), sk = four(tail->sum_k, i), skd = four(tail->sum_kd, i), sv = four(tail->sum_v, i);
    float dg = sq - skd + tail->beta[i] * tail->eg[i] * sk;
    if ((i & 63) == 63) {
      float tot = 0.f;
      for (int j = 0; j < CH; ++j) tot += four(tail->sum_kd, c * 64 + j);
      dg += tot + tail->eg[i] * ((tail->dss[c][0] + tail->dss[c][1]) + (tail->dss[c][2] + tail->dss[c][3]));
    }
    gpart[static_cast<long long>(x) * Tp + t0 + i] = dg;
    bpart[static_cast<long long>(x) * Tp + t0 + i] = sv + tail->eg[i] * sk;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// pair kernel

constexpr int P_OFF_TAIL = 5 * T32;
constexpr int PAIR_SMEM = P_OFF_TAIL + TAIL_BYTES;

__global__ void __launch_bounds__(THREADS, 1)
gdn_bwd_pair_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tq,
                    const __grid_constant__ CUtensorMap tdo, const __grid_constant__ CUtensorMap tvn,
                    const __grid_constant__ CUtensorMap tdkt, const __grid_constant__ CUtensorMap tdvt,
                    const __grid_constant__ CUtensorMap tw, const __grid_constant__ CUtensorMap tu,
                    const float* __restrict__ gc, const float* __restrict__ beta, const __nv_bfloat16* __restrict__ P,
                    const float* __restrict__ dq_part, const float* __restrict__ dk_part, const float* __restrict__ gpart,
                    const float* __restrict__ bpart, __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk,
                    float* __restrict__ dg, float* __restrict__ dbeta, int T, int H, int rep, int Tp, float scale,
                    int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    return;
  }
  Tail* tail = reinterpret_cast<Tail*>(smem + P_OFF_TAIL);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) tail->poisoned = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (tail->poisoned != 0) return;
  const int x = blockIdx.y, b = x / H, h = x % H;
  const int t0 = blockIdx.x * PT;
  uint8_t* b0 = smem;              // K
  uint8_t* b1 = smem + T32;        // dO, then dVt, then Bt
  uint8_t* b2 = smem + 2 * T32;    // Vn, then U, then the fp32 matrix dP o P + dA o A
  uint8_t* b3 = smem + 3 * T32;    // dKt, then Q
  uint8_t* b4 = smem + 4 * T32;    // W, then Gt
  uint64_t* bar_a = &tail->bar[0];   // K, dO, Vn, dKt, W landed
  uint64_t* bar_x = &tail->bar[1];   // K K^T, dO Vn^T, dKt W^T complete
  uint64_t* bar_b = &tail->bar[2];   // dVt, U, Q landed
  uint64_t* bar_y = &tail->bar[3];   // dVt U^T complete
  uint64_t* bar_z = &tail->bar[4];   // final products complete
  if (tid == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&tail->bar[i], 1);
    tail->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) { tmem_alloc(&tail->tmem_base, 512); tmem_relinquish(); }
  if (tid < PT) {
    const int t = t0 + tid;
    const float gi = gc[static_cast<long long>(x) * Tp + t];
    tail->g[tid] = gi;
    tail->eg[tid] = __expf(gi);
    tail->beta[tid] = t < T ? beta[(static_cast<long long>(b) * T + t) * H + h] : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  constexpr int TM_KK = 0, TM_DP = 128, TM_DA = 256;     // later: TM_KK -> dq2^T, TM_DP -> dk2^T
  const int prow = x * Tp + t0;                          // row of the pair in the [X * Tp, .] intermediates
  constexpr uint32_t idesc_kk = make_idesc(128, 128, 1, 1, 0, 0);

  if (tid == 0) {
    mbar_expect_tx(bar_a, 5 * T32);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      tma_load_4d(b0 + s * (PT * 128), &tk, bar_a, s * 64, h / rep, t0, b);
      tma_load_4d(b1 + s * (PT * 128), &tdo, bar_a, s * 64, h, t0, b);
      tma_load_2d(b2 + s * (PT * 128), &tvn, bar_a, s * 64, prow);
      tma_load_2d(b3 + s * (PT * 128), &tdkt, bar_a, s * 64, prow);
      tma_load_2d(b4 + s * (PT * 128), &tw, bar_a, s * 64, prow);
    }
    bool ok = mbar_wait(bar_a, 0, abort_flag);
    if (!ok) atomicCAS(err, 0, ERR_WAIT_FULL);
    if (ok) {
      tc_fence_after();
      const uint32_t a0 = smem_u32(b0), a1 = smem_u32(b1), a2 = smem_u32(b2), a3 = smem_u32(b3), a4 = smem_u32(b4);
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
        umma_bf16_ss(tmem + TM_KK, make_sdesc_sw128(a0 + off, 16, 1024), make_sdesc_sw128(a0 + off, 16, 1024), idesc_kk, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
        umma_bf16_ss(tmem + TM_DP, make_sdesc_sw128(a1 + off, 16, 1024), make_sdesc_sw128(a2 + off, 16, 1024), idesc_kk, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
        umma_bf16_ss(tmem + TM_DA, make_sdesc_sw128(a3 + off, 16, 1024), make_sdesc_sw128(a4 + off, 16, 1024), idesc_kk, kk > 0 ? 1u : 0u);
      }
      umma_commit(bar_x);
      ok = mbar_wait(bar_x, 0, abort_flag);
      if (!ok) atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
    }
    if (ok) {
      // dO, Vn, dKt are consumed: their space takes dVt, U, Q
      mbar_expect_tx(bar_b, 3 * T32);
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        tma_load_2d(b1 + s * (PT * 128), &tdvt, bar_b, s * 64, prow);
        tma_load_2d(b2 + s * (PT * 128), &tu, bar_b, s * 64, prow);
        tma_load_4d(b3 + s * (PT * 128), &tq, bar_b, s * 64, h / rep, t0, b);
      }
      ok = mbar_wait(bar_b, 0, abort_flag);
      if (!ok) atomicCAS(err, 0, ERR_WAIT_FULL);
    }
    if (ok) {
      tc_fence_after();
      const uint32_t a1 = smem_u32(b1), a2 = smem_u32(b2);
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
        umma_bf16_ss(tmem + TM_DA, make_sdesc_sw128(a1 + off, 16, 1024), make_sdesc_sw128(a2 + off, 16, 1024), idesc_kk, 1u);
      }
      umma_commit(bar_y);
    }
  }
  if (warp == 0) __syncwarp();
  float row_gp = 0.f, row_e = 0.f, row_b = 0.f;
  if (warp < 4) {
    // token row i: its chunk's 64 columns of K K^T, dP and dA -> the Gt and Bt operand tiles and the decay / strength sums
    const int i = tid, c = i >> 6, il = i & 63;
    // this row of P (64 bf16) is fetched before the waits so that its latency hides behind the products
    uint4 pv8[8];
    {
      const uint4* pr = reinterpret_cast<const uint4*>(P + (static_cast<long long>(prow) + i) * CH);
#pragma unroll
      for (int u = 0; u < 8; ++u) pv8[u] = __ldg(pr + u);
    }
    bool ok = mbar_wait(bar_y, 0, abort_flag);
    ok = mbar_wait(bar_b, 0, abort_flag) && ok;
    ok = __all_sync(FULL, ok);
    if (!ok && lane == 0) atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
      const float gi = tail->g[i], bi = tail->beta[i];
      uint8_t* gt_row = b4 + c * (PT * 128);        // Gt[i][j]: column block c (64 columns) is sub-tile c
      uint8_t* bt_row = b1 + c * (PT * 128);
      const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
      // the other chunk's column block of this row is zero
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        *reinterpret_cast<uint4*>(b4 + (c ^ 1) * (PT * 128) + swz(i, c16)) = zero4;
        *reinterpret_cast<uint4*>(b1 + (c ^ 1) * (PT * 128) + swz(i, c16)) = zero4;
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t kk[32], dp[32], da[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_KK + c * 64 + half * 32, kk);
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DP + c * 64 + half * 32, dp);
        tmem_ld_32x32b_x32(tmem + lane_addr + TM_DA + c * 64 + half * 32, da);
        tmem_ld_wait();
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const uint4 pv = pv8[half * 4 + j8];
          const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
          float gt[8], bt[8], mrow[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const int j = half * 32 + j8 * 8 + jj;
            const float dcy = (j <= il) ? __expf(gi - tail->g[c * 64 + j]) : 0.f;
            const float dpr = (j <= il) ? __uint_as_float(dp[j8 * 8 + jj]) : 0.f;
            const float pj = (jj & 1) ? bf16_hi(pw[jj >> 1]) : bf16_lo(pw[jj >> 1]);
            gt[jj] = scale * dpr * dcy;
            const float gp = dpr * pj;
            const float dav = (j < il) ? -__uint_as_float(da[j8 * 8 + jj]) : 0.f;
            const float kkd = (j < il) ? __uint_as_float(kk[j8 * 8 + jj]) * dcy : 0.f;
            bt[jj] = dav * bi * dcy;
            const float e = dav * bi * kkd;
            row_gp += gp; row_e += e; row_b += dav * kkd;
            mrow[jj] = gp + e;
          }
          // dP o P + dA o A of this row, kept for the column sums (rows rotated by one float4 per row: no bank conflicts
          // for these stores nor for the column reads below)
          float4* mr = reinterpret_cast<float4*>(b2) + (c * CH + il) * 16;
          mr[(half * 8 + j8 * 2 + il) & 15] = make_float4(mrow[0], mrow[1], mrow[2], mrow[3]);
          mr[(half * 8 + j8 * 2 + 1 + il) & 15] = make_float4(mrow[4], mrow[5], mrow[6], mrow[7]);
          uint4 g4, b4v;
          g4.x = pack_bf16(gt[0], gt[1]); g4.y = pack_bf16(gt[2], gt[3]); g4.z = pack_bf16(gt[4], gt[5]); g4.w = pack_bf16(gt[6], gt[7]);
          b4v.x = pack_bf16(bt[0], bt[1]); b4v.y = pack_bf16(bt[2], bt[3]); b4v.z = pack_bf16(bt[4], bt[5]); b4v.w = pack_bf16(bt[6], bt[7]);
          *reinterpret_cast<uint4*>(gt_row + swz(i, half * 4 + j8)) = g4;
          *reinterpret_cast<uint4*>(bt_row + swz(i, half * 4 + j8)) = b4v;
        }
      }
      fence_proxy_async();
      tc_fence_before();
    }
  }
  __syncthreads();
  if (tid == 0 && tail->abort_flag == 0) {
    tc_fence_after();
    // transposed products (rows = key feature index, columns = the 128 tokens of the pair):
    //   dq2^T = K^T Gt^T                          -> TM_KK
    //   dk2^T = Q^T Gt + K^T Bt^T + K^T Bt        -> TM_DP
    // K and Q in their natural [token][feature] layout are MN-major A operands; Gt / Bt natural are K-major B operands
    // for the "^T" forms and MN-major B operands otherwise.
    constexpr uint32_t idesc_nk = make_idesc(128, 128, 1, 1, 1, 0);
    constexpr uint32_t idesc_nn = make_idesc(128, 128, 1, 1, 1, 1);
    const uint32_t ka = smem_u32(b0), qa = smem_u32(b3), gta = smem_u32(b4), bta = smem_u32(b1);
#pragma unroll
    for (int kk = 0; kk < PT / 16; ++kk) {
      const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
      umma_bf16_ss(tmem + TM_KK, make_sdesc_sw128(ka + kk * 2048, PT * 128, 1024), make_sdesc_sw128(gta + off, 16, 1024), idesc_nk, kk > 0 ? 1u : 0u);
    }
#pragma unroll
    for (int kk = 0; kk < PT / 16; ++kk) {
      umma_bf16_ss(tmem + TM_DP, make_sdesc_sw128(qa + kk * 2048, PT * 128, 1024), make_sdesc_sw128(gta + kk * 2048, PT * 128, 1024), idesc_nn, kk > 0 ? 1u : 0u);
    }
#pragma unroll
    for (int kk = 0; kk < PT / 16; ++kk) {
      const uint32_t off = (kk >> 2) * (PT * 128) + (kk & 3) * 32;
      umma_bf16_ss(tmem + TM_DP, make_sdesc_sw128(ka + kk * 2048, PT * 128, 1024), make_sdesc_sw128(bta + off, 16, 1024), idesc_nk, 1u);
    }
#pragma unroll
    for (int kk = 0; kk < PT / 16; ++kk) {
      umma_bf16_ss(tmem + TM_DP, make_sdesc_sw128(ka + kk * 2048, PT * 128, 1024), make_sdesc_sw128(bta + kk * 2048, PT * 128, 1024), idesc_nn, 1u);
    }
    umma_commit(bar_z);
  }
  if (warp < 4 && tail->abort_flag == 0) {
    // d gc of token i, then d g by the reverse running sum inside the chunk; d beta
    const int i = tid;
    float col = 0.f;
    {
      // column (i & 63) of this chunk's 64 x 64 block of dP o P + dA o A
      const float* m = reinterpret_cast<const float*>(b2) + (i >> 6) * (CH * CH);
      const int j = i & 63;
#pragma unroll 8
      for (int r = 0; r < CH; ++r) col += m[r * CH + ((j + 4 * r) & 63)];
    }
    float dgc = gpart[static_cast<long long>(prow) + i] + row_gp + row_e - col;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float dn = __shfl_down_sync(FULL, dgc, d);
      if (lane + d < 32) dgc += dn;
    }
    if (lane == 0) tail->red[warp] = dgc;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if ((warp & 1) == 0) dgc += tail->red[warp + 1];
    const int t = t0 + i;
    if (t < T) {
      dg[(static_cast<long long>(b) * T + t) * H + h] = dgc;
      dbeta[(static_cast<long long>(b) * T + t) * H + h] = bpart[static_cast<long long>(prow) + i] + row_b;
    }
  }
  // epilogue: rows = key feature index (threads 0..127), columns = tokens
  bool okz = mbar_wait(bar_z, 0, abort_flag);
  okz = __all_sync(FULL, okz);
  if (warp < 4 && okz) {
    tc_fence_after();
    const int f = tid;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      uint32_t a[32], c2[32];
      // all 64 loads of the partial sums are in flight before the first of them is used
      float pq[32], pk[32];
#pragma unroll
      for (int ii = 0; ii < 32; ++ii) {
        const int t = min(t0 + q4 * 32 + ii, T - 1);
        const long long o = ((static_cast<long long>(b) * T + t) * H + h) * HD + f;
        pq[ii] = __ldg(dq_part + o);
        pk[ii] = __ldg(dk_part + o);
      }
      tmem_ld_32x32b_x32(tmem + lane_addr + TM_KK + q4 * 32, a);
      tmem_ld_32x32b_x32(tmem + lane_addr + TM_DP + q4 * 32, c2);
      tmem_ld_wait();
#pragma unroll
      for (int ii = 0; ii < 32; ++ii) {
        const int t = t0 + q4 * 32 + ii;
        if (t < T) {
          const long long o = ((static_cast<long long>(b) * T + t) * H + h) * HD + f;
          dq[o] = __float2bfloat16(pq[ii] + __uint_as_float(a[ii]));
          dk[o] = __float2bfloat16(pk[ii] + __uint_as_float(c2[ii]));
        }
      }
    }
  } else if (warp < 4 && lane == 0) {
    atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

static int make_bthd_map(CUtensorMap* m, const void* base, int B, int T, int H, long long sb, long long st, long long sh,
                         int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(H), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(st) * 2, static_cast<uint64_t>(sb) * 2};
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return make_tmap_nd(m, base, 4, dims, strides, box, 2, true);
}

}  // namespace gdnb
}  // namespace dewb

// q, k: bf16 [B, T, H / rep, 128], v, d_out: bf16 [B, T, H, 128], contiguous (`rep` value heads share one key head; dq and dk come
// back per value head and the caller sums each group of `rep`).  With X = B * H, N = ceil(T / 64), Tp = T rounded up to 128:
// vn, dvn, W, U bf16 [X, Tp, 128]; P bf16 [X, Tp, 64]; gc fp32 [X, Tp]; beta fp32 [B, T, H];
// states bf16 [X, N, 128 (value), 128 (key)]; dstates bf16 [X, N, 128 (key), 128 (value)].
// Scratch (caller-allocated): dKt, dVt bf16 [X, Tp, 128]; dq_part, dk_part fp32 [B, T, H, 128]; gpart, bpart fp32 [X, Tp].
// Outputs: dq, dk, dv bf16 [B, T, H, 128]; dg, dbeta fp32 [B, T, H].
extern "C" int dewb_gdn_bwd_local(const void* q, const void* k, const void* v, const void* d_out, const void* vn,
                                  const void* dvn, const void* W, const void* U, const void* P, const float* gc,
                                  const float* beta, const void* states, const void* dstates, void* dKt, void* dVt,
                                  float* dq_part, float* dk_part, float* gpart, float* bpart, void* dq, void* dk, void* dv,
                                  float* dg, float* dbeta, int B, int T, int H, int rep, int Tp, float scale, int* err,
                                  void* stream_ptr) {
  using namespace dewb::gdnb;
  using bf = __nv_bfloat16;
  if (B <= 0 || T <= 0 || H <= 0 || Tp % PT != 0 || Tp < T || rep <= 0 || H % rep != 0) return -3;
  const int N = (T + CH - 1) / CH;
  const int X = B * H;
  const int Hk = H / rep;
  const long long sb = static_cast<long long>(T) * H * HD, st = static_cast<long long>(H) * HD, sh = HD;
  const long long sbk = static_cast<long long>(T) * Hk * HD, stk = static_cast<long long>(Hk) * HD;
  const uint64_t rows = static_cast<uint64_t>(X) * Tp, srows = static_cast<uint64_t>(X) * N * HD;
  CUtensorMap tq64, tv64, tdo64, tk128, tq128, tdo128, tvn64, tdvn64, tvn128, tst, tds, tdkt, tdvt, tw, tu;
  int r;
  if ((r = make_bthd_map(&tk128, k, B, T, Hk, sbk, stk, sh, PT))) return 1000 + r;
  if ((r = make_bthd_map(&tq128, q, B, T, Hk, sbk, stk, sh, PT))) return 1100 + r;
  if ((r = make_bthd_map(&tdo128, d_out, B, T, H, sb, st, sh, PT))) return 1200 + r;
  if ((r = make_bthd_map(&tq64, q, B, T, Hk, sbk, stk, sh, CH))) return 1300 + r;
  if ((r = make_bthd_map(&tv64, v, B, T, H, sb, st, sh, CH))) return 1400 + r;
  if ((r = make_bthd_map(&tdo64, d_out, B, T, H, sb, st, sh, CH))) return 1500 + r;
  if ((r = dewb::make_tmap_2d(&tvn64, vn, rows, HD, HD, CH, 64, 2, true))) return 2000 + r;
  if ((r = dewb::make_tmap_2d(&tdvn64, dvn, rows, HD, HD, CH, 64, 2, true))) return 2100 + r;
  if ((r = dewb::make_tmap_2d(&tvn128, vn, rows, HD, HD, PT, 64, 2, true))) return 2200 + r;
  if ((r = dewb::make_tmap_2d(&tst, states, srows, HD, HD, PT, 64, 2, true))) return 2300 + r;
  if ((r = dewb::make_tmap_2d(&tds, dstates, srows, HD, HD, PT, 64, 2, true))) return 2400 + r;
  if ((r = dewb::make_tmap_2d(&tdkt, dKt, rows, HD, HD, PT, 64, 2, true))) return 2500 + r;
  if ((r = dewb::make_tmap_2d(&tdvt, dVt, rows, HD, HD, PT, 64, 2, true))) return 2600 + r;
  if ((r = dewb::make_tmap_2d(&tw, W, rows, HD, HD, PT, 64, 2, true))) return 2700 + r;
  if ((r = dewb::make_tmap_2d(&tu, U, rows, HD, HD, PT, 64, 2, true))) return 2800 + r;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  cudaError_t e = cudaFuncSetAttribute(gdn_bwd_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STATE_SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaFuncSetAttribute(gdn_bwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(Tp / PT, X);
  gdn_bwd_state_kernel<<<grid, THREADS, STATE_SMEM, stream>>>(
      tk128, tq64, tv64, tdo64, tvn64, tdvn64, tst, tds, gc, beta, reinterpret_cast<bf*>(dKt), reinterpret_cast<bf*>(dVt),
      reinterpret_cast<bf*>(dv), dq_part, dk_part, gpart, bpart, T, H, rep, Tp, N, scale, err);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  gdn_bwd_pair_kernel<<<grid, THREADS, PAIR_SMEM, stream>>>(
      tk128, tq128, tdo128, tvn128, tdkt, tdvt, tw, tu, gc, beta, reinterpret_cast<const bf*>(P), dq_part, dk_part, gpart,
      bpart, reinterpret_cast<bf*>(dq), reinterpret_cast<bf*>(dk), dg, dbeta, T, H, rep, Tp, scale, err);
  return static_cast<int>(cudaGetLastError());
}
