// Flash attention backward for sm_100a (head_dim 128 or 64, bf16, causal or full, GQA), in three kernels:
//
//   delta   : delta[b,h,s] = sum_d dO * O                                   (row kernel)
//   dQ      : one CTA per 128 query rows; loops over key tiles:
//                S = Q K^T, dP = dO V^T (tcgen05, TMEM) -> dS = P o (dP - delta) (bf16, written over S in TMEM) -> dQ += dS K
//   dK / dV : one CTA per 128 keys of one KV head; loops over the query heads of its group and 64-row query blocks:
//                S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T (bf16, written over S^T / dP^T in TMEM) -> dV += P^T dO, dK += dS^T Q
// Both MMA kernels recompute the probabilities from the saved log-sum-exp, keep their output accumulators in tensor
// memory for the whole loop and never use atomics, so results are deterministic. A Q / dO / K / V tile sits in shared
// memory once and serves two products through two descriptors (K-major for the score products, MN-major for the
// gradient products). The gradient products read their A operand (P^T, dS^T, dS) from tensor memory, where the softmax
// threads leave it with tcgen05.st: with both operands in shared memory the operand fetch (about 95 bytes per cycle
// measured against 128 needed), not the tensor pipe, set the pace. The exponentials, not the tensor core, bound both MMA kernels, so each runs eight softmax warps:
// two threads per TMEM lane, each taking half of the tile's columns (no reduction crosses the two: the row statistics
// come from the forward pass and the delta kernel).
//
// Replaces the reference's attention template backward (src/dew/nn/kernels/templates/attention_mosaic_dkv.py,
// attention_mosaic_dq.py), which it records as 6-9x slower than cuDNN on B200 (src/dew/nn/attention_kernels.py:772-796).
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/attn_variant.cuh"
#include <type_traits>

namespace dewb {
namespace flashbwd {

constexpr int THREADS = 320;            // 8 softmax warps (two threads per TMEM lane), a TMA warp, an MMA warp
constexpr int TMA_WARP = 8, MMA_WARP = 9;
constexpr float LOG2E = 1.4426950408889634f;
using attn::Variant;
using attn::fast_tanh;

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                             const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2, int B,
                             int S, int H, int D, long long do_sb, long long do_ss,
                             long long do_sh, long long o_sb, long long o_ss, long long o_sh) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;   // one warp per (b, s, h)
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long long>(B) * S * H) return;
  const int h = static_cast<int>(row % H);
  const long long bs = row / H;
  const int s = static_cast<int>(bs % S);
  const int b = static_cast<int>(bs / S);
  const __nv_bfloat16* a = dO + b * do_sb + s * do_ss + h * do_sh;
  const __nv_bfloat16* c = O + b * o_sb + s * o_ss + h * o_sh;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const uint32_t x = *reinterpret_cast<const uint32_t*>(a + i);
    const uint32_t y = *reinterpret_cast<const uint32_t*>(c + i);
    acc += bf16_lo(x) * bf16_lo(y) + bf16_hi(x) * bf16_hi(y);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const long long o = (static_cast<long long>(b) * H + h) * S + s;
    delta[o] = acc;
    lse2[o] = lse[o] * LOG2E;          // the log-sum-exp in log2 units, as both MMA kernels use it
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dQ kernel: one CTA per 128 query rows of one head; key blocks of 64 stream through a 5-stage K / V ring. Q and dO are
// the A operands of every score product of the CTA: the softmax threads copy them once from shared to tensor memory, so
// the score products fetch only the 64-key K / V block from shared memory (with Q / dO read from shared memory for every
// block, the operand fetch and not the tensor pipe set the pace).
//   warps 0..3  softmax group 0 : key blocks 0, 2, 4, ...   one thread per query row (its lse and delta in registers)
//   warps 4..7  softmax group 1 : key blocks 1, 3, 5, ...
//               each group owns a pair of TMEM score buffers (S, dP) and writes dS (bf16) over the first 32 columns of
//               its S buffer; dQ is one accumulator
//   warp 8      TMA producer;  warp 9  MMA issuer (scores two blocks ahead, dQ += dS K as each group delivers dS)
template <int D>
struct DqCfg {
  static constexpr int BM = 128, BN = 64, KSTAGES = 5;
  static constexpr int SUB = D / 64;
  static constexpr int Q_TILE = BM * D * 2;          // [128 x D]
  static constexpr int KV_TILE = BN * D * 2;         // [64 x D]
  static constexpr int SMEM = 2 * Q_TILE + KSTAGES * 2 * KV_TILE + 1024 + 256;
  static constexpr int TM_S0 = 0, TM_DP0 = 64, TM_S1 = 128, TM_DP1 = 192, TM_DQ = 256, TM_COLS = 512;
  static constexpr int TM_QA = 384, TM_DOA = 448;    // Q and dO as tensor-memory A operands (D / 2 packed columns each)
};

struct DqBars {
  uint64_t q_full;
  uint64_t kv_full[5], kv_empty[5];
  uint64_t sdp_full[2];                 // per softmax group
  uint64_t ds_full[2];                  // per softmax group
  uint64_t a_ready;                     // Q and dO copied to tensor memory (one arrival per softmax warp)
  uint64_t all_done;
  uint32_t tmem_base;
  int abort_flag;
  int it_lo;                            // first key block this query tile sees (variants only)
};

template <int D, bool CAUSAL, bool VAR>
__global__ void __launch_bounds__(THREADS, 1)
flash_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tdo,
                const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dq, int S,
                int T, int Hq, int Hkv, long long dq_sb, long long dq_ss, long long dq_sh, float scale, Variant var,
                int* __restrict__ err) {
  using C = DqCfg<D>;
  constexpr int BM = C::BM, BN = C::BN, KS = C::KSTAGES;
  extern __shared__ uint8_t smem_raw[];
  {
    // An earlier launch reported a timed-out wait: leave at once instead of queueing more waits behind it. One
    // thread reads the status so the whole CTA takes the same branch.
    __shared__ int poisoned;
    if (threadIdx.x == 0) poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (poisoned != 0) return;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::Q_TILE;
  uint8_t* sK = sdO + C::Q_TILE;             // KS stages
  uint8_t* sV = sK + KS * C::KV_TILE;        // KS stages
  DqBars* bars = reinterpret_cast<DqBars*>(sV + KS * C::KV_TILE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = CAUSAL ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (Hq / Hkv);
  const int q0 = qt * BM;
  const int n_all = CAUSAL ? min((q0 + BM + (T - S) + BN - 1) / BN, (T + BN - 1) / BN) : (T + BN - 1) / BN;
  const float scale_log2 = scale * LOG2E;

  if (threadIdx.x == 0) {
    if (VAR) bars->it_lo = attn::first_key_tile(var, b, q0, S, T, BN, n_all);
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < KS; ++i) { mbar_init(&bars->kv_full[i], 1); mbar_init(&bars->kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->sdp_full[i], 1);
      mbar_init(&bars->ds_full[i], 4);
    }
    mbar_init(&bars->all_done, 1);
    mbar_init(&bars->a_ready, 8);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == MMA_WARP) { tmem_alloc(&bars->tmem_base, C::TM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  // every role walks the key blocks it_lo .. n_all - 1; rings, phases and "first block" tests count from it_lo
  const int it_lo = VAR ? bars->it_lo : 0;
  const int iters = n_all - it_lo;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, 2 * C::Q_TILE);
#pragma unroll
      for (int t = 0; t < C::SUB; ++t) {
        tma_load_4d(sQ + t * (BM * 128), &tq, &bars->q_full, t * 64, h, q0, b);
        tma_load_4d(sdO + t * (BM * 128), &tdo, &bars->q_full, t * 64, h, q0, b);
      }
      for (int it = 0; it < iters; ++it) {
        const int ks = it % KS; const uint32_t ph = (it / KS) & 1;
        if (!mbar_wait(&bars->kv_empty[ks], ph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&bars->kv_full[ks], 2 * C::KV_TILE);
#pragma unroll
        for (int t = 0; t < C::SUB; ++t) {
          tma_load_4d(sK + ks * C::KV_TILE + t * (BN * 128), &tk, &bars->kv_full[ks], t * 64, hk, (it_lo + it) * BN, b);
          tma_load_4d(sV + ks * C::KV_TILE + t * (BN * 128), &tv, &bars->kv_full[ks], t * 64, hk, (it_lo + it) * BN, b);
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // Key block `it` belongs to group g = it & 1 (its number within the group is it >> 1) and to ring stage it % KS.
    // The whole warp runs this loop and waits together; one elected lane issues (see mbar_wait_warp).
    constexpr uint32_t idesc_s = make_idesc(BM, BN, 1, 1, 0, 0);
    constexpr uint32_t idesc_dq = make_idesc(BM, D, 1, 1, 0, 1);
    bool ok = mbar_wait_warp(&bars->a_ready, 0, abort_flag);
    if (!ok && lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL);
    tc_fence_after();
    // The score products of block `it` (one lane, inside an elected region).  The group's score buffers hold dS of its
    // previous block until that block's dQ product has read it; that product was issued by the same lane before these
    // and the tensor pipe runs one thread's products in order.
    auto score_products = [&](int it) {
      const int g = it & 1;
      const int ks = it % KS;
      const uint32_t ka = smem_u32(sK + ks * C::KV_TILE), va = smem_u32(sV + ks * C::KV_TILE);
      const uint32_t ts = tmem + (g ? C::TM_S1 : C::TM_S0), tdp = tmem + (g ? C::TM_DP1 : C::TM_DP0);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {           // 16 features of Q / dO = 8 packed 32-bit columns
        const uint32_t boff = (kk >> 2) * (BN * 128) + (kk & 3) * 32;
        umma_bf16_ts(ts, tmem + C::TM_QA + kk * 8, make_sdesc_sw128(ka + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t boff = (kk >> 2) * (BN * 128) + (kk & 3) * 32;
        umma_bf16_ts(tdp, tmem + C::TM_DOA + kk * 8, make_sdesc_sw128(va + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit(&bars->sdp_full[g]);
    };
    auto issue_scores = [&](int it) -> bool {
      if (!mbar_wait_warp(&bars->kv_full[it % KS], (it / KS) & 1, abort_flag)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); return false; }
      tc_fence_after();
      if (elect_one()) score_products(it);
      __syncwarp();
      return true;
    };
    if (ok && iters > 0) ok = issue_scores(0);
    if (ok && iters > 1) ok = issue_scores(1);
    for (int it = 0; it < iters && ok; ++it) {
      const int g = it & 1; const uint32_t phg = (it >> 1) & 1;
      const int ks = it % KS;
      {
        // two lanes wait at the same time: for this block's dS and for the K / V block the next score products read
        bool got = true;
        if (lane == 0) got = mbar_wait(&bars->ds_full[g], phg, abort_flag);
        else if (lane == 1 && it + 2 < iters) got = mbar_wait(&bars->kv_full[(it + 2) % KS], ((it + 2) / KS) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; break; }
      }
      tc_fence_after();
      const uint32_t ka = smem_u32(sK + ks * C::KV_TILE);
      const uint32_t tds = tmem + (g ? C::TM_S1 : C::TM_S0);      // 16 keys of dS = 8 packed 32-bit columns
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma_bf16_ts(tmem + C::TM_DQ, tds + kk * 8, make_sdesc_sw128(ka + kk * 2048, BN * 128, 1024), idesc_dq,
                       (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bars->kv_empty[ks]);
        if (it + 2 < iters) score_products(it + 2);
      }
      __syncwarp();
    }
    if (ok && elect_one()) umma_commit(&bars->all_done);
    __syncwarp();
  } else {
    const int q4 = warp & 3, g = warp >> 2;
    const int r = q4 * 32 + lane;                   // query row within the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
    const int row = q0 + r;
    const long long stat = (static_cast<long long>(b) * Hq + h) * S + row;
    const float lse2 = row < S ? lse[stat] * LOG2E : 0.f;
    const float dl = row < S ? delta[stat] : 0.f;
    const int limit = CAUSAL ? (row + (T - S)) : (T - 1);
    const uint32_t s_col = g ? C::TM_S1 : C::TM_S0, dp_col = g ? C::TM_DP1 : C::TM_DP0;
    bool ok = true;
    {
      // Group 0 copies its row of Q, group 1 its row of dO, from the swizzled shared tile to tensor memory: lane = row,
      // 32-bit column w = features 2w, 2w + 1 (the layout of a tensor-memory A operand).
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->q_full, 0, abort_flag))) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; }
      if (ok) {
        const uint8_t* src = (g ? sdO : sQ) + r * 128;
        const uint32_t dst = tmem + lane_addr + (g ? C::TM_DOA : C::TM_QA);
#pragma unroll
        for (int t = 0; t < C::SUB; ++t) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t w[16];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 x = *reinterpret_cast<const uint4*>(src + t * (BM * 128) + (((hf * 4 + c) ^ (r & 7)) << 4));
              w[c * 4] = x.x; w[c * 4 + 1] = x.y; w[c * 4 + 2] = x.z; w[c * 4 + 3] = x.w;
            }
            tmem_st_32x32b_x16(dst + t * 32 + hf * 16, w);
          }
        }
        tmem_st_wait();
        tc_fence_before();
      }
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&bars->a_ready);
    }
    int mine = 0;
    for (int it = g; it < iters && ok; it += 2, ++mine) {
      const uint32_t phg = mine & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->sdp_full[g], phg, abort_flag))) { atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; break; }
      tc_fence_after();
      const int k0 = (it_lo + it) * BN;
      uint32_t packed[BN / 2];
      auto block = [&](auto masked_tag) {
        constexpr bool MASKED = decltype(masked_tag)::value;
        const float cap2 = VAR ? var.softcap * LOG2E : 0.f, inv_cap2 = (VAR && var.softcap > 0.f) ? 1.f / cap2 : 0.f;
        const int first = VAR && var.window > 0 ? row + (T - S) - var.window + 1 : -0x40000000;   // first visible key of this row
        const int* ksp = (VAR && var.q_seg != nullptr) ? var.k_seg + static_cast<long long>(b) * T : nullptr;
        const int my_seg = ksp != nullptr ? var.q_seg[static_cast<long long>(b) * S + min(row, S - 1)] : 0;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32b_x32(tmem + lane_addr + s_col + c * 32, sv);
          tmem_ld_32x32b_x32(tmem + lane_addr + dp_col + c * 32, dv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int key = k0 + c * 32 + i;
            float x0 = __uint_as_float(sv[i]) * scale_log2, x1 = __uint_as_float(sv[i + 1]) * scale_log2;
            float f0 = 1.f, f1 = 1.f;               // d(capped score) / d(score)
            if (VAR && var.softcap > 0.f) {
              const float t0 = fast_tanh(x0 * inv_cap2), t1 = fast_tanh(x1 * inv_cap2);
              x0 = cap2 * t0; x1 = cap2 * t1;
              f0 = 1.f - t0 * t0; f1 = 1.f - t1 * t1;
            }
            float p0 = fast_exp2(x0 - lse2);
            float p1 = fast_exp2(x1 - lse2);
            if (MASKED) {
              if (key > limit || key >= T) p0 = 0.f;
              if (key + 1 > limit || key + 1 >= T) p1 = 0.f;
              if (VAR) {
                if (key < first) p0 = 0.f;
                if (key + 1 < first) p1 = 0.f;
                if (ksp != nullptr) {
                  if (key < T && ksp[key] != my_seg) p0 = 0.f;
                  if (key + 1 < T && ksp[key + 1] != my_seg) p1 = 0.f;
                }
              }
            }
            packed[(c * 32 + i) >> 1] = pack_bf16(p0 * (__uint_as_float(dv[i]) - dl) * f0, p1 * (__uint_as_float(dv[i + 1]) - dl) * f1);
          }
        }
      };
      // only blocks that reach past the first row's last visible key (or past T) need the comparisons: one branch per warp;
      // with a window or packed documents every block is compared
      const int warp_limit = CAUSAL ? (q0 + q4 * 32 + (T - S)) : (T - 1);
      if ((VAR && (var.window > 0 || var.q_seg != nullptr)) || k0 + BN - 1 > warp_limit || k0 + BN > T) block(std::true_type{});
      else block(std::false_type{});
      // dS (bf16 pairs) over the first 32 columns of this group's S buffer: each thread overwrites only its own row,
      // whose scores it holds in registers
      {
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = packed[i]; hi[i] = packed[16 + i]; }
        tmem_st_32x32b_x16(tmem + lane_addr + s_col, lo);
        tmem_st_32x32b_x16(tmem + lane_addr + s_col + 16, hi);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_full[g]);
    }
    if (ok && iters > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->all_done, 0, abort_flag))) { atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; }
    }
    if (ok) {
      tc_fence_after();
      // group g writes gradient columns [g * D/2, (g + 1) * D/2)
      __nv_bfloat16* orow = dq + b * dq_sb + static_cast<long long>(row) * dq_ss + h * dq_sh + g * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t v[32];
        if (iters > 0) { tmem_ld_32x32b_x32(tmem + lane_addr + C::TM_DQ + g * (D / 2) + c * 32, v); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row < S) {
          uint4* o4 = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(v[q * 8 + 0]) * scale, __uint_as_float(v[q * 8 + 1]) * scale);
            pk.y = pack_bf16(__uint_as_float(v[q * 8 + 2]) * scale, __uint_as_float(v[q * 8 + 3]) * scale);
            pk.z = pack_bf16(__uint_as_float(v[q * 8 + 4]) * scale, __uint_as_float(v[q * 8 + 5]) * scale);
            pk.w = pack_bf16(__uint_as_float(v[q * 8 + 6]) * scale, __uint_as_float(v[q * 8 + 7]) * scale);
            o4[q] = pk;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, C::TM_COLS); }
}

// ---------------------------------------------------------------------------------------------------------------
// dK / dV kernel
//   warps 0..3  softmax group 0 : iterations 0, 2, 4, ...   one thread per key row, all 64 query columns
//   warps 4..7  softmax group 1 : iterations 1, 3, 5, ...
//               Each group owns a pair of TMEM score buffers (S^T, dP^T) and writes P^T and dS^T (bf16) over their first
//               32 columns; the gradient accumulators dV and dK are shared (the MMA thread issues every product,
//               and accumulation commutes). While one group computes its exponentials the other loads scores or
//               stores operands. No reduction crosses threads: the row statistics come with the Q / dO tiles.
//   warp 8      TMA producer : K, V once; then Q, dO tiles and the block's 64 + 64 statistics into a 4-stage ring
//   warp 9      MMA issuer   : scores two iterations ahead, gradient products as each group delivers its operands
template <int D>
struct DkvCfg {
  static constexpr int BKV = 128, BQ = 64, QSTAGES = 4;
  static constexpr int SUB = D / 64;
  static constexpr int KV_TILE = BKV * D * 2;        // [128 x D]
  static constexpr int Q_TILE = BQ * D * 2;          // [64 x D]
  static constexpr int STAT_BYTES = 2 * BQ * 4;      // per stage: 64 log-sum-exps, 64 deltas
  static constexpr int SMEM = 2 * KV_TILE + QSTAGES * 2 * Q_TILE + QSTAGES * STAT_BYTES + 1024 + 256;
  static constexpr int TM_ST0 = 0, TM_DPT0 = 64, TM_ST1 = 128, TM_DPT1 = 192, TM_DV = 256, TM_DK = 256 + D, TM_COLS = 512;
};

struct DkvBars {
  uint64_t kv_full;
  uint64_t q_full[5], q_empty[5];
  uint64_t st_full[2];                  // per softmax group
  uint64_t pds_full[2];                 // per softmax group
  uint64_t all_done;
  uint32_t tmem_base;
  int abort_flag;
  int q_end;                            // one past the last query block that sees this key tile
};

template <int D, bool CAUSAL, bool VAR>
__global__ void __launch_bounds__(THREADS, 1)
flash_dkv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tdo,
                 const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                 const float* __restrict__ lse2, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dk,
                 __nv_bfloat16* __restrict__ dv, int S, int T, int Hq, int Hkv, long long dk_sb, long long dk_ss,
                 long long dk_sh, long long dv_sb, long long dv_ss, long long dv_sh, float scale, Variant var,
                 int* __restrict__ err) {
  using C = DkvCfg<D>;
  constexpr int BKV = C::BKV, BQ = C::BQ, QS = C::QSTAGES;
  extern __shared__ uint8_t smem_raw[];
  {
    // An earlier launch reported a timed-out wait: leave at once instead of queueing more waits behind it. One
    // thread reads the status so the whole CTA takes the same branch.
    __shared__ int poisoned;
    if (threadIdx.x == 0) poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (poisoned != 0) return;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::KV_TILE;
  uint8_t* sQ = sV + C::KV_TILE;             // QS stages
  uint8_t* sdO = sQ + QS * C::Q_TILE;        // QS stages
  float* sStat = reinterpret_cast<float*>(sdO + QS * C::Q_TILE);   // [QS stages][lse2 64 | delta 64]
  DkvBars* bars = reinterpret_cast<DkvBars*>(reinterpret_cast<uint8_t*>(sStat) + QS * C::STAT_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid ordered by key tile first, so that with causal masking the long CTAs (early key tiles see every later
  // query block) of ALL heads start first and the short ones fill the tail: blocks are issued in index order.
  const int per_tile = static_cast<int>(gridDim.x) / ((T + BKV - 1) / BKV);      // = Hkv * batch
  const int kt = blockIdx.x / per_tile;
  const int hk = (blockIdx.x % per_tile) % Hkv, b = (blockIdx.x % per_tile) / Hkv;
  const int rep = Hq / Hkv;
  const int kv0 = kt * BKV;
  // first query block that can see any key of this tile (causal, bottom-right aligned): q + (T - S) >= kv0
  const int q_first = CAUSAL ? max(0, kv0 - (T - S)) / BQ : 0;
  const float scale_log2 = scale * LOG2E;

  if (threadIdx.x == 0) {
    // one past the last query block that sees this key tile (a window or packed documents end it early)
    bars->q_end = VAR ? attn::end_query_block(var, b, kv0, BKV, S, T, BQ) : (S + BQ - 1) / BQ;
    mbar_init(&bars->kv_full, 1);
    for (int i = 0; i < QS; ++i) { mbar_init(&bars->q_full[i], 1); mbar_init(&bars->q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->st_full[i], 1);
      mbar_init(&bars->pds_full[i], 4);
    }
    mbar_init(&bars->all_done, 1);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == MMA_WARP) { tmem_alloc(&bars->tmem_base, C::TM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  const int nqb = bars->q_end - q_first;                // query blocks per head
  const int iters = nqb > 0 ? nqb * rep : 0;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      mbar_expect_tx(&bars->kv_full, 2 * C::KV_TILE);
#pragma unroll
      for (int t = 0; t < C::SUB; ++t) {
        tma_load_4d(sK + t * (BKV * 128), &tk, &bars->kv_full, t * 64, hk, kv0, b);
        tma_load_4d(sV + t * (BKV * 128), &tv, &bars->kv_full, t * 64, hk, kv0, b);
      }
      for (int it = 0; it < iters; ++it) {
        const int qs = it % QS; const uint32_t ph = (it / QS) & 1;
        const int h = hk * rep + it / nqb;
        const int qb = (q_first + it % nqb) * BQ;
        if (!mbar_wait(&bars->q_empty[qs], ph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&bars->q_full[qs], 2 * C::Q_TILE + C::STAT_BYTES);
#pragma unroll
        for (int t = 0; t < C::SUB; ++t) {
          tma_load_4d(sQ + qs * C::Q_TILE + t * (BQ * 128), &tq, &bars->q_full[qs], t * 64, h, qb, b);
          tma_load_4d(sdO + qs * C::Q_TILE + t * (BQ * 128), &tdo, &bars->q_full[qs], t * 64, h, qb, b);
        }
        // the block's per-query statistics ride the same barrier: 64 log-sum-exps (log2 units) and 64 deltas
        const long long stat = (static_cast<long long>(b) * Hq + h) * S + qb;
        bulk_load_1d(sStat + qs * 2 * BQ, lse2 + stat, BQ * 4, &bars->q_full[qs]);
        bulk_load_1d(sStat + qs * 2 * BQ + BQ, delta + stat, BQ * 4, &bars->q_full[qs]);
      }
    }
  } else if (warp == MMA_WARP) {
    // Iteration `it` belongs to group g = it & 1 (its number within the group is it >> 1) and to Q stage it % QS.
    // The whole warp runs this loop and waits together; one elected lane issues (see mbar_wait_warp).
    constexpr uint32_t idesc_st = make_idesc(BKV, BQ, 1, 1, 0, 0);
    constexpr uint32_t idesc_acc = make_idesc(BKV, D, 1, 1, 0, 1);
    bool ok = mbar_wait_warp(&bars->kv_full, 0, abort_flag);
    if (!ok && lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL);
    const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
    // The score products of iteration `it` (one lane, inside an elected region).  The group's score buffers hold P^T /
    // dS^T of its previous iteration until that iteration's gradient products have read them; those were issued by the
    // same lane before these and the tensor pipe runs one thread's products in order.
    auto score_products = [&](int it) {
      const int g = it & 1;
      const int qs = it % QS;
      const uint32_t qa = smem_u32(sQ + qs * C::Q_TILE), da = smem_u32(sdO + qs * C::Q_TILE);
      const uint32_t tst = tmem + (g ? C::TM_ST1 : C::TM_ST0), tdp = tmem + (g ? C::TM_DPT1 : C::TM_DPT0);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t aoff = (kk >> 2) * (BKV * 128) + (kk & 3) * 32;
        const uint32_t boff = (kk >> 2) * (BQ * 128) + (kk & 3) * 32;
        umma_bf16_ss(tst, make_sdesc_sw128(ka + aoff, 16, 1024), make_sdesc_sw128(qa + boff, 16, 1024), idesc_st, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t aoff = (kk >> 2) * (BKV * 128) + (kk & 3) * 32;
        const uint32_t boff = (kk >> 2) * (BQ * 128) + (kk & 3) * 32;
        umma_bf16_ss(tdp, make_sdesc_sw128(va + aoff, 16, 1024), make_sdesc_sw128(da + boff, 16, 1024), idesc_st, kk > 0 ? 1u : 0u);
      }
      umma_commit(&bars->st_full[g]);
    };
    auto issue_scores = [&](int it) -> bool {
      if (!mbar_wait_warp(&bars->q_full[it % QS], (it / QS) & 1, abort_flag)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); return false; }
      tc_fence_after();
      if (elect_one()) score_products(it);
      __syncwarp();
      return true;
    };
    if (ok && iters > 0) ok = issue_scores(0);
    if (ok && iters > 1) ok = issue_scores(1);
    for (int it = 0; it < iters && ok; ++it) {
      const int g = it & 1; const uint32_t phg = (it >> 1) & 1;
      const int qs = it % QS;
      {
        // two lanes wait at the same time: for this iteration's P^T / dS^T and for the Q / dO block the next score
        // products read
        bool got = true;
        if (lane == 0) got = mbar_wait(&bars->pds_full[g], phg, abort_flag);
        else if (lane == 1 && it + 2 < iters) got = mbar_wait(&bars->q_full[(it + 2) % QS], ((it + 2) / QS) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; break; }
      }
      tc_fence_after();
      const uint32_t qa = smem_u32(sQ + qs * C::Q_TILE), da = smem_u32(sdO + qs * C::Q_TILE);
      const uint32_t tp = tmem + (g ? C::TM_ST1 : C::TM_ST0), tds = tmem + (g ? C::TM_DPT1 : C::TM_DPT0);
      if (elect_one()) {
        // 16 queries of P^T / dS^T = 8 packed 32-bit columns
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk)
          umma_bf16_ts(tmem + C::TM_DV, tp + kk * 8, make_sdesc_sw128(da + kk * 2048, BQ * 128, 1024), idesc_acc,
                       (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk)
          umma_bf16_ts(tmem + C::TM_DK, tds + kk * 8, make_sdesc_sw128(qa + kk * 2048, BQ * 128, 1024), idesc_acc,
                       (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bars->q_empty[qs]);
        if (it + 2 < iters) score_products(it + 2);
      }
      __syncwarp();
    }
    if (ok && elect_one()) umma_commit(&bars->all_done);        // every product issued above has completed when this fires
    __syncwarp();
  } else {
    const int q4 = warp & 3, g = warp >> 2;
    const int r = q4 * 32 + lane;                   // key row within the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
    const int key = kv0 + r;
    const uint32_t st_col = g ? C::TM_ST1 : C::TM_ST0, dp_col = g ? C::TM_DPT1 : C::TM_DPT0;
    bool ok = true;
    int mine = 0;
    for (int it = g; it < iters && ok; it += 2, ++mine) {
      const uint32_t phg = mine & 1;
      const int qs = it % QS; const uint32_t phq = (it / QS) & 1;
      const int qb = (q_first + it % nqb) * BQ;
      // the block's statistics arrived with its Q / dO tiles
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->q_full[qs], phq, abort_flag))) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
      const float4* lse4 = reinterpret_cast<const float4*>(sStat + qs * 2 * BQ);
      const float4* dlt4 = reinterpret_cast<const float4*>(sStat + qs * 2 * BQ + BQ);
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->st_full[g], phg, abort_flag))) { atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; break; }
      tc_fence_after();
      uint32_t pp[BQ / 2], ds[BQ / 2];
      auto block = [&](auto masked_tag) {
        constexpr bool MASKED = decltype(masked_tag)::value;
        const float cap2 = VAR ? var.softcap * LOG2E : 0.f, inv_cap2 = (VAR && var.softcap > 0.f) ? 1.f / cap2 : 0.f;
        const int* qsp = (VAR && var.q_seg != nullptr) ? var.q_seg + static_cast<long long>(b) * S + qb : nullptr;
        const int my_seg = qsp != nullptr ? var.k_seg[static_cast<long long>(b) * T + min(key, T - 1)] : 0;
#pragma unroll
        for (int c = 0; c < BQ / 32; ++c) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32b_x32(tmem + lane_addr + st_col + c * 32, sv);
          tmem_ld_32x32b_x32(tmem + lane_addr + dp_col + c * 32, dv);
          tmem_ld_wait();
          const int qbase = qb + c * 32 + (T - S);
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 l4 = lse4[(c * 32 + i) >> 2], d4 = dlt4[(c * 32 + i) >> 2];
            float x0 = __uint_as_float(sv[i]) * scale_log2, x1 = __uint_as_float(sv[i + 1]) * scale_log2;
            float x2 = __uint_as_float(sv[i + 2]) * scale_log2, x3 = __uint_as_float(sv[i + 3]) * scale_log2;
            float f0 = 1.f, f1 = 1.f, f2 = 1.f, f3 = 1.f;       // d(capped score) / d(score)
            if (VAR && var.softcap > 0.f) {
              const float t0 = fast_tanh(x0 * inv_cap2), t1 = fast_tanh(x1 * inv_cap2);
              const float t2 = fast_tanh(x2 * inv_cap2), t3 = fast_tanh(x3 * inv_cap2);
              x0 = cap2 * t0; x1 = cap2 * t1; x2 = cap2 * t2; x3 = cap2 * t3;
              f0 = 1.f - t0 * t0; f1 = 1.f - t1 * t1; f2 = 1.f - t2 * t2; f3 = 1.f - t3 * t3;
            }
            float p0 = fast_exp2(x0 - l4.x);
            float p1 = fast_exp2(x1 - l4.y);
            float p2 = fast_exp2(x2 - l4.z);
            float p3 = fast_exp2(x3 - l4.w);
            if (MASKED) {
              if (CAUSAL) {
                if (key > qbase + i) p0 = 0.f;
                if (key > qbase + i + 1) p1 = 0.f;
                if (key > qbase + i + 2) p2 = 0.f;
                if (key > qbase + i + 3) p3 = 0.f;
              }
              if (key >= T) { p0 = 0.f; p1 = 0.f; p2 = 0.f; p3 = 0.f; }
              if (VAR) {
                if (var.window > 0) {           // key visible iff key > (query + T - S) - window
                  if (key + var.window <= qbase + i) p0 = 0.f;
                  if (key + var.window <= qbase + i + 1) p1 = 0.f;
                  if (key + var.window <= qbase + i + 2) p2 = 0.f;
                  if (key + var.window <= qbase + i + 3) p3 = 0.f;
                }
                if (qsp != nullptr) {
                  const int qi = c * 32 + i;
                  if (qb + qi + 3 < S) {
                    const int4 id = *reinterpret_cast<const int4*>(qsp + qi);
                    if (id.x != my_seg) p0 = 0.f;
                    if (id.y != my_seg) p1 = 0.f;
                    if (id.z != my_seg) p2 = 0.f;
                    if (id.w != my_seg) p3 = 0.f;
                  } else {
                    if (qb + qi < S && qsp[qi] != my_seg) p0 = 0.f;
                    if (qb + qi + 1 < S && qsp[qi + 1] != my_seg) p1 = 0.f;
                    if (qb + qi + 2 < S && qsp[qi + 2] != my_seg) p2 = 0.f;
                    if (qb + qi + 3 < S && qsp[qi + 3] != my_seg) p3 = 0.f;
                  }
                }
              }
            }
            const int o = (c * 32 + i) >> 1;
            pp[o] = pack_bf16(p0, p1);
            pp[o + 1] = pack_bf16(p2, p3);
            ds[o] = pack_bf16(p0 * (__uint_as_float(dv[i]) - d4.x) * f0, p1 * (__uint_as_float(dv[i + 1]) - d4.y) * f1);
            ds[o + 1] = pack_bf16(p2 * (__uint_as_float(dv[i + 2]) - d4.z) * f2, p3 * (__uint_as_float(dv[i + 3]) - d4.w) * f3);
          }
        }
      };
      // only query blocks that start before this warp's last key (or key rows past T) need the comparisons: one branch
      // per warp; with a window or packed documents every block is compared
      const int warp_last_key = kv0 + q4 * 32 + 31;
      if ((VAR && (var.window > 0 || var.q_seg != nullptr)) || (CAUSAL && warp_last_key > qb + (T - S)) || warp_last_key >= T)
        block(std::true_type{});
      else block(std::false_type{});
      // P^T and dS^T (bf16 pairs) over the first 32 columns of this group's S^T and dP^T buffers: each thread overwrites
      // only its own row, whose scores it holds in registers
      {
        uint32_t t0[16], t1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { t0[i] = pp[i]; t1[i] = pp[16 + i]; }
        tmem_st_32x32b_x16(tmem + lane_addr + st_col, t0);
        tmem_st_32x32b_x16(tmem + lane_addr + st_col + 16, t1);
#pragma unroll
        for (int i = 0; i < 16; ++i) { t0[i] = ds[i]; t1[i] = ds[16 + i]; }
        tmem_st_32x32b_x16(tmem + lane_addr + dp_col, t0);
        tmem_st_32x32b_x16(tmem + lane_addr + dp_col + 16, t1);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_full[g]);
    }
    if (ok && iters > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->all_done, 0, abort_flag))) { atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; }
    }
    if (ok) {
      tc_fence_after();
      // group g writes gradient columns [g * D/2, (g + 1) * D/2)
      __nv_bfloat16* kout = dk + b * dk_sb + static_cast<long long>(key) * dk_ss + hk * dk_sh + g * (D / 2);
      __nv_bfloat16* vout = dv + b * dv_sb + static_cast<long long>(key) * dv_ss + hk * dv_sh + g * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t a[32], gr[32];
        if (iters > 0) {
          tmem_ld_32x32b_x32(tmem + lane_addr + C::TM_DV + g * (D / 2) + c * 32, a);
          tmem_ld_32x32b_x32(tmem + lane_addr + C::TM_DK + g * (D / 2) + c * 32, gr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0; gr[i] = 0; }
        }
        if (key < T) {
          uint4* v4 = reinterpret_cast<uint4*>(vout + c * 32);
          uint4* k4 = reinterpret_cast<uint4*>(kout + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 pv, pk;
            pv.x = pack_bf16(__uint_as_float(a[q * 8 + 0]), __uint_as_float(a[q * 8 + 1]));
            pv.y = pack_bf16(__uint_as_float(a[q * 8 + 2]), __uint_as_float(a[q * 8 + 3]));
            pv.z = pack_bf16(__uint_as_float(a[q * 8 + 4]), __uint_as_float(a[q * 8 + 5]));
            pv.w = pack_bf16(__uint_as_float(a[q * 8 + 6]), __uint_as_float(a[q * 8 + 7]));
            pk.x = pack_bf16(__uint_as_float(gr[q * 8 + 0]) * scale, __uint_as_float(gr[q * 8 + 1]) * scale);
            pk.y = pack_bf16(__uint_as_float(gr[q * 8 + 2]) * scale, __uint_as_float(gr[q * 8 + 3]) * scale);
            pk.z = pack_bf16(__uint_as_float(gr[q * 8 + 4]) * scale, __uint_as_float(gr[q * 8 + 5]) * scale);
            pk.w = pack_bf16(__uint_as_float(gr[q * 8 + 6]) * scale, __uint_as_float(gr[q * 8 + 7]) * scale);
            v4[q] = pv; k4[q] = pk;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, C::TM_COLS); }
}

static int make_map(CUtensorMap* m, const void* base, int B, int L, int H, int D, long long sb, long long sl, long long sh,
                    int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(L), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sl) * 2, static_cast<uint64_t>(sb) * 2};
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return make_tmap_nd(m, base, 4, dims, strides, box, 2, true);
}

static_assert(DqCfg<128>::SMEM + 64 <= 232448 && DkvCfg<128>::SMEM + 64 <= 232448, "over the 227 KB a CTA may use");

template <int D, bool CAUSAL, bool VAR>
static int launch_bwd(const void* dO, const void* q, const void* k, const void* v, const float* lse, const float* lse2, const float* delta,
                      void* dq, void* dk, void* dv, int B, int S, int T, int Hq, int Hkv, const long long* qs,
                      const long long* ks, const long long* vs, const long long* os, const long long* dos,
                      const long long* dqs, const long long* dks, const long long* dvs, float scale, const Variant& var,
                      int* err, cudaStream_t stream) {
  const long long do_sb = dos[0], do_ss = dos[1], do_sh = dos[2];
  int r;
  {
    CUtensorMap tq, tdo, tk, tv;
    if ((r = make_map(&tq, q, B, S, Hq, D, qs[0], qs[1], qs[2], 128))) return 1000 + r;
    if ((r = make_map(&tdo, dO, B, S, Hq, D, do_sb, do_ss, do_sh, 128))) return 1100 + r;
    if ((r = make_map(&tk, k, B, T, Hkv, D, ks[0], ks[1], ks[2], 64))) return 1200 + r;
    if ((r = make_map(&tv, v, B, T, Hkv, D, vs[0], vs[1], vs[2], 64))) return 1300 + r;
    auto kern = flash_dq_kernel<D, CAUSAL, VAR>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<D>::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    dim3 grid((S + 127) / 128, Hq, B);
    kern<<<grid, THREADS, DqCfg<D>::SMEM, stream>>>(tq, tdo, tk, tv, lse, delta, reinterpret_cast<__nv_bfloat16*>(dq), S, T,
                                                     Hq, Hkv, dqs[0], dqs[1], dqs[2], scale, var, err);
    if ((r = static_cast<int>(cudaGetLastError()))) return r;
  }
  {
    CUtensorMap tq, tdo, tk, tv;
    if ((r = make_map(&tq, q, B, S, Hq, D, qs[0], qs[1], qs[2], 64))) return 2000 + r;
    if ((r = make_map(&tdo, dO, B, S, Hq, D, do_sb, do_ss, do_sh, 64))) return 2100 + r;
    if ((r = make_map(&tk, k, B, T, Hkv, D, ks[0], ks[1], ks[2], 128))) return 2200 + r;
    if ((r = make_map(&tv, v, B, T, Hkv, D, vs[0], vs[1], vs[2], 128))) return 2300 + r;
    auto kern = flash_dkv_kernel<D, CAUSAL, VAR>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<D>::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    dim3 grid(((T + 127) / 128) * Hkv * B, 1, 1);
    kern<<<grid, THREADS, DkvCfg<D>::SMEM, stream>>>(tq, tdo, tk, tv, lse2, delta, reinterpret_cast<__nv_bfloat16*>(dk),
                                                      reinterpret_cast<__nv_bfloat16*>(dv), S, T, Hq, Hkv, dks[0], dks[1],
                                                      dks[2], dvs[0], dvs[1], dvs[2], scale, var, err);
    if ((r = static_cast<int>(cudaGetLastError()))) return r;
  }
  return 0;
}

}  // namespace flashbwd
}  // namespace dewb

// Every tensor is [B, length, heads, D] bf16 with unit stride along D and its own (batch, sequence, head) element
// strides, so q / k / v may be views of one fused projection output and dq / dk / dv views of one fused gradient
// buffer. lse [B,Hq,S] comes from the forward; delta is scratch of 2 * B * Hq * S floats this call fills (delta, then
// the log-sum-exp in log2 units). S must be a multiple of 64 (the statistics travel by 256-byte bulk copies).
// `strides` holds 8 triples in the order q, k, v, out, dO, dq, dk, dv.
// Variants as in the forward (window, softcap, segment ids of packed documents); `lse` must come from a forward run with the
// same variants (and sinks, if any).
extern "C" int dewb_flash_bwd_var(const void* dO, const void* q, const void* k, const void* v, const void* out,
                                  const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int T, int Hq,
                                  int Hkv, int D, const long long* strides, float scale, int causal, int window, float softcap,
                                  const int* q_seg, const int* k_seg, int* err, void* stream_ptr) {
  using namespace dewb::flashbwd;
  if ((D != 128 && D != 64) || Hq % Hkv != 0 || S % 64 != 0) return -3;
  if ((q_seg != nullptr) != (k_seg != nullptr) || window < 0 || softcap < 0.f) return -3;
  if (q_seg != nullptr && ((S % 4) || (T % 4) || (reinterpret_cast<uintptr_t>(q_seg) & 15) || (reinterpret_cast<uintptr_t>(k_seg) & 15))) return -3;
  const long long *qs = strides, *ks = strides + 3, *vs = strides + 6, *os = strides + 9, *dos = strides + 12,
                  *dqs = strides + 15, *dks = strides + 18, *dvs = strides + 21;
  for (int i = 0; i < 24; ++i) if (strides[i] % 8) return -3;       // 16-byte rows for TMA and the uint4 stores
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  const long long rows = static_cast<long long>(B) * S * Hq;
  delta_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dO), reinterpret_cast<const __nv_bfloat16*>(out), lse, delta,
      delta + static_cast<long long>(B) * Hq * S, B, S, Hq, D, dos[0], dos[1], dos[2], os[0], os[1], os[2]);
  const float* lse2 = delta + static_cast<long long>(B) * Hq * S;
  // the sink logits reach the backward through the saved log-sum-exp alone
  const Variant var{window, softcap, nullptr, q_seg, k_seg};
  const bool any = window > 0 || softcap > 0.f || q_seg != nullptr;
#define DEWB_BWD_GO(DD, CC, VV) launch_bwd<DD, CC, VV>(dO, q, k, v, lse, lse2, delta, dq, dk, dv, B, S, T, Hq, Hkv, qs, ks, vs, os, dos, dqs, dks, dvs, scale, var, err, stream)
  if (D == 128) {
    if (any) return causal ? DEWB_BWD_GO(128, true, true) : DEWB_BWD_GO(128, false, true);
    return causal ? DEWB_BWD_GO(128, true, false) : DEWB_BWD_GO(128, false, false);
  }
  if (any) return causal ? DEWB_BWD_GO(64, true, true) : DEWB_BWD_GO(64, false, true);
  return causal ? DEWB_BWD_GO(64, true, false) : DEWB_BWD_GO(64, false, false);
#undef DEWB_BWD_GO
}

extern "C" int dewb_flash_bwd(const void* dO, const void* q, const void* k, const void* v, const void* out,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int T, int Hq,
                              int Hkv, int D, const long long* strides, float scale, int causal, int* err,
                              void* stream_ptr) {
  return dewb_flash_bwd_var(dO, q, k, v, out, lse, delta, dq, dk, dv, B, S, T, Hq, Hkv, D, strides, scale, causal, 0, 0.f, nullptr,
                            nullptr, err, stream_ptr);
}
