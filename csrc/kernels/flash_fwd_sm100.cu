// Flash attention forward for sm_100a (head_dim 128 or 64, bf16, causal or full, GQA).
//
// One CTA per (query tile of 128 rows, query head, batch); 320 threads:
//   warps 0..7  softmax      : two threads per query row (warps w and w + 4 share TMEM lane quarter w & 3 and take 64
//                              of the 128 key columns each; the row maximum is exchanged through shared memory);
//                              tcgen05.ld the scores, online softmax in the log2 domain, write P (bf16) into shared
//                              memory in the 128-byte-swizzled layout.  The exponentials, not the tensor core, bound
//                              this kernel, so the softmax gets eight warps.
//   warp 8      TMA producer : Q once, then K and V tiles into 2-stage rings (cp.async.bulk.tensor, no multicast)
//   warp 9      MMA issuer   : S = Q K^T into one of two TMEM score buffers (so the next tile's scores are computed
//                              while this tile's softmax runs), then O += P V into the TMEM output accumulator
// The running maximum is applied lazily: O and l are rescaled only when a row's maximum has grown by more than 2^8
// since the last rescale, so the TMEM read-modify-write of O is rare.
//
// Replaces the reference's attention template forward (src/dew/nn/kernels/templates/attention_mosaic_forward.py) and
// the vendored FlashAttention wheels, which carry no sm_100 code (kernels/flash_attn/CMakeLists.txt:16,57).
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/attn_variant.cuh"

namespace dewb {
namespace attnfwd {

constexpr int BM = 128;        // query rows per CTA
constexpr int BN = 128;        // keys per tile
constexpr int THREADS = 320;
constexpr int TMA_WARP = 8, MMA_WARP = 9;
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

using attn::Variant;
using attn::fast_tanh;

template <int D>
struct Cfg {
  static constexpr int SUB = D / 64;                 // 64-column (128-byte) sub-tiles per row
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int KSTAGES = 3;                  // K is consumed one tile ahead of V: it needs the deeper ring
  static constexpr int TILE_BYTES = Q_BYTES + (KSTAGES + 2) * KV_BYTES + P_BYTES;
  static constexpr int SMEM = TILE_BYTES + 2560;      // + barriers and the row-maximum exchange (see Bars); no slack to spare
  static constexpr int TMEM_S0 = 0, TMEM_S1 = 128, TMEM_O = 256, TMEM_COLS = 512;
  static constexpr int TMEM_QA = 384;                // PT: Q as a tensor-memory A operand (D / 2 packed columns)
};

struct Bars {
  uint64_t q_full;
  uint64_t k_full[3], k_empty[3], v_full[2], v_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, pv_done;
  uint64_t qa_ready;                   // PT: Q copied to tensor memory (one arrival per softmax warp)
  uint32_t tmem_base;
  int abort_flag;
  int poisoned;
  int j_lo;                            // first key tile this query tile sees (variants only)
  float xmax[2][2][BM];   // [tile parity][column half][row]: partial row maxima exchanged between the two halves; the
                          // parity the last tile did not use carries the partial row sums at the end
};

static_assert(sizeof(Bars) <= 2560, "Bars must fit the space Cfg::SMEM leaves after the tiles");

// PT = true keeps P in tensor memory: each softmax thread overwrites its part of the score buffer with the packed bf16
// probabilities (tcgen05.st) and the P V product reads its A operand from there, so P never crosses shared memory (no
// 32 KB store + 32 KB operand fetch per tile) and the softmax of the next tile need not wait for the product to drain
// a shared buffer.  PT = false is the shared-memory form (P in the 128-byte-swizzled K-major layout).
template <int D, bool CAUSAL, bool PT, bool VAR>
__global__ void __launch_bounds__(THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                 int S, int T, int Hq, int Hkv, long long o_stride_b, long long o_stride_s, long long o_stride_h,
                 float scale_log2, Variant var, int* __restrict__ err) {
  using C = Cfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // The tiles fill 224 KiB, so this kernel has no static shared memory and no alignment slack: the dynamic window must
  // start on a 1024-byte boundary (the 128-byte swizzle atoms need it). If it ever did not, refuse instead of overrunning.
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    return;
  }
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;             // KSTAGES stages
  uint8_t* sV = sK + C::KSTAGES * C::KV_BYTES;   // 2 stages
  uint8_t* sP = sV + 2 * C::KV_BYTES;
  Bars* bars = reinterpret_cast<Bars*>(sP + C::P_BYTES);
  {
    // An earlier launch reported a timed-out wait: leave at once instead of queueing more waits behind it. One
    // thread reads the status so the whole CTA takes the same branch.
    if (threadIdx.x == 0) bars->poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (bars->poisoned != 0) return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = CAUSAL ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;   // heavy causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (Hq / Hkv);
  const int q0 = qt * BM;
  // keys visible to this query tile: causal alignment is bottom-right (query i sees keys <= i + T - S)
  const int n_all = CAUSAL ? min((q0 + BM + (T - S) + BN - 1) / BN, (T + BN - 1) / BN) : (T + BN - 1) / BN;

  if (threadIdx.x == 0) {
    if (VAR) bars->j_lo = attn::first_key_tile(var, b, q0, S, T, BN, n_all);
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < C::KSTAGES; ++i) { mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->s_empty[i], 8);
    }
    mbar_init(&bars->p_full, 8);
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->qa_ready, 8);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == MMA_WARP) { tmem_alloc(&bars->tmem_base, C::TMEM_COLS); tmem_relinquish(); }
  if (warp == TMA_WARP && lane == 0) { tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  // every role walks the key tiles j_lo .. n_all - 1; rings, phases and "first tile" tests count from j_lo
  const int j_lo = VAR ? bars->j_lo : 0;
  const int n_tiles = n_all - j_lo;

  if (warp == TMA_WARP) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, C::Q_BYTES);
#pragma unroll
      for (int t = 0; t < C::SUB; ++t) tma_load_4d(sQ + t * (BM * 128), &tq, &bars->q_full, t * 64, h, q0, b);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        const int ks = j % C::KSTAGES; const uint32_t kph = (j / C::KSTAGES) & 1;
        if (!mbar_wait(&bars->k_empty[ks], kph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
        mbar_expect_tx(&bars->k_full[ks], C::KV_BYTES);
#pragma unroll
        for (int t = 0; t < C::SUB; ++t) tma_load_4d(sK + ks * C::KV_BYTES + t * (BN * 128), &tk, &bars->k_full[ks], t * 64, hk, (j_lo + j) * BN, b);
        if (!mbar_wait(&bars->v_empty[st], ph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
        mbar_expect_tx(&bars->v_full[st], C::KV_BYTES);
#pragma unroll
        for (int t = 0; t < C::SUB; ++t) tma_load_4d(sV + st * C::KV_BYTES + t * (BN * 128), &tv, &bars->v_full[st], t * 64, hk, (j_lo + j) * BN, b);
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this loop and waits together; one elected lane issues (see mbar_wait_warp).
    constexpr uint32_t idesc_qk = make_idesc(BM, BN, 1, 1, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(BM, D, 1, 1, 0, 1);
    // PT: Q is the A operand of every score product of the CTA, so the softmax warps copy it once to tensor memory and
    // the score products fetch only K from shared memory
    bool ok = mbar_wait_warp(PT ? &bars->qa_ready : &bars->q_full, 0, abort_flag);
    if (!ok && lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL);
    tc_fence_after();
    const uint32_t qa = smem_u32(sQ), pa = smem_u32(sP);
    auto issue_qk = [&](int j) -> bool {
      const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
      const int ks = j % C::KSTAGES; const uint32_t kph = (j / C::KSTAGES) & 1;
      if (!mbar_wait_warp(&bars->k_full[ks], kph, abort_flag)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); return false; }
      // PT: the score buffer holds P(j - 2) until P V(j - 2) has read it; that product was issued by the same lane before
      // this one and the tensor pipe runs one thread's products in order, so no barrier is needed.
      if (!PT && !mbar_wait_warp(&bars->s_empty[st], ph ^ 1, abort_flag)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_TMEM_EMPTY); return false; }
      tc_fence_after();
      const uint32_t ka = smem_u32(sK + ks * C::KV_BYTES);
      const uint32_t ts = tmem + (st ? C::TMEM_S1 : C::TMEM_S0);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (BM * 128) + (kk & 3) * 32;
          if (PT) umma_bf16_ts(ts, tmem + C::TMEM_QA + kk * 8, make_sdesc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
          else umma_bf16_ss(ts, make_sdesc_sw128(qa + off, 16, 1024), make_sdesc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->k_empty[ks]);
        umma_commit(&bars->s_full[st]);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_tiles > 0) ok = issue_qk(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) { ok = issue_qk(j + 1); if (!ok) break; }
      const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait_warp(&bars->p_full, j & 1, abort_flag)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; break; }
      if (!mbar_wait_warp(&bars->v_full[st], ph, abort_flag)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
      tc_fence_after();
      const uint32_t va = smem_u32(sV + st * C::KV_BYTES);
      const uint32_t tp = tmem + (st ? C::TMEM_S1 : C::TMEM_S0);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          if (PT) {
            // 16 keys of P = 8 packed 32-bit columns of the score buffer this tile used
            umma_bf16_ts(tmem + C::TMEM_O, tp + kk * 8, make_sdesc_sw128(va + kk * 2048, BN * 128, 1024), idesc_pv,
                         (j > 0 || kk > 0) ? 1u : 0u);
          } else {
            const uint32_t aoff = (kk >> 2) * (BM * 128) + (kk & 3) * 32;
            umma_bf16_ss(tmem + C::TMEM_O, make_sdesc_sw128(pa + aoff, 16, 1024),
                         make_sdesc_sw128(va + kk * 2048, BN * 128, 1024), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bars->v_empty[st]);
        umma_commit(&bars->pv_done);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 0..7)
    constexpr int HC = BN / 2;                       // key columns per thread
    const int q4 = warp & 3, half = warp >> 2;
    const int r = q4 * 32 + lane;                    // query row within the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    if (PT) {
      // this thread's half of its query row, from the swizzled shared tile to tensor memory: lane = row, 32-bit column w
      // = features 2w, 2w + 1 (the layout of a tensor-memory A operand)
      const bool got = mbar_wait(&bars->q_full, 0, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; }
      if (ok) {
        constexpr int CH16 = D / 16;                  // 16-byte chunks (8 features, 4 columns) per thread
#pragma unroll
        for (int g4 = 0; g4 < CH16 / 4; ++g4) {
          uint32_t w[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int chunk = half * CH16 + g4 * 4 + c;         // within the row of D features
            const uint4 x = *reinterpret_cast<const uint4*>(sQ + (chunk >> 3) * (BM * 128) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4));
            w[c * 4] = x.x; w[c * 4 + 1] = x.y; w[c * 4 + 2] = x.z; w[c * 4 + 3] = x.w;
          }
          tmem_st_32x32b_x16(tmem + lane_addr + C::TMEM_QA + (half * CH16 + g4 * 4) * 4, w);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&bars->qa_ready);
    }
    // Both threads of a row meet at a named barrier once per tile, so no thread may leave the loop early: after a
    // wait gives up, `ok` turns false for the whole warp and the remaining iterations only keep the barrier count.
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
      float s[HC];
      float mt = -INFINITY;
      if (ok) {
        const bool got = mbar_wait(&bars->s_full[st], ph, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; }
      }
      if (ok) {
        tc_fence_after();
        {
          // both 32-column loads are in flight before the single wait
          uint32_t v0[32], v1[32];
          const uint32_t sbase = tmem + lane_addr + (st ? C::TMEM_S1 : C::TMEM_S0) + half * HC;
          tmem_ld_32x32b_x32(sbase, v0);
          tmem_ld_32x32b_x32(sbase + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(v0[i]) * scale_log2; s[32 + i] = __uint_as_float(v1[i]) * scale_log2; }
        }
        tc_fence_before();
        __syncwarp();
        if (!PT && lane == 0) mbar_arrive(&bars->s_empty[st]);   // the score buffer may be overwritten by tile j + 2
        const int k0 = (j_lo + j) * BN + half * HC;
        const int limit = CAUSAL ? (q0 + r + (T - S)) : (T - 1);   // last visible key index for this row
        if (VAR && var.softcap > 0.f) {
          // cap * tanh(score / cap), kept in the log2 domain: scale_log2 = scale * log2(e)
          const float inv_cap = 1.f / (var.softcap * 1.4426950408889634f), cap2 = var.softcap * 1.4426950408889634f;
#pragma unroll
          for (int i = 0; i < HC; ++i) s[i] = cap2 * fast_tanh(s[i] * inv_cap);
        }
        if (k0 + HC - 1 > limit || k0 + HC > T) {
#pragma unroll
          for (int i = 0; i < HC; ++i) if (k0 + i > limit || k0 + i >= T) s[i] = -INFINITY;
        }
        if (VAR) {
          if (var.window > 0) {
            const int first = q0 + r + (T - S) - var.window + 1;   // first visible key of this row
            if (k0 < first) {
#pragma unroll
              for (int i = 0; i < HC; ++i) if (k0 + i < first) s[i] = -INFINITY;
            }
          }
          if (var.q_seg != nullptr && k0 < T) {
            const int row_q = min(q0 + r, S - 1);
            const int mine = var.q_seg[static_cast<long long>(b) * S + row_q];
            const int* ks = var.k_seg + static_cast<long long>(b) * T + k0;
            // ids are non-decreasing: the whole half-tile matches iff its ends do
            const int e0 = ks[0], e1 = ks[min(HC - 1, T - 1 - k0)];
            if (e0 != mine || e1 != mine) {
#pragma unroll
              for (int i = 0; i < HC; i += 4) {
                if (k0 + i + 3 < T) {
                  const int4 id = *reinterpret_cast<const int4*>(ks + i);
                  if (id.x != mine) s[i] = -INFINITY;
                  if (id.y != mine) s[i + 1] = -INFINITY;
                  if (id.z != mine) s[i + 2] = -INFINITY;
                  if (id.w != mine) s[i + 3] = -INFINITY;
                } else {
                  for (int q = 0; q < 4; ++q) if (k0 + i + q < T && ks[i + q] != mine) s[i + q] = -INFINITY;
                }
              }
            }
          }
        }
        {
          // four independent chains, not one of 64 dependent maxima
          float m0 = s[0], m1 = s[1], m2 = s[2], m3 = s[3];
#pragma unroll
          for (int i = 4; i < HC; i += 4) { m0 = fmaxf(m0, s[i]); m1 = fmaxf(m1, s[i + 1]); m2 = fmaxf(m2, s[i + 2]); m3 = fmaxf(m3, s[i + 3]); }
          mt = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        }
      }
      // the row's maximum over all 128 columns: exchange with the thread that holds the other half of the row
      bars->xmax[j & 1][half][r] = mt;
      named_barrier_sync(1 + q4, 64);
      if (!ok) continue;
      mt = fmaxf(mt, bars->xmax[j & 1][half ^ 1][r]);
      const float m_new = fmaxf(m_used, mt);
      const bool need = (m_new - m_used > RESCALE_THRESHOLD) || (m_used == -INFINITY && m_new > -INFINITY);
      const bool any_need = __any_sync(0xffffffffu, need);
      // PV(j-1) must be complete before the shared P buffer is overwritten or O is rescaled (PT: only the latter)
      if (j > 0 && (!PT || any_need)) {
        const bool got = mbar_wait(&bars->pv_done, (j - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; continue; }
        tc_fence_after();
      }
      if (any_need) {
        const float alpha = (need && m_used > -INFINITY) ? fast_exp2(m_used - m_new) : 1.f;
        if (need) { m_used = m_new; l *= alpha; }
        if (j > 0) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {           // this thread's half of the output columns
            uint32_t v[16];
            const uint32_t col = C::TMEM_O + half * (D / 2) + c * 16;
            tmem_ld_32x32b_x16(tmem + lane_addr + col, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32b_x16(tmem + lane_addr + col, v);
          }
          tmem_st_wait();
        }
      }
      // P = exp2(s - m_used) -> bf16, swizzled into shared memory as the A operand of the PV product
      const float mu = (m_used == -INFINITY) ? 0.f : m_used;
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;      // independent partial sums (fp32, before the bf16 rounding)
      if (PT) {
        // keys [half * 64, half * 64 + 64) of this row -> packed columns [half * 32, half * 32 + 32) of the score buffer.
        // Both threads of the row hold their scores in registers since the barrier above, so the columns may be reused.
        const uint32_t pbase = tmem + lane_addr + (st ? C::TMEM_S1 : C::TMEM_S0) + half * (HC / 2);
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = fast_exp2(s[c * 32 + 2 * i] - mu), b2 = fast_exp2(s[c * 32 + 2 * i + 1] - mu);
            pk[i] = pack_bf16(a, b2);
            if (i & 1) { rs2 += a; rs3 += b2; } else { rs0 += a; rs1 += b2; }
          }
          tmem_st_32x32b_x16(pbase + c * 16, pk);
        }
        tmem_st_wait();
      } else
#pragma unroll
      for (int i8 = 0; i8 < HC / 8; ++i8) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { p[i] = fast_exp2(s[i8 * 8 + i] - mu); }
        uint4 pk;
        pk.x = pack_bf16(p[0], p[1]); pk.y = pack_bf16(p[2], p[3]); pk.z = pack_bf16(p[4], p[5]); pk.w = pack_bf16(p[6], p[7]);
        rs0 += p[0] + p[4]; rs1 += p[1] + p[5]; rs2 += p[2] + p[6]; rs3 += p[3] + p[7];
        // column half `half` is the 64-column (128-byte) sub-tile `half` of P; i8 is the 16-byte chunk within the row
        *reinterpret_cast<uint4*>(sP + half * (BM * 128) + r * 128 + ((i8 ^ (r & 7)) << 4)) = pk;
      }
      l += (rs0 + rs1) + (rs2 + rs3);
      if (!PT) fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
    }
    // epilogue: O / l -> bf16, lse
    if (ok && n_tiles > 0) {
      const bool got = mbar_wait(&bars->pv_done, (n_tiles - 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { atomicCAS(err, 0, ERR_WAIT_OTHER); ok = false; }
    }
    // the row sum over all columns (both threads of a row reach this barrier: neither branch above skips it)
    bars->xmax[n_tiles & 1][half][r] = l;      // the parity buffer the last tile left alone
    named_barrier_sync(1 + q4, 64);
    l += bars->xmax[n_tiles & 1][half ^ 1][r];
    float lse_shift = 0.f;     // log2 of the factor the sink adds to the denominator's scale
    float inv = l > 0.f ? 1.f / l : 0.f;
    if (VAR && var.sinks != nullptr) {
      // the sink joins the denominator only: softmax over [scores, sink] with the sink's value column dropped
      const float sink2 = var.sinks[h] * 1.4426950408889634f;
      const float m_fin = fmaxf(m_used, sink2);
      const float a = m_used > -INFINITY ? fast_exp2(m_used - m_fin) : 0.f;
      const float l_fin = l * a + fast_exp2(sink2 - m_fin);
      inv = a / l_fin;
      lse_shift = m_fin + log2f(l_fin);
    }
    if (ok) {
      tc_fence_after();
      const int row = q0 + r;
      __nv_bfloat16* orow = out + b * o_stride_b + static_cast<long long>(row) * o_stride_s + h * o_stride_h + half * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t v[32];
        if (n_tiles > 0) { tmem_ld_32x32b_x32(tmem + lane_addr + C::TMEM_O + half * (D / 2) + c * 32, v); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row < S) {
          uint4* o4 = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(v[q * 8 + 0]) * inv, __uint_as_float(v[q * 8 + 1]) * inv);
            pk.y = pack_bf16(__uint_as_float(v[q * 8 + 2]) * inv, __uint_as_float(v[q * 8 + 3]) * inv);
            pk.z = pack_bf16(__uint_as_float(v[q * 8 + 4]) * inv, __uint_as_float(v[q * 8 + 5]) * inv);
            pk.w = pack_bf16(__uint_as_float(v[q * 8 + 6]) * inv, __uint_as_float(v[q * 8 + 7]) * inv);
            o4[q] = pk;
          }
        }
      }
      if (half == 0 && row < S && lse != nullptr) {
        float v = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
        if (VAR && var.sinks != nullptr) v = lse_shift * 0.6931471805599453f;
        lse[(static_cast<long long>(b) * Hq + h) * S + row] = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

template <int D, bool CAUSAL, bool PT, bool VAR>
static int launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, void* out, float* lse, int B,
                  int S, int T, int Hq, int Hkv, long long osb, long long oss, long long osh, float scale_log2,
                  const Variant& var, int* err, cudaStream_t stream) {
  auto kern = flash_fwd_kernel<D, CAUSAL, PT, VAR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((S + BM - 1) / BM, Hq, B);
  kern<<<grid, THREADS, Cfg<D>::SMEM, stream>>>(tq, tk, tv, reinterpret_cast<__nv_bfloat16*>(out), lse, S, T, Hq, Hkv,
                                                 osb, oss, osh, scale_log2, var, err);
  return static_cast<int>(cudaGetLastError());
}

// A [B, L, H, D] bf16 tensor with element strides (sb, sl, sh) and unit stride along D, tiled [128 rows x 64 cols].
static int make_qkv_map(CUtensorMap* m, const void* base, int B, int L, int H, int D, long long sb, long long sl,
                        long long sh) {
  const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(L),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sl) * 2, static_cast<uint64_t>(sb) * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd(m, base, 4, dims, strides, box, 2, true);
}

static int g_variant = 1;     // 0: P through shared memory, 1: P in tensor memory (default)

}  // namespace attnfwd
}  // namespace dewb

// Selects the forward variant for later launches of this process (0: P through shared memory, 1: P in tensor memory);
// returns the previous value.
extern "C" int dewb_flash_set_variant(int variant) {
  const int old = dewb::attnfwd::g_variant;
  dewb::attnfwd::g_variant = variant;
  return old;
}

// q [B,S,Hq,D], k/v [B,T,Hkv,D] (bf16, unit stride along D, other strides in elements: batch, sequence, head);
// out [B,S,Hq,D] with its own strides; lse [B,Hq,S] fp32 (natural log), may be null.
// Variants (each off at 0 / null): `window` keys visible behind each query, `softcap`, `sinks` [Hq] fp32, `q_seg` [B,S] /
// `k_seg` [B,T] int32 segment ids of packed documents (non-decreasing along the sequence, rows 16-byte aligned: S, T % 4 == 0).
extern "C" int dewb_flash_fwd_var(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int T,
                                  int Hq, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                                  long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                                  long long o_sb, long long o_ss, long long o_sh, float scale, int causal, int window,
                                  float softcap, const float* sinks, const int* q_seg, const int* k_seg, int* err,
                                  void* stream_ptr) {
  using namespace dewb::attnfwd;
  if (D != 128 && D != 64) return -3;
  if (Hq % Hkv != 0) return -3;
  if ((q_ss % 8) || (q_sh % 8) || (q_sb % 8) || (k_ss % 8) || (k_sh % 8) || (k_sb % 8) || (v_ss % 8) || (v_sh % 8) ||
      (v_sb % 8) || (o_ss % 8) || (o_sh % 8) || (o_sb % 8))
    return -3;
  if ((q_seg != nullptr) != (k_seg != nullptr)) return -3;
  if (q_seg != nullptr && ((T % 4) || (reinterpret_cast<uintptr_t>(k_seg) & 15))) return -3;
  if (window < 0 || softcap < 0.f) return -3;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_qkv_map(&tq, q, B, S, Hq, D, q_sb, q_ss, q_sh))) return 1000 + r;
  if ((r = make_qkv_map(&tk, k, B, T, Hkv, D, k_sb, k_ss, k_sh))) return 2000 + r;
  if ((r = make_qkv_map(&tv, v, B, T, Hkv, D, v_sb, v_ss, v_sh))) return 3000 + r;
  const float scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  const Variant var{window, softcap, sinks, q_seg, k_seg};
  const bool any = window > 0 || softcap > 0.f || sinks != nullptr || q_seg != nullptr;
#define DEWB_FLASH_GO(DD, CC, PP, VV) launch<DD, CC, PP, VV>(tq, tk, tv, out, lse, B, S, T, Hq, Hkv, o_sb, o_ss, o_sh, scale_log2, var, err, stream)
  const bool pt = g_variant != 0;
  if (any) {
    // the variants run the tensor-memory form only
    if (D == 128) return causal ? DEWB_FLASH_GO(128, true, true, true) : DEWB_FLASH_GO(128, false, true, true);
    return causal ? DEWB_FLASH_GO(64, true, true, true) : DEWB_FLASH_GO(64, false, true, true);
  }
  if (D == 128) {
    if (causal) return pt ? DEWB_FLASH_GO(128, true, true, false) : DEWB_FLASH_GO(128, true, false, false);
    return pt ? DEWB_FLASH_GO(128, false, true, false) : DEWB_FLASH_GO(128, false, false, false);
  }
  if (causal) return pt ? DEWB_FLASH_GO(64, true, true, false) : DEWB_FLASH_GO(64, true, false, false);
  return pt ? DEWB_FLASH_GO(64, false, true, false) : DEWB_FLASH_GO(64, false, false, false);
#undef DEWB_FLASH_GO
}

extern "C" int dewb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int T,
                              int Hq, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                              long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                              long long o_sb, long long o_ss, long long o_sh, float scale, int causal, int* err,
                              void* stream_ptr) {
  return dewb_flash_fwd_var(q, k, v, out, lse, B, S, T, Hq, Hkv, D, q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb,
                            o_ss, o_sh, scale, causal, 0, 0.f, nullptr, nullptr, nullptr, err, stream_ptr);
}
