// Block-scaled fp8 GEMM for sm_100a (MXFP8: e4m3 values, one power-of-two ue8m0 scale per 32 consecutive elements of the
// reduction dimension), dense or grouped by rows (mixture-of-experts):
//
//     D[M,N] (bf16) = sum_k (A_q[m,k] * 2^(sa[m, k / 32] - 127)) * (B_q[n,k] * 2^(sb[n, k / 32] - 127))
//
// computed by tcgen05.mma kind::mxf8f6f4.block_scale: the tensor core applies both operands' scales per 32-element block
// while it accumulates in fp32, so nothing is rescaled in the epilogue and a block with small values keeps its precision.
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer : A [128 x 128 B] and B [192 x 128 B] tiles into a 5-stage ring (cp.async.bulk.tensor, no multicast)
//   warp 1      MMA issuer   : four K = 32 products per stage into one of two TMEM accumulators; each product names the scale
//                              factors of its 32-element block through the descriptor's scale-factor ids
//   warps 2..5  epilogue     : tcgen05.ld the finished accumulator, store bf16; overlaps the next tile's products
//   warps 6..9  scale stagers: per stage, load the packed scales of the tile's 128 A rows and 192 B rows (one 32-bit word =
//                              the four blocks of the stage for one row) and write them to tensor memory (tcgen05.st) in the
//                              layout the tensor core reads them from: lane = row % 32, column = row / 32, byte = block,
//                              the same words in all four lane quarters
//
// Tensor memory: 2 accumulators x 192 columns, then 5 scale slots x 16 columns (4 for A, 6 for B) = 464 of 512 columns.
//
// Scale storage (what `dewb_quantize_mx` writes): sf[kb][row] is one 32-bit word holding the four ue8m0 bytes of row `row`
// for reduction blocks 4 kb .. 4 kb + 3 (byte j = block 4 kb + j), rows padded so that a tile's loads stay in range.
//
// Replaces the reference's MX grouped GEMM (src/dew/nn/kernels/grouped_matmul.py:1746 `MosaicMxGmm`; formats.py:186 `MxFp8`).
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include <cuda_fp8.h>

namespace dewb {
namespace gemm_mx {

constexpr int BM = 128;
constexpr int BN = 192;
constexpr int BK = 128;                 // fp8 elements = bytes per row of a stage: one 128-byte swizzle row, four K = 32 products
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BK;        // 16 KiB
constexpr int B_BYTES = BN * BK;        // 24 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_COLS = BN;
constexpr int SF_BASE = 2 * ACC_COLS;   // 384
constexpr int SF_SLOT = 16;             // columns per stage: A at +0 (4 columns), B at +4 (6 columns)
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 320;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Shared {
  uint64_t full[STAGES];        // TMA bytes of the stage have landed
  uint64_t sf_full[STAGES];     // the stage's scale factors are in tensor memory (4 arrivals: one per stager warp)
  uint64_t empty[STAGES];       // the products that read the stage (operands and scales) have completed
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Args {
  const int* tile_group;        // grouped rows: group of each 128-row tile of A (< 0: empty), or null for a dense product
  int b_rows_per_group;         // rows of B per group (N)
  const uint32_t* sfa;          // [K / 128][sfa_rows] packed scales of A
  const uint32_t* sfb;          // [K / 128][sfb_rows] packed scales of the stacked B
  long long sfa_rows, sfb_rows;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& m_blk, int& n_blk) {
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * tiles_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int gsize = min(tiles_m - first_m, GROUP_M);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

// Instruction descriptor of kind::mxf8f6f4.block_scale: e4m3 x e4m3, both K-major, ue8m0 scales, dense, K = 32.
//   [4,6) B scale-factor id, [7,10) A format (0 = e4m3), [10,13) B format, [15] A major, [16] B major, [17,23) N >> 3,
//   [23] scale format (1 = ue8m0), [24,29) M >> 4, [29,31) A scale-factor id.  The ids pick the byte of the 32-bit scale word.
__host__ __device__ constexpr uint32_t make_idesc_mx(int M, int N, int sf_id) {
  return (static_cast<uint32_t>(sf_id) << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(M >> 4) << 24) | (static_cast<uint32_t>(sf_id) << 29);
}

__device__ __forceinline__ void umma_mxf8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x2(uint32_t taddr, uint32_t a, uint32_t b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               __nv_bfloat16* __restrict__ D, int M, int N, int K, long long ldd, const Args ga, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  {
    __shared__ int poisoned;
    if (threadIdx.x == 0) poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (poisoned != 0) return;        // an earlier launch reported a timed-out wait
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_iters = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->sf_full[s], 4); mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 4); }
    sh->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) { tmem_alloc(&sh->tmem_base, TMEM_COLS); tmem_relinquish(); }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_a); tma_prefetch_desc(&tma_b); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  auto tile_of = [&](int t, int& m0, int& n0, int& b_row0) -> bool {       // false: the tile holds no rows
    int m_blk, n_blk;
    tile_coords(t, tiles_m, tiles_n, m_blk, n_blk);
    m0 = m_blk * BM; n0 = n_blk * BN; b_row0 = 0;
    if (ga.tile_group != nullptr) {
      const int g = ga.tile_group[m_blk];
      if (g < 0) return false;
      b_row0 = g * ga.b_rows_per_group;
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0, b_row0;
        if (!tile_of(t, m0, n0, b_row0)) continue;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
          tma_load_2d(sa, &tma_a, &sh->full[stage], k * BK, m0);
          tma_load_2d(sa + A_BYTES, &tma_b, &sh->full[stage], k * BK, b_row0 + n0);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const long long pending = issued < STAGES ? issued : STAGES;
        for (long long i = 0; i < pending; ++i) {
          int s = static_cast<int>((issued - 1 - i) % STAGES);
          uint32_t ph = static_cast<uint32_t>(((issued - 1 - i) / STAGES) & 1);
          mbar_wait(&sh->full[s], ph, nullptr, 20000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0, b_row0;
        if (!tile_of(t, m0, n0, b_row0)) continue;
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_TMEM_EMPTY); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
          if (!mbar_wait(&sh->sf_full[stage], phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t sfa = tmem_base + SF_BASE + stage * SF_SLOT, sfb = sfa + 4;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {          // 32 fp8 elements = 32 bytes per product
            const uint64_t da = make_sdesc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = make_sdesc_sw128(sb + kk * 32, 16, 1024);
            umma_mxf8_ss(d_tmem, da, db, make_idesc_mx(BM, BN, kk), sfa, sfb, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&sh->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&sh->tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m0, n0, b_row0;
      if (!tile_of(t, m0, n0, b_row0)) continue;
      const int row = m0 + q * 32 + lane;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          __nv_bfloat16* out = D + static_cast<long long>(row) * ldd + col;
          if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
            uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 pk;
              pk.x = pack_bf16(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
              pk.y = pack_bf16(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
              pk.z = pack_bf16(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
              pk.w = pack_bf16(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
              o4[j] = pk;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (col + i < N) out[i] = __float2bfloat16(__uint_as_float(r[i]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------------------------ scale stagers (warps 6..9): warp w fills lane quarter w & 3
    const int q = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m0, n0, b_row0;
      if (!tile_of(t, m0, n0, b_row0)) continue;
      for (int k = 0; k < k_iters; ++k) {
        // the slot is free once the products of its previous use have completed (the same event that frees the operands)
        const bool got = mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
        tc_fence_after();
        const uint32_t* pa = ga.sfa + static_cast<long long>(k) * ga.sfa_rows + m0 + lane;
        const uint32_t* pb = ga.sfb + static_cast<long long>(k) * ga.sfb_rows + b_row0 + n0 + lane;
        const uint32_t a0 = pa[0], a1 = pa[32], a2 = pa[64], a3 = pa[96];
        const uint32_t b0 = pb[0], b1 = pb[32], b2 = pb[64], b3 = pb[96], b4 = pb[128], b5 = pb[160];
        const uint32_t base = tmem_base + lane_addr + SF_BASE + stage * SF_SLOT;
        tmem_st_32x32b_x4(base, a0, a1, a2, a3);
        tmem_st_32x32b_x4(base + 4, b0, b1, b2, b3);
        tmem_st_32x32b_x2(base + 8, b4, b5);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->sf_full[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Quantiser: x [rows, K] bf16 -> q [rows, K] e4m3 and packed scales sf[K / 128][sf_rows] (one word per row per 128
// elements, byte j = block 4 kb + j).  The scale of a block is the smallest power of two that brings its largest magnitude
// within e4m3's range (448): e = ceil(log2(amax / 448)), stored as e + 127 (ue8m0); an all-zero block stores 2^-127.
// One thread per 8 elements; the four threads of a 32-element block share the maximum through shuffles.
__global__ void quantize_mx_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                   long long rows, int K, long long ldx, long long sf_rows) {
  const long long chunks_per_row = K >> 3;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long total = rows * chunks_per_row;
  const bool live = idx < total;
  const long long row = live ? idx / chunks_per_row : 0;
  const int chunk = live ? static_cast<int>(idx - row * chunks_per_row) : 0;
  float v[8];
  float amax = 0.f;
  if (live) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + row * ldx + chunk * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]); }
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  // K is a multiple of 32, so the four threads of a block are consecutive lanes of one warp and all live or all not
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!live) return;
  int e = -127;
  if (amax > 0.f) {
    // smallest integer e with amax <= 448 * 2^e, from the bits (exact): amax = f * 2^k with f in [1, 2) and 448 = 1.75 * 2^8
    const uint32_t bits = __float_as_uint(amax);
    const int k = static_cast<int>((bits >> 23) & 0xff) - 127;
    e = k - 8 + ((bits & 0x7fffffu) > 0x600000u ? 1 : 0);
    e = max(-127, min(127, e));
  }
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);      // 2^-e, exact (e in [-127, 127] -> exponent field 0..254)
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_fp8_storage_t a = __nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v[4 + i] * inv, __NV_SATFINITE, __NV_E4M3);
    lo |= static_cast<uint32_t>(a) << (8 * i);
    hi |= static_cast<uint32_t>(b) << (8 * i);
  }
  *reinterpret_cast<uint2*>(q + row * K + chunk * 8) = make_uint2(lo, hi);
  if ((chunk & 3) == 0) {
    const int block = chunk >> 2;                       // 32-element block index along K
    sf[(static_cast<long long>(block >> 2) * sf_rows + row) * 4 + (block & 3)] = static_cast<uint8_t>(e + 127);
  }
}

static int sm_count_mx() {
  static int n[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (n[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

}  // namespace gemm_mx
}  // namespace dewb

// x [rows, K] bf16 (row stride ldx, K a multiple of 32, rows 16-byte aligned) -> q [rows, K] e4m3 bytes (contiguous) and packed
// ue8m0 scales sf [ceil(K / 128)][sf_rows] words (sf_rows >= rows; bytes of blocks past K and rows past `rows` are left as they are:
// allocate the array zeroed).
extern "C" int dewb_quantize_mx(const void* x, void* q, void* sf, long long rows, int K, long long ldx, long long sf_rows,
                                void* stream) {
  using namespace dewb::gemm_mx;
  if (K % 32 != 0 || (ldx % 8) != 0 || sf_rows < rows) return -3;
  if (rows <= 0) return 0;
  const long long total = rows * (K >> 3);
  quantize_mx_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(sf), rows, K, ldx, sf_rows);
  return static_cast<int>(cudaGetLastError());
}

// D[M,N] (bf16, row stride ldd) = block-scaled A_q [M,K] x B_q [groups * N, K]^T (e4m3 bytes, K contiguous, row strides lda / ldb
// multiples of 16 bytes, K a multiple of 128).  sfa [K / 128][sfa_rows], sfb [K / 128][sfb_rows]: packed scales as written by
// dewb_quantize_mx, with sfa_rows >= M rounded up to 128 and sfb_rows >= groups * N + 192 (a tile's loads stay in range).
// tile_group: null for a dense product (groups = 1), else the group of each 128-row tile of A (< 0: no rows).
extern "C" int dewb_gemm_mxfp8(const void* A, const void* B, void* D, const void* sfa, const void* sfb, const int* tile_group,
                               int M, int N, int K, int groups, long long lda, long long ldb, long long ldd, long long sfa_rows,
                               long long sfb_rows, int* err, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm_mx;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % BK) || (lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (sfa_rows < (M + BM - 1) / BM * BM || sfb_rows < static_cast<long long>(groups) * N + BN) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 1, true);
  if (r) return 1000 + r;
  r = make_tmap_2d(&tb, B, static_cast<uint64_t>(groups) * N, K, ldb, BN, BK, 1, true);
  if (r) return 2000 + r;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int ctas = sm_count_mx();
  if (tiles < ctas) ctas = tiles;
  Args ga{tile_group, N, reinterpret_cast<const uint32_t*>(sfa), reinterpret_cast<const uint32_t*>(sfb), sfa_rows, sfb_rows};
  gemm_mx_kernel<<<ctas, THREADS, SMEM_BYTES, stream>>>(ta, tb, reinterpret_cast<__nv_bfloat16*>(D), M, N, K, ldd, ga, err);
  return static_cast<int>(cudaGetLastError());
}
