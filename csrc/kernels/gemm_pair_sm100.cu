// Dense bf16 GEMM for sm_100a on CTA pairs: D[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory.
//
// Two CTAs on neighbouring SMs (a thread-block cluster of 2) compute one 256 x 256 output tile with tcgen05.mma
// cta_group::2. Each CTA stages 128 rows of A and 128 rows of B per reduction step (32 KiB instead of the 48 KiB a
// lone CTA needs for a 128 x 256 tile), so the shared-memory fill rate per FLOP drops by a third - the limiter the
// single-CTA kernel's counters showed (L2 -> SM operand delivery). Each CTA keeps its 128 x 256 half of the
// accumulator in its own tensor memory and runs its own epilogue.
//
//   warp 0      TMA producer (both CTAs): own halves of A and B into a 6-stage ring; the byte counts of both CTAs are
//               credited to the leader CTA's "full" barrier (no multicast: every load lands in the issuing CTA only)
//   warp 1      MMA issuer (leader CTA only): tcgen05.mma.cta_group::2 256x256x16; tcgen05.commit to the "empty"
//               barrier of BOTH CTAs frees a stage; commit to both CTAs' "accumulator full" barriers ends a tile
//   warps 2..5  epilogue (both CTAs): tcgen05.ld the CTA's own accumulator half, convert, store; the leader's MMA
//               warp learns from both CTAs' epilogues (remote mbarrier arrive) that an accumulator is free again
//
// Operand layouts as in the single-CTA kernel (K-major or MN-major per operand), so forward, input gradient and weight
// gradient of a linear layer read their operands in place.
//
// Replaces the reference's paired ("PAIRED" topology, 2-CTA UMMA 256x256) GEMM bundle
// (src/dew/nn/kernels/templates/mosaic_sm100.py:1-220).
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include <cstdlib>

namespace dewb {
namespace gemm_pair {

constexpr int BM = 128;          // accumulator rows per CTA (pair tile: 256)
constexpr int PAIR_M = 256;
constexpr int BN = 256;          // pair tile columns
constexpr int HALF_N = BN / 2;   // rows of B staged by each CTA
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = HALF_N * BK * 2;    // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_COLS = BN;
constexpr int TMEM_COLS = 2 * ACC_COLS;     // both accumulators
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

enum Epilogue : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_BF16_ACC = 3 };

struct Shared {
  uint64_t full[STAGES];       // used in the leader: both CTAs' loads of a stage have landed
  uint64_t empty[STAGES];      // in each CTA: the pair MMAs that read the stage have completed
  uint64_t tmem_full[2];       // in each CTA: the accumulator is complete
  uint64_t tmem_empty[2];      // used in the leader: both CTAs' epilogues have drained the accumulator (8 warps)
  uint32_t tmem_base;
  int abort_flag;
  int poisoned;
};

// `group_m` row blocks (of 256 rows) share their B tiles in L2 before the walk moves along N: the A rows of a group stay
// resident while B streams past once per group.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& m_blk, int& n_blk) {
  const int per_group = group_m * tiles_n;
  const int group = t / per_group;
  const int first_m = group * group_m;
  const int gsize = min(tiles_m - first_m, group_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

template <int EPI>
__device__ __forceinline__ void store_chunk(const uint32_t (&r_in)[32], void* Dptr, int row, int col, int N, long long ldd,
                                            float alpha_in, const __nv_bfloat16* __restrict__ bias) {
  const bool full = (col + 32 <= N);
  // scale, then the bias (one bf16 value per output column); the stores below see the finished values
  uint32_t r[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float v = alpha_in * __uint_as_float(r_in[i]);
    if (bias != nullptr && col + i < N) v += __bfloat162float(bias[col + i]);
    r[i] = __float_as_uint(v);
  }
  constexpr float alpha = 1.f;
  if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(Dptr) + static_cast<long long>(row) * ldd + col;
    if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
      uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = alpha * __uint_as_float(r[j * 8 + i]);
        if (EPI == EPI_BF16_ACC) {
          const uint4 old = o4[j];
          v[0] += bf16_lo(old.x); v[1] += bf16_hi(old.x); v[2] += bf16_lo(old.y); v[3] += bf16_hi(old.y);
          v[4] += bf16_lo(old.z); v[5] += bf16_hi(old.z); v[6] += bf16_lo(old.w); v[7] += bf16_hi(old.w);
        }
        uint4 pk;
        pk.x = pack_bf16(v[0], v[1]); pk.y = pack_bf16(v[2], v[3]);
        pk.z = pack_bf16(v[4], v[5]); pk.w = pack_bf16(v[6], v[7]);
        o4[j] = pk;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i < N) {
          float v = alpha * __uint_as_float(r[i]);
          if (EPI == EPI_BF16_ACC) v += __bfloat162float(out[i]);
          out[i] = __float2bfloat16(v);
        }
      }
    }
  } else {
    float* out = reinterpret_cast<float*>(Dptr) + static_cast<long long>(row) * ldd + col;
    if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
      float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v = make_float4(alpha * __uint_as_float(r[j * 4 + 0]), alpha * __uint_as_float(r[j * 4 + 1]),
                               alpha * __uint_as_float(r[j * 4 + 2]), alpha * __uint_as_float(r[j * 4 + 3]));
        if (EPI == EPI_F32_ACC) { const float4 o = o4[j]; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
        o4[j] = v;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i < N) {
          float v = alpha * __uint_as_float(r[i]);
          if (EPI == EPI_F32_ACC) v += out[i];
          out[i] = v;
        }
      }
    }
  }
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Dptr, int M, int N, int K, long long ldd, float alpha, int group_m,
                 const __nv_bfloat16* __restrict__ bias,
                 int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms the descriptors assume. The dynamic shared memory
  // starts at the same offset in both CTAs, so the aligned layout is identical in both (the pair MMA addresses the
  // two CTAs' operands by one shared-memory offset).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const uint32_t leader = 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + PAIR_M - 1) / PAIR_M;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_iters = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 8); }
    sh->abort_flag = 0;
    // an earlier launch reported a timed-out wait: do no work (decided for the pair as a whole, below)
    sh->poisoned = *reinterpret_cast<volatile int*>(err);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_a); tma_prefetch_desc(&tma_b); }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();            // both CTAs' barriers exist before either CTA's copies or commits can reach them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  const bool poisoned = (sh->poisoned | ld_remote_s32(map_to_cta(smem_u32(&sh->poisoned), rank ^ 1))) != 0;

  if (poisoned) {
    // fall through to the teardown: the pair leaves together
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m_blk, n_blk;
        tile_coords(t, tiles_m, tiles_n, group_m, m_blk, n_blk);
        const int m0 = m_blk * PAIR_M + static_cast<int>(rank) * BM;
        const int n0 = n_blk * BN + static_cast<int>(rank) * HALF_N;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (rank == leader) mbar_expect_tx(&sh->full[stage], 2 * STAGE_BYTES);     // both CTAs' bytes
          const uint32_t full_bar = map_to_cta(smem_u32(&sh->full[stage]), leader);
          const int k0 = k * BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, full_bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tma_a, full_bar, m0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, full_bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < HALF_N / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tma_b, full_bar, n0 + j * 64, k0);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Give the stages still in use a bounded chance to drain before shared memory is released: a stage is
        // drained when its "empty" barrier completes (the MMAs that read it are done), which implies its copies landed.
        const long long pending = issued < STAGES ? issued : STAGES;
        for (long long i = 0; i < pending; ++i) {
          int s = static_cast<int>((issued - 1 - i) % STAGES);
          uint32_t ph = static_cast<uint32_t>(((issued - 1 - i) / STAGES) & 1);
          mbar_wait(&sh->empty[s], ph, nullptr, 20000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(PAIR_M, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      const uint32_t peer = rank ^ 1;
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_TMEM_EMPTY); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_sdesc_sw128(sa + kk * 2048, 8192, 1024) : make_sdesc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_sdesc_sw128(sb + kk * 2048, 8192, 1024) : make_sdesc_sw128(sb + kk * 32, 16, 1024);
            umma_bf16_ss_pair(d_tmem, da, db, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          // frees the stage in both CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&sh->empty[stage]));
          umma_commit_pair(map_to_cta(smem_u32(&sh->empty[stage]), peer));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&sh->tmem_full[acc]));                         // accumulator complete, both halves
        umma_commit_pair(map_to_cta(smem_u32(&sh->tmem_full[acc]), peer));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      int m_blk, n_blk;
      tile_coords(t, tiles_m, tiles_n, group_m, m_blk, n_blk);
      const int row = m_blk * PAIR_M + static_cast<int>(rank) * BM + q * 32 + lane;
      const int n0 = n_blk * BN;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) store_chunk<EPI>(r, Dptr, row, col, N, ldd, alpha, bias);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&sh->tmem_empty[acc]), leader));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ------------------------------------------------------------------ teardown
  // Neither CTA may exit, nor tensor memory be freed, while the other's MMAs, commits or remote arrives can still
  // reach it: the pair meets at a cluster barrier first.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, void* D, int M, int N, int K, long long ldd,
                      float alpha, int* err, int max_pairs, cudaStream_t stream, const __nv_bfloat16* bias = nullptr) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, EPI>;
  static int resident[64] = {};          // co-resident clusters of this instantiation per device (0 = not asked yet)
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -5;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (resident[dev] == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    cfg.gridDim = dim3(static_cast<unsigned>(sms), 1, 1);
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
    if (e != cudaSuccess || clusters <= 0) { cudaGetLastError(); return -6; }   // pairs cannot be placed: caller falls back
    resident[dev] = clusters;
  }
  int pairs = resident[dev];
  if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
  const int tiles = ((M + PAIR_M - 1) / PAIR_M) * ((N + BN - 1) / BN);
  if (tiles < pairs) pairs = tiles;
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  // Measured on the layer shapes (gate|up forward, 8192 / 16384 x 28672 x 4096): 16 row blocks per group are 5 % faster than 4
  // (B streams from DRAM once per group); with a deep reduction (K >= 14336) 8 is as good and keeps the A rows of a group in L2.
  static int forced_group_m = -1;
  if (forced_group_m < 0) {
    const char* env = getenv("DEWB_PAIR_GROUP_M");
    forced_group_m = env != nullptr ? atoi(env) : 0;
  }
  int group_m = forced_group_m;
  if (group_m <= 0) {
    group_m = K <= 8192 ? 16 : 8;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, D, M, N, K, ldd, alpha, group_m, bias, err);
  return static_cast<int>(e);
}

template <bool A_MN, bool B_MN>
static int launch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, void* D, int M, int N, int K,
                      long long ldd, float alpha, int* err, int max_pairs, cudaStream_t stream, const __nv_bfloat16* bias = nullptr) {
  switch (epi) {
    case EPI_BF16: return launch_one<A_MN, B_MN, EPI_BF16>(ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
    case EPI_F32: return launch_one<A_MN, B_MN, EPI_F32>(ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
    case EPI_F32_ACC: return launch_one<A_MN, B_MN, EPI_F32_ACC>(ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
    case EPI_BF16_ACC: return launch_one<A_MN, B_MN, EPI_BF16_ACC>(ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
  }
  return -2;
}

}  // namespace gemm_pair
}  // namespace dewb

// host-side: the bias row of the call in flight on this thread (set by the `_bias` entry point around the common launcher)
static thread_local const __nv_bfloat16* g_pair_bias = nullptr;

// Same contract as dewb_gemm_bf16 (D[M,N] = alpha * op(A) * op(B)^T, operand layouts a_mn / b_mn, epilogues 0..3),
// computed by CTA pairs. `max_ctas` > 0 caps the grid (pairs = max_ctas / 2). Returns -6 if the device cannot place
// clusters of two CTAs of this kernel.
extern "C" int dewb_gemm_pair_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                   long long ldb, long long ldd, int a_mn, int b_mn, int epi, float alpha, int* err,
                                   int max_ctas, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm_pair;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  else       r = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2, true);
  if (r) return 1000 + r;
  if (!b_mn) r = make_tmap_2d(&tb, B, N, K, ldb, HALF_N, BK, 2, true);
  else       r = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2, true);
  if (r) return 2000 + r;
  const int max_pairs = max_ctas > 0 ? (max_ctas / 2 > 0 ? max_ctas / 2 : 1) : 0;
  const __nv_bfloat16* bias = g_pair_bias;
  if (!a_mn && !b_mn) return launch_epi<false, false>(epi, ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
  if (!a_mn && b_mn) return launch_epi<false, true>(epi, ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
  if (a_mn && !b_mn) return launch_epi<true, false>(epi, ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
  return launch_epi<true, true>(epi, ta, tb, D, M, N, K, ldd, alpha, err, max_pairs, stream, bias);
}

// The same product with a bias row (bf16 [N]) added in the epilogue: D = alpha * op(A) op(B)^T + bias.
extern "C" int dewb_gemm_pair_bf16_bias(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                                        long long ldb, long long ldd, int a_mn, int b_mn, int epi, float alpha, int* err,
                                        int max_ctas, void* stream_ptr) {
  g_pair_bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  const int rc = dewb_gemm_pair_bf16(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, epi, alpha, err, max_ctas, stream_ptr);
  g_pair_bias = nullptr;
  return rc;
}
