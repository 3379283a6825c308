// Dense bf16 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer   : cp.async.bulk.tensor tiles of A and B into a 4-stage shared-memory ring
//   warp 1      MMA issuer     : one elected lane issues tcgen05.mma (128x256x16) into one of two TMEM accumulators
//   warps 2..5  epilogue       : tcgen05.ld the finished accumulator, convert, store; overlaps the next tile's MMAs
//
// Operand layouts. "K-major" means the reduction index is contiguous in global memory; "MN-major" means the
// M (for A) or N (for B) index is contiguous. The three combinations cover a linear layer's forward
// (x[M,K], W[N,K]), its input gradient (dY[M,N'] K-major, W[N',K'] MN-major) and its weight gradient (both
// MN-major), so no operand is ever transposed in memory.
//
// Replaces the reference's GEMM template for tcgen05 (src/dew/nn/kernels/gemm.py:84, templates/gemm/mosaic_gpu.py).
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace dewb {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;        // 64 bf16 = 128 bytes = one swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_COLS = BN;           // fp32 columns per accumulator
constexpr int TMEM_COLS = 2 * ACC_COLS;  // 512: both accumulators
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

enum Epilogue : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_BF16_ACC = 3 };

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Grouped operation (mixture-of-experts): rows of A are sorted by group and every group's row range starts on a
// multiple of 128 (padding rows are zero), so an output tile never straddles two groups and a reduction tail never
// reads another group's rows.
//   mode 0  dense
//   mode 1  grouped rows      D[rows of g] = A[rows of g] * B_g^T   (forward and input gradient); B stacks the
//           groups along its row dimension, `b_rows_per_group` rows each; `tile_group[m_tile]` names the group of
//           each 128-row tile (< 0: the tile holds no rows)
//   mode 2  grouped reduction D_g = A[rows of g]^T-style product over the rows of g (weight gradient); the reduction
//           runs over rows [group_offsets[g], group_offsets[g+1]) and D stacks the groups, `d_group_stride` apart
struct GroupArgs {
  const int* tile_group;
  const int* group_offsets;
  int mode;
  int b_rows_per_group;
  int groups;
  long long d_group_stride;
  const float* row_scale;   // fp8: per-row scale of A (length M), or null
  const float* col_scale;   // fp8: per-row scale of the stacked B operand (indexed by B's row), or null
  const __nv_bfloat16* bias; // one value per output column added after the scale (dense mode), or null
};

struct Tile {
  int m0, n0;        // output tile origin (within the group for mode 2)
  int b_row0;        // row offset added to B's stacked-row coordinate (mode 1)
  int k_begin;       // first reduction index
  int k_iters;       // reduction steps of BK
  long long d_off;   // element offset of the group's output (mode 2)
  bool skip;         // nothing to compute and nothing to store
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

__device__ __forceinline__ Tile decode_tile(int t, int tiles_m, int tiles_n, int K, const GroupArgs& ga, int bk = BK) {
  Tile ti;
  int m_blk, n_blk;
  ti.b_row0 = 0; ti.k_begin = 0; ti.k_iters = (K + bk - 1) / bk; ti.d_off = 0; ti.skip = false;
  if (ga.mode == 2) {
    const int per = tiles_m * tiles_n;
    const int g = t / per;
    tile_coords(t - g * per, tiles_m, tiles_n, m_blk, n_blk);
    const int r0 = ga.group_offsets[g], r1 = ga.group_offsets[g + 1];
    ti.k_begin = r0;
    ti.k_iters = (r1 - r0 + BK - 1) / BK;
    ti.d_off = static_cast<long long>(g) * ga.d_group_stride;
  } else {
    tile_coords(t, tiles_m, tiles_n, m_blk, n_blk);
    if (ga.mode == 1) {
      const int g = ga.tile_group[m_blk];
      ti.skip = g < 0;
      ti.b_row0 = (g < 0 ? 0 : g) * ga.b_rows_per_group;
    }
  }
  ti.m0 = m_blk * BM;
  ti.n0 = n_blk * BN;
  return ti;
}

// FP8 = true: operands are e4m3 bytes (K-major only), 128 elements per 128-byte swizzle row, tcgen05 kind::f8f6f4
// with K = 32 per instruction; the epilogue applies the row-wise scales of both operands.
template <bool A_MN, bool B_MN, int EPI, bool FP8 = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Dptr, int M, int N, int K, long long ldd, float alpha, const GroupArgs ga,
                 int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  {
    // An earlier launch reported a timed-out wait: leave at once instead of queueing more waits behind it. One
    // thread reads the status so the whole CTA takes the same branch.
    __shared__ int poisoned;
    if (threadIdx.x == 0) poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (poisoned != 0) return;
  }
  // 1024-byte alignment: required by the 128-byte swizzle atoms the descriptors assume (base_offset = 0)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * (ga.mode == 2 ? ga.groups : 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 4); }
    sh->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_a); tma_prefetch_desc(&tma_b); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile ti = decode_tile(t, tiles_m, tiles_n, K, ga, FP8 ? 2 * BK : BK);
        if (ti.skip || ti.k_iters == 0) continue;
        const int m0 = ti.m0, n0 = ti.n0;
        for (int k = 0; k < ti.k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
          const int k0 = ti.k_begin + k * (FP8 ? 2 * BK : BK);
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, &sh->full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tma_a, &sh->full[stage], m0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &sh->full[stage], k0, ti.b_row0 + n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tma_b, &sh->full[stage], n0 + j * 64, ti.b_row0 + k0);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Give the copies already in flight a bounded chance to land before shared memory is released.
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
      constexpr uint32_t idesc = FP8 ? make_idesc(BM, BN, 0, 0, 0, 0) : make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile ti = decode_tile(t, tiles_m, tiles_n, K, ga, FP8 ? 2 * BK : BK);
        if (ti.skip || ti.k_iters == 0) continue;
        const int k_iters = ti.k_iters;
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
            if (FP8) umma_f8_ss(d_tmem, da, db, idesc, (k > 0 || kk > 0) ? 1u : 0u);
            else umma_bf16_ss(d_tmem, da, db, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&sh->empty[stage]);   // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&sh->tmem_full[acc]);   // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile ti = decode_tile(t, tiles_m, tiles_n, K, ga, FP8 ? 2 * BK : BK);
      if (ti.skip) continue;
      const int row = ti.m0 + q * 32 + lane;
      const int n0 = ti.n0;
      if (ti.k_iters == 0) {
        // an empty group: its product is zero (nothing to add when accumulating)
        if ((EPI == EPI_BF16 || EPI == EPI_F32) && row < M) {
          for (int c = 0; c < BN && n0 + c < N; ++c) {
            if (EPI == EPI_BF16) reinterpret_cast<__nv_bfloat16*>(Dptr)[ti.d_off + static_cast<long long>(row) * ldd + n0 + c] = __float2bfloat16(0.f);
            else reinterpret_cast<float*>(Dptr)[ti.d_off + static_cast<long long>(row) * ldd + n0 + c] = 0.f;
          }
        }
        continue;
      }
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_TMEM_FULL); ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (FP8 && row < M && col < N) {
          const float rs = ga.row_scale != nullptr ? ga.row_scale[row] : 1.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float cs = (ga.col_scale != nullptr && col + i < N) ? ga.col_scale[ti.b_row0 + col + i] : 1.f;
            r[i] = __float_as_uint(__uint_as_float(r[i]) * rs * cs);
          }
        }
        float al = alpha;
        if (ga.bias != nullptr && row < M && col < N) {
          // scale, then the bias: the stores below see the finished values
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col + i < N) r[i] = __float_as_uint(alpha * __uint_as_float(r[i]) + __bfloat162float(ga.bias[col + i]));
          al = 1.f;
        }
        if (row < M && col < N) {
          const bool full = (col + 32 <= N);
          if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(Dptr) + ti.d_off + static_cast<long long>(row) * ldd + col;
            if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
              uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = al * __uint_as_float(r[j * 8 + i]);
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
                  float v = al * __uint_as_float(r[i]);
                  if (EPI == EPI_BF16_ACC) v += __bfloat162float(out[i]);
                  out[i] = __float2bfloat16(v);
                }
              }
            }
          } else {
            float* out = reinterpret_cast<float*>(Dptr) + ti.d_off + static_cast<long long>(row) * ldd + col;
            if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
              float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(al * __uint_as_float(r[j * 4 + 0]), al * __uint_as_float(r[j * 4 + 1]),
                                       al * __uint_as_float(r[j * 4 + 2]), al * __uint_as_float(r[j * 4 + 3]));
                if (EPI == EPI_F32_ACC) { const float4 o = o4[j]; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
                o4[j] = v;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (col + i < N) {
                  float v = al * __uint_as_float(r[i]);
                  if (EPI == EPI_F32_ACC) v += out[i];
                  out[i] = v;
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, void* D, int M, int N, int K, long long ldd,
                      float alpha, const GroupArgs& ga, int* err, int sms, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, EPI>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (ga.mode == 2 ? ga.groups : 1);
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, D, M, N, K, ldd, alpha, ga, err);
  return static_cast<int>(cudaGetLastError());
}

template <bool A_MN, bool B_MN>
static int launch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, void* D, int M, int N, int K,
                      long long ldd, float alpha, const GroupArgs& ga, int* err, int sms, cudaStream_t stream) {
  switch (epi) {
    case EPI_BF16: return launch_one<A_MN, B_MN, EPI_BF16>(ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
    case EPI_F32: return launch_one<A_MN, B_MN, EPI_F32>(ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
    case EPI_F32_ACC: return launch_one<A_MN, B_MN, EPI_F32_ACC>(ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
    case EPI_BF16_ACC: return launch_one<A_MN, B_MN, EPI_BF16_ACC>(ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
  }
  return -2;
}

static int launch_fp8(const CUtensorMap& ta, const CUtensorMap& tb, void* D, int M, int N, int K, long long ldd, float alpha,
                      const GroupArgs& ga, int* err, int sms, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<false, false, EPI_BF16, true>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, D, M, N, K, ldd, alpha, ga, err);
  return static_cast<int>(cudaGetLastError());
}

static int dispatch(int a_mn, int b_mn, int epi, const CUtensorMap& ta, const CUtensorMap& tb, void* D, int M, int N,
                    int K, long long ldd, float alpha, const GroupArgs& ga, int* err, int sms, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_epi<false, false>(epi, ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
  if (!a_mn && b_mn) return launch_epi<false, true>(epi, ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
  if (a_mn && !b_mn) return launch_epi<true, false>(epi, ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
  return launch_epi<true, true>(epi, ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
}

}  // namespace gemm
}  // namespace dewb

static int g_sm_count[64];

static int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

// host-side: the bias row of the call in flight on this thread (set by the `_bias` entry point around the common launcher)
static thread_local const __nv_bfloat16* g_dense_bias = nullptr;

// D[M,N] (ldd) = alpha * op(A) * op(B)^T.
//   a_mn = 0: A is [M, K] row-major with row stride lda;  a_mn = 1: A is stored as [K, M] row-major (lda = row stride)
//   b_mn = 0: B is [N, K] row-major with row stride ldb;  b_mn = 1: B is stored as [K, N] row-major
//   epi: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (D += ...), 3 bf16 accumulate
// All row strides must be multiples of 8 elements and base pointers 16-byte aligned (TMA rules).
// `err` is a device int the kernel sets to a non-zero code if one of its bounded waits gave up.
// `max_ctas` > 0 caps the persistent grid (used to leave SMs to a concurrent communication kernel).
extern "C" int dewb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                              long long ldd, int a_mn, int b_mn, int epi, float alpha, int* err, int max_ctas,
                              void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  else       r = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2, true);
  if (r) return 1000 + r;
  if (!b_mn) r = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2, true);
  else       r = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2, true);
  if (r) return 2000 + r;
  int sms = sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  GroupArgs ga{nullptr, nullptr, 0, 0, 1, 0, nullptr, nullptr, g_dense_bias};
  return dispatch(a_mn, b_mn, epi, ta, tb, D, M, N, K, ldd, alpha, ga, err, sms, stream);
}

// The same product with a bias row (bf16 [N]) added in the epilogue: D = alpha * op(A) op(B)^T + bias.
extern "C" int dewb_gemm_bf16_bias(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                                   long long ldb, long long ldd, int a_mn, int b_mn, int epi, float alpha, int* err, int max_ctas,
                                   void* stream_ptr) {
  g_dense_bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  const int rc = dewb_gemm_bf16(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, epi, alpha, err, max_ctas, stream_ptr);
  g_dense_bias = nullptr;
  return rc;
}

// Grouped rows (mixture-of-experts forward and input gradient):
//   D[M, N] rows of group g = A[rows of g, K] * B_g^T, with B the groups stacked along rows:
//     b_mn = 0: B is [G * N, K] (each group [N, K], K contiguous)     - forward with weights [G, N, K]
//     b_mn = 1: B is [G * K, N] (each group [K, N], N contiguous)     - input gradient with weights [G, K(red), N]
//   tile_group[ceil(M / 128)]: group id of each 128-row tile of A (group row ranges start on multiples of 128)
extern "C" int dewb_gmm_bf16(const void* A, const void* B, void* D, const int* tile_group, int M, int N, int K,
                             int groups, long long lda, long long ldb, long long ldd, int b_mn, int epi, float alpha,
                             int* err, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (b_mn && (K % BK)) return -4;      // a reduction tail would read the next group's rows
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  if (r) return 1000 + r;
  if (!b_mn) r = make_tmap_2d(&tb, B, static_cast<uint64_t>(groups) * N, K, ldb, BN, BK, 2, true);
  else       r = make_tmap_2d(&tb, B, static_cast<uint64_t>(groups) * K, N, ldb, BK, 64, 2, true);
  if (r) return 2000 + r;
  GroupArgs ga{tile_group, nullptr, 1, b_mn ? K : N, groups, 0, nullptr, nullptr, nullptr};
  return dispatch(0, b_mn, epi, ta, tb, D, M, N, K, ldd, alpha, ga, err, sm_count(), stream);
}

// Grouped reduction (mixture-of-experts weight gradient): for every group g,
//   D_g[M, N] (+)= A[rows of g, M]^T * B[rows of g, N]   with A stored [R, M] and B stored [R, N] (R = all rows),
//   rows of g = [group_offsets[g], group_offsets[g + 1]) (multiples of 64; padding rows are zero)
//   D stacks the groups: D_g = D + g * d_group_stride, row stride ldd.
extern "C" int dewb_tgmm_bf16(const void* A, const void* B, void* D, const int* group_offsets, int R, int M, int N,
                              int groups, long long lda, long long ldb, long long ldd, long long d_group_stride, int epi,
                              float alpha, int* err, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm;
  if (R <= 0 || M <= 0 || N <= 0 || groups <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, R, M, lda, BK, 64, 2, true);
  if (r) return 1000 + r;
  r = make_tmap_2d(&tb, B, R, N, ldb, BK, 64, 2, true);
  if (r) return 2000 + r;
  GroupArgs ga{nullptr, group_offsets, 2, 0, groups, d_group_stride, nullptr, nullptr, nullptr};
  return dispatch(1, 1, epi, ta, tb, D, M, N, R, ldd, alpha, ga, err, sm_count(), stream);
}

// Row-wise scaled fp8 (e4m3) GEMM, dense or grouped rows: D[M,N] (bf16) = (A_q * a_scale[row]) * (B_q * b_scale[row of B])^T.
//   A_q [M, K] and B_q [groups * N, K] are e4m3 bytes, K contiguous, K a multiple of 16; scales are fp32.
//   tile_group: null for a dense product (groups = 1), else the group of each 128-row tile of A as in dewb_gmm_bf16.
extern "C" int dewb_gemm_fp8(const void* A, const void* B, void* D, const float* a_scale, const float* b_scale,
                             const int* tile_group, int M, int N, int K, int groups, long long lda, long long ldb,
                             long long ldd, int* err, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, M, K, lda, BM, 2 * BK, 1, true);
  if (r) return 1000 + r;
  r = make_tmap_2d(&tb, B, static_cast<uint64_t>(groups) * N, K, ldb, BN, 2 * BK, 1, true);
  if (r) return 2000 + r;
  GroupArgs ga{tile_group, nullptr, tile_group != nullptr ? 1 : 0, N, groups, 0, a_scale, b_scale, nullptr};
  return launch_fp8(ta, tb, D, M, N, K, ldd, 1.f, ga, err, sm_count(), stream);
}
