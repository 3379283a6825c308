// Weight-streaming GEMM for the decode step: C[M <= 128, N] = X[M, K] W[N, K]^T in bf16 with fp32 accumulation, where the
// activations are a handful of rows and the time goes into reading W once.
//
//   * One CTA owns 128 rows of W (an output tile 128 x 128 whose M rows are the batch rows; rows beyond M are zero-filled by
//     TMA) and a slice of K; `split` CTAs that share a tile form a thread-block cluster, so a product with few tiles still
//     streams W from every SM.  Each CTA runs the usual ring: TMA (no multicast) -> tcgen05.mma (cta_group::1, accumulator
//     in tensor memory) -> tcgen05.ld.
//   * The K slices are summed inside the cluster over distributed shared memory: every CTA parks its 128 x 128 fp32 partial in
//     its own (by then idle) operand ring, and after a cluster barrier each CTA sums one column slice over all the CTAs
//     (`ld.shared::cluster`) and writes that slice of the output.  No global workspace, no second kernel, a fixed summation
//     order (bitwise repeatable).
//   * SwiGLU mode: W is the packed gate | up projection ([2 F, K]); the tile takes 64 gate rows and the matching 64 up rows,
//     so one thread holds gate and up of the same output element and writes silu(gate) * up: the activation kernel and its pass
//     over HBM disappear.
//   * Launched with programmatic dependent launch: the weight tiles of the first ring stages are requested BEFORE
//     `griddepcontrol.wait` (they do not depend on the previous kernel), the activation tiles after it.
// Every wait is bounded (status word); the two cluster barriers are reached on every path.
//
// Capability parity: the skinny / split-K cells of the reference's GEMM selector (src/dew/nn/kernels/gemm.py:84,
// templates/gemm/mosaic_gpu.py) and its fused SwiGLU epilogue (src/dew/nn/kernels/fused_gemm.py).
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace dewb {
namespace skinny {

constexpr int BM = 128;               // batch rows (MMA M)
constexpr int BN = 128;               // rows of W per tile (MMA N)
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int X_BYTES = BM * BK * 2;  // 16 KiB
constexpr int W_BYTES = BN * BK * 2;  // 16 KiB
constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
constexpr int THREADS = 192;          // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int PARK_LD = BN + 4;       // fp32 row stride of the parked partial (bank-conflict-free 16-byte accesses)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
static_assert(BM * PARK_LD * 4 <= STAGES * STAGE_BYTES, "the parked partial must fit the operand ring");

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
  int dead;
};

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }


__device__ __forceinline__ void store4(__nv_bfloat16* o, int col, int N, const float (&a)[4]) {
  if (col + 4 <= N && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {
    uint2 pk;
    pk.x = pack_bf16(a[0], a[1]); pk.y = pack_bf16(a[2], a[3]);
    *reinterpret_cast<uint2*>(o) = pk;
  } else {
    for (int i = 0; i < 4; ++i)
      if (col + i < N) o[i] = __float2bfloat16(a[i]);
  }
}

// Part 2 of the epilogue: this CTA's column slice of the tile, summed over the SPLIT parked partials of the cluster.  Eight
// 16-byte loads over distributed shared memory are in flight per thread before any is used (one round trip per batch, not per load).
template <int SPLIT>
__device__ __forceinline__ void reduce_slices(uint32_t park_addr, __nv_bfloat16* __restrict__ out, int row, int M, int N, long long ldo,
                                              int tile, int crank, int mode) {
  constexpr int GROUPS = 8 / SPLIT;                              // 4-column groups summed per batch
  uint32_t peer[SPLIT];
#pragma unroll
  for (int s = 0; s < SPLIT; ++s) peer[s] = map_to_cta(park_addr, s);
  if (mode == 0) {
    constexpr int W = BN / SPLIT;                                // columns of this CTA's slice
    const int c0 = crank * W;
#pragma unroll 1
    for (int cc = 0; cc < W; cc += 4 * GROUPS) {
      float4 v[GROUPS][SPLIT];
#pragma unroll
      for (int g = 0; g < GROUPS; ++g)
#pragma unroll
        for (int s = 0; s < SPLIT; ++s) v[g][s] = ld_cluster_f4(peer[s] + (row * PARK_LD + c0 + cc + 4 * g) * 4);
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < SPLIT; ++s) { a[0] += v[g][s].x; a[1] += v[g][s].y; a[2] += v[g][s].z; a[3] += v[g][s].w; }
        const int col = tile * 128 + c0 + cc + 4 * g;
        if (row < M) store4(out + static_cast<long long>(row) * ldo + col, col, N, a);
      }
    }
  } else {
    constexpr int W = 64 / SPLIT;                                // output columns of this CTA's slice
    constexpr int G2 = GROUPS > 1 ? GROUPS / 2 : 1;              // gate and up double the loads per group
    const int c0 = crank * W;
#pragma unroll 1
    for (int cc = 0; cc < W; cc += 4 * G2) {
      float4 gv[G2][SPLIT], uv[G2][SPLIT];
#pragma unroll
      for (int g = 0; g < G2; ++g)
#pragma unroll
        for (int s = 0; s < SPLIT; ++s) {
          gv[g][s] = ld_cluster_f4(peer[s] + (row * PARK_LD + c0 + cc + 4 * g) * 4);
          uv[g][s] = ld_cluster_f4(peer[s] + (row * PARK_LD + 64 + c0 + cc + 4 * g) * 4);
        }
#pragma unroll
      for (int g = 0; g < G2; ++g) {
        float ga[4] = {0.f, 0.f, 0.f, 0.f}, ua[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < SPLIT; ++s) {
          ga[0] += gv[g][s].x; ga[1] += gv[g][s].y; ga[2] += gv[g][s].z; ga[3] += gv[g][s].w;
          ua[0] += uv[g][s].x; ua[1] += uv[g][s].y; ua[2] += uv[g][s].z; ua[3] += uv[g][s].w;
        }
        const float a[4] = {silu(ga[0]) * ua[0], silu(ga[1]) * ua[1], silu(ga[2]) * ua[2], silu(ga[3]) * ua[3]};
        const int col = tile * 64 + c0 + cc + 4 * g;
        if (row < M) store4(out + static_cast<long long>(row) * ldo + col, col, N, a);
      }
    }
  }
}

// mode 0: out[M, N] = X W^T.  mode 1 (SwiGLU): W = [gate (F rows); up (F rows)], N = F, out[M, F] = silu(X gate^T) * (X up^T).
__global__ void __launch_bounds__(THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                   __nv_bfloat16* __restrict__ out, int M, int N, int K, long long ldo, int split, int mode, int pdl,
                   int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int crank = split > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int tile = blockIdx.x / split;
  // this CTA's K steps
  const int steps = (K + BK - 1) / BK;
  const int chunk = (steps + split - 1) / split;
  const int k_first = crank * chunk;
  const int k_iters = max(0, min(steps, k_first + chunk) - k_first);
  // rows of W of this tile: two boxes of 64 rows
  const int w_row0 = mode == 1 ? tile * 64 : tile * 128;
  const int w_row1 = mode == 1 ? N + tile * 64 : tile * 128 + 64;

  if (threadIdx.x == 0) {
    // every CTA of the cluster must take the same path through the cluster barriers, whatever the status word says
    sh->dead = *reinterpret_cast<volatile int*>(err) != 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    mbar_init(&sh->acc_full, 1);
    sh->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, BN);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_x); tma_prefetch_desc(&tma_w); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  const bool dead = sh->dead != 0;

  if (!dead && k_iters > 0) {
    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        // weights first: they do not depend on the kernel in front of this one
        const int ahead = min(k_iters, STAGES);
        for (int k = 0; k < ahead; ++k) {
          uint8_t* sw = smem + k * STAGE_BYTES + X_BYTES;
          mbar_expect_tx(&sh->full[k], STAGE_BYTES);
          tma_load_2d(sw, &tma_w, &sh->full[k], (k_first + k) * BK, w_row0);
          tma_load_2d(sw + 8192, &tma_w, &sh->full[k], (k_first + k) * BK, w_row1);
        }
        if (pdl) griddep_wait();
        for (int k = 0; k < ahead; ++k) tma_load_2d(smem + k * STAGE_BYTES, &tma_x, &sh->full[k], (k_first + k) * BK, 0);
        int stage = ahead == STAGES ? 0 : ahead;
        uint32_t phase = ahead == STAGES ? 1 : 0;
        for (int k = ahead; k < k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); break; }
          uint8_t* sx = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
          tma_load_2d(sx, &tma_x, &sh->full[stage], (k_first + k) * BK, 0);
          tma_load_2d(sx + X_BYTES, &tma_w, &sh->full[stage], (k_first + k) * BK, w_row0);
          tma_load_2d(sx + X_BYTES + 8192, &tma_w, &sh->full[stage], (k_first + k) * BK, w_row1);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, 0, 0);
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t sx = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sw = sx + X_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            umma_bf16_ss(tmem_base, make_sdesc_sw128(sx + kk * 32, 16, 1024), make_sdesc_sw128(sw + kk * 32, 16, 1024), idesc,
                         (k > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&sh->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&sh->acc_full);
      }
    }
  } else if (!dead && pdl && threadIdx.x == 0) {
    griddep_wait();                    // a kernel launched as a programmatic dependent always executes the wait
  }
  if (dead && pdl && threadIdx.x == 0) griddep_wait();

  // -------------------------------------------------------------------- epilogue, part 1: the partial leaves tensor memory
  float* park = reinterpret_cast<float*>(smem);                    // [128][PARK_LD] fp32 over the (idle) operand ring
  const int q = warp & 3;                                          // tensor-memory lane quarter of an epilogue warp
  const int row = q * 32 + lane;                                   // batch row of this thread
  bool have = false;
  if (!dead && warp >= 2) {
    if (k_iters > 0) {
      have = mbar_wait(&sh->acc_full, 0, abort_flag);
      if (!have) atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
      have = __all_sync(0xffffffffu, have);
    }
    tc_fence_after();
    if (split == 1) {
      // no K split: straight from tensor memory to the output
      if (have) {
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        if (mode == 0) {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_ld_wait();
            const int col = tile * 128 + c * 32;
            if (row < M) {
              __nv_bfloat16* o = out + static_cast<long long>(row) * ldo + col;
              if (col + 32 <= N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 pk;
                  pk.x = pack_bf16(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
                  pk.y = pack_bf16(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
                  pk.z = pack_bf16(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
                  pk.w = pack_bf16(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
                  reinterpret_cast<uint4*>(o)[j] = pk;
                }
              } else {
                for (int i = 0; i < 32; ++i)
                  if (col + i < N) o[i] = __float2bfloat16(__uint_as_float(r[i]));
              }
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t g[32], u[32];
            tmem_ld_32x32b_x32(taddr + c * 32, g);
            tmem_ld_32x32b_x32(taddr + 64 + c * 32, u);
            tmem_ld_wait();
            const int col = tile * 64 + c * 32;
            if (row < M) {
              __nv_bfloat16* o = out + static_cast<long long>(row) * ldo + col;
              for (int i = 0; i < 32; ++i)
                if (col + i < N) o[i] = __float2bfloat16(silu(__uint_as_float(g[i])) * __uint_as_float(u[i]));
            }
          }
        }
      }
    } else {
      // park the partial (zeros when this CTA had no K steps or gave up: the sum stays defined)
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        if (have) {
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        float4* dst = reinterpret_cast<float4*>(park + row * PARK_LD + c * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(__uint_as_float(r[j * 4]), __uint_as_float(r[j * 4 + 1]), __uint_as_float(r[j * 4 + 2]), __uint_as_float(r[j * 4 + 3]));
      }
    }
  }
  if (split > 1) {
    // -------------------------------------------------------------------- part 2: sum the K slices over the cluster
    tc_fence_before();
    cluster_arrive();
    cluster_wait();
    if (!dead && warp >= 2) {
      const uint32_t park_addr = smem_u32(park);
      switch (split) {
        case 2: reduce_slices<2>(park_addr, out, row, M, N, ldo, tile, crank, mode); break;
        case 4: reduce_slices<4>(park_addr, out, row, M, N, ldo, tile, crank, mode); break;
        default: reduce_slices<8>(park_addr, out, row, M, N, ldo, tile, crank, mode); break;
      }
    }
    // nobody leaves while a peer may still read its shared memory
    cluster_arrive();
    cluster_wait();
  }
  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

}  // namespace skinny
}  // namespace dewb

// X [M <= 128, K] (row stride ldx), W [rows, K] (row stride ldw) bf16, K-major.  mode 0: out [M, N] with N = rows of W;
// mode 1: W = [gate; up] of F rows each, N = F, out [M, F] = silu(gate) * up.  split in {1, 2, 4, 8}: CTAs of a cluster that share
// a tile and split K.  pdl != 0: launch as a programmatic dependent of the previous kernel in the stream.
extern "C" int dewb_gemm_skinny_bf16(const void* X, const void* W, void* out, int M, int N, int K, long long ldx, long long ldw,
                                     long long ldo, int split, int mode, int pdl, int* err, void* stream_ptr) {
  using namespace dewb::skinny;
  if (M <= 0 || N <= 0) return 0;
  if (M > BM || K <= 0 || (K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0 || (split != 1 && split != 2 && split != 4 && split != 8) ||
      (mode != 0 && mode != 1) || (mode == 1 && (N % 64) != 0))
    return -3;
  const int w_rows = mode == 1 ? 2 * N : N;
  CUtensorMap tx, tw;
  int r;
  if ((r = dewb::make_tmap_2d(&tx, X, static_cast<uint64_t>(M), static_cast<uint64_t>(K), static_cast<uint64_t>(ldx), BM, BK, 2, true))) return 1000 + r;
  if ((r = dewb::make_tmap_2d(&tw, W, static_cast<uint64_t>(w_rows), static_cast<uint64_t>(K), static_cast<uint64_t>(ldw), 64, BK, 2, true))) return 2000 + r;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -5;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const int tiles = mode == 1 ? N / 64 : (N + 127) / 128;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (split > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = static_cast<unsigned>(split); attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, tx, tw, reinterpret_cast<__nv_bfloat16*>(out), M, N, K, ldo, split, mode,
                                     pdl, err);
  return static_cast<int>(e);
}
