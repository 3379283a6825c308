// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a, bf16, fp32 accumulation).
//
//   all-gather -> GEMM   (column-parallel layer after a sequence-parallel region)
//       D[M, N] = A[M, K] * B[N, K]^T where rank s holds rows [s * M/W, (s+1) * M/W) of A in its symmetric buffer.
//       Nothing is gathered first: the TMA producer reads each A tile straight from the owning rank's memory
//       (cp.async.bulk.tensor through a per-rank tensor map; plain peer loads over NVSwitch, no multicast). Tiles of
//       the local shard go first, so the first products overlap the peers' "my shard is written" flags; the producer
//       waits (bounded) for a peer's flag only before its first load from that peer.
//
//   GEMM -> reduce-scatter   (row-parallel layer before a sequence-parallel region)
//       every rank computes a partial P_r[M, N] = A_r * B_r^T over its slice of K; rank j owns rows
//       [j * M/W, (j+1) * M/W) of the sum. The epilogue stores each finished tile directly into slot `rank` of the
//       owner's symmetric partial buffer (peer st.global), so the transfer rides under the remaining tiles; the last
//       CTA to finish publishes a flag to every peer. `dewb_reduce_partials` on the owner waits for the W flags and
//       sums the W slots (+ optional residual).
//
// Kernel skeleton as the dense kernel: warp 0 TMA producer, warp 1 tcgen05 issuer, warps 2..5 epilogue, 4-stage ring,
// two TMEM accumulators. Every wait is bounded and reports through the status word.
//
// Replaces the XLA-inserted all-gather / reduce-scatter around the Megatron-split projections
// (src/dew/mesh.py:101-146, src/dew/nn/sharding.py:76-99, 262-280).
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace dewb {
namespace gemm_comm {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_COLS = BN, TMEM_COLS = 2 * ACC_COLS;
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int MAX_RANKS = 8;

struct alignas(64) TmaSet { CUtensorMap m[MAX_RANKS]; };
struct Peers { unsigned long long p[MAX_RANKS]; };

struct Shared {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// MODE 0: all-gather -> GEMM (A per rank through `maps`, D local)   MODE 1: GEMM -> reduce-scatter (A local = maps.m[0],
// D scattered to `partials` of the owners)
struct CommArgs {
  int rank, world;
  int tiles_per_shard;           // 128-row tiles per rank's row range
  const uint32_t* my_flags;      // MODE 0: flags peers write into this rank's memory
  Peers flag_ptrs;               // MODE 1: every rank's flag array
  Peers partials;                // MODE 1: every rank's partial buffer [W, M/W, N]
  int slot;
  uint32_t seq;
  unsigned long long limit_ns;
  unsigned int* counter;         // MODE 1: CTAs that have finished (reset by the last one)
};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_comm_kernel(const __grid_constant__ TmaSet maps, const __grid_constant__ CUtensorMap tma_b, void* __restrict__ Dptr,
                 int M, int N, int K, long long ldd, const CommArgs ca, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  {
    __shared__ int poisoned;
    if (threadIdx.x == 0) poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (poisoned != 0) return;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_iters = (K + BK - 1) / BK;
  // Tile t -> (row block, column block): row blocks rotate so that rank r starts with shard r (MODE 0: its own rows
  // need no flag; MODE 1: with shard r + 1, so that the W ranks store to W different owners at any moment).
  const int first_shard = MODE == 0 ? ca.rank : (ca.rank + 1) % ca.world;
  auto tile_of = [&](int t, int& m_blk, int& n_blk) {
    const int mr = t / tiles_n;                       // rotated row-block index
    n_blk = t - mr * tiles_n;
    m_blk = (mr + first_shard * ca.tiles_per_shard) % tiles_m;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 4); }
    sh->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) { tmem_alloc(&sh->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      uint32_t ready = 1u << ca.rank;                 // ranks whose shard is known to be written
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_of(t, m_blk, n_blk);
        const int src = MODE == 0 ? m_blk / ca.tiles_per_shard : 0;
        const int m0 = MODE == 0 ? (m_blk - src * ca.tiles_per_shard) * BM : m_blk * BM;
        if (MODE == 0 && !((ready >> src) & 1u)) {
          // bounded wait for "rank src has written its shard", then order the peer reads of the async proxy after it
          const uint32_t* f = ca.my_flags + ca.slot * ca.world + src;
          const uint64_t t0 = globaltimer_ns();
          while (static_cast<int32_t>(ld_acquire_sys(f) - ca.seq) < 0) {
            if (*abort_flag != 0 || globaltimer_ns() - t0 > ca.limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); *abort_flag = 1; ok = false; break; }
            __nanosleep(64);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
          ready |= 1u << src;
        }
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
          tma_load_2d(sa, &maps.m[src], &sh->full[stage], k * BK, m0);
          tma_load_2d(sa + A_BYTES, &tma_b, &sh->full[stage], k * BK, n_blk * BN);
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
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_TMEM_EMPTY); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            umma_bf16_ss(d_tmem, make_sdesc_sw128(sa + kk * 32, 16, 1024), make_sdesc_sw128(sb + kk * 32, 16, 1024), idesc,
                         (k > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&sh->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&sh->tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int q = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m_blk, n_blk;
      tile_of(t, m_blk, n_blk);
      const int row = m_blk * BM + q * 32 + lane;
      const int n0 = n_blk * BN;
      __nv_bfloat16* base;
      long long out_row;
      if (MODE == 0) {
        base = reinterpret_cast<__nv_bfloat16*>(Dptr);
        out_row = row;
      } else {
        // the owner's partial buffer, slot `rank`: [W, rows_per_shard, N]
        const int owner = m_blk / ca.tiles_per_shard;
        const long long rows_per_shard = static_cast<long long>(ca.tiles_per_shard) * BM;
        base = reinterpret_cast<__nv_bfloat16*>(ca.partials.p[owner]) + static_cast<long long>(ca.rank) * rows_per_shard * ldd;
        out_row = row - owner * rows_per_shard;
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
        if (row < M && col < N) {
          __nv_bfloat16* out = base + out_row * ldd + col;
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
    if (MODE == 1) {
      // every store of this CTA (many of them to peers) is visible system-wide before the CTA counts itself done
      __threadfence_system();
      named_barrier_sync(1, 128);
      if (warp == 2 && lane == 0) {
        const unsigned int done = atomicAdd(ca.counter, 1u);
        if (done == gridDim.x - 1) {
          *ca.counter = 0;                               // ready for the next launch on this stream
          __threadfence_system();
          if (ok && *abort_flag == 0)
            for (int p = 0; p < ca.world; ++p)
              st_release_sys(reinterpret_cast<uint32_t*>(ca.flag_ptrs.p[p]) + ca.slot * ca.world + ca.rank, ca.seq);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// out[rows, N] = sum over the W slots of partials[W, rows, N] (+ residual), once every rank's flag has arrived
__global__ void reduce_partials_kernel(const __nv_bfloat16* __restrict__ partials, const __nv_bfloat16* __restrict__ residual,
                                       __nv_bfloat16* __restrict__ out, long long rows, int N, long long ld, int world,
                                       const uint32_t* my_flags, int slot, uint32_t seq, unsigned long long limit_ns,
                                       int* __restrict__ err) {
  __shared__ int go;
  if (threadIdx.x == 0) {
    int okv = *reinterpret_cast<volatile int*>(err) == 0 ? 1 : 0;
    const uint64_t t0 = globaltimer_ns();
    for (int r = 0; r < world && okv; ++r) {
      const uint32_t* f = my_flags + slot * world + r;
      while (static_cast<int32_t>(ld_acquire_sys(f) - seq) < 0) {
        if (globaltimer_ns() - t0 > limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); okv = 0; break; }
        __nanosleep(64);
      }
    }
    go = okv;
  }
  __syncthreads();
  if (!go) return;
  const int nvec = N >> 3;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nvec;
    const int c = static_cast<int>(i - r * nvec);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < world; ++w) {
      const uint4 v = *reinterpret_cast<const uint4*>(partials + (static_cast<long long>(w) * rows + r) * ld + c * 8);
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
    if (residual != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + r * N + c * 8);
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
    uint4 pk;
    pk.x = pack_bf16(acc[0], acc[1]); pk.y = pack_bf16(acc[2], acc[3]); pk.z = pack_bf16(acc[4], acc[5]); pk.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * N + c * 8) = pk;
  }
}

static int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return n;
}

template <int MODE>
static int launch(const TmaSet& maps, const CUtensorMap& tb, void* D, int M, int N, int K, long long ldd, const CommArgs& ca,
                  int* err, cudaStream_t stream) {
  auto kern = gemm_comm_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sms = sm_count();
  kern<<<tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, stream>>>(maps, tb, D, M, N, K, ldd, ca, err);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm_comm
}  // namespace dewb

// D[M, N] (bf16, row stride ldd) = gather_rows(A) * B^T. a_ptrs[s]: rank s's shard [M / world, K] (row stride lda, the
// same on every rank); B [N, K] local. my_flags[slot * world + s] >= seq once rank s has written its shard (the local
// rank's own flag is not consulted). M / world must be a multiple of 128.
extern "C" int dewb_ag_gemm_bf16(const unsigned long long* a_ptrs, const void* B, void* D, int M, int N, int K,
                                 long long lda, long long ldb, long long ldd, int rank, int world, const void* my_flags,
                                 int slot, unsigned int seq, unsigned long long limit_ns, int* err, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm_comm;
  if (world < 1 || world > MAX_RANKS || M % (world * BM) != 0 || (lda % 8) || (ldb % 8) || (ldd % 8)) return -3;
  TmaSet maps;
  const int Ms = M / world;
  for (int s = 0; s < world; ++s) {
    const int r = make_tmap_2d(&maps.m[s], reinterpret_cast<const void*>(a_ptrs[s]), Ms, K, lda, BM, BK, 2, true);
    if (r) return 1000 + r;
  }
  for (int s = world; s < MAX_RANKS; ++s) maps.m[s] = maps.m[0];
  CUtensorMap tb;
  const int r = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2, true);
  if (r) return 2000 + r;
  CommArgs ca{};
  ca.rank = rank; ca.world = world; ca.tiles_per_shard = Ms / BM;
  ca.my_flags = reinterpret_cast<const uint32_t*>(my_flags); ca.slot = slot; ca.seq = seq; ca.limit_ns = limit_ns;
  return launch<0>(maps, tb, D, M, N, K, ldd, ca, err, reinterpret_cast<cudaStream_t>(stream_ptr));
}

// Partial product scattered to its owners: rows [j * M/world, (j+1) * M/world) of A * B^T land in slot `rank` of rank j's
// partial buffer partial_ptrs[j] ([world, M / world, N] bf16, contiguous). flag_ptrs[p][slot * world + rank] = seq is
// published to every rank p once all of this rank's tiles are stored. counter: one zero-initialised device word.
extern "C" int dewb_gemm_rs_bf16(const void* A, const void* B, const unsigned long long* partial_ptrs, int M, int N, int K,
                                 long long lda, long long ldb, int rank, int world, const unsigned long long* flag_ptrs,
                                 int slot, unsigned int seq, unsigned int* counter, int* err, void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm_comm;
  if (world < 1 || world > MAX_RANKS || M % (world * BM) != 0 || (lda % 8) || (ldb % 8) || (N % 8)) return -3;
  TmaSet maps;
  int r = make_tmap_2d(&maps.m[0], A, M, K, lda, BM, BK, 2, true);
  if (r) return 1000 + r;
  for (int s = 1; s < MAX_RANKS; ++s) maps.m[s] = maps.m[0];
  CUtensorMap tb;
  r = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2, true);
  if (r) return 2000 + r;
  CommArgs ca{};
  ca.rank = rank; ca.world = world; ca.tiles_per_shard = (M / world) / BM;
  for (int p = 0; p < world; ++p) { ca.flag_ptrs.p[p] = flag_ptrs[p]; ca.partials.p[p] = partial_ptrs[p]; }
  ca.slot = slot; ca.seq = seq; ca.counter = counter;
  return launch<1>(maps, tb, nullptr, M, N, K, N, ca, err, reinterpret_cast<cudaStream_t>(stream_ptr));
}

// out[rows, N] = sum_w partials[w, rows, N] (+ residual[rows, N]) after my_flags[slot * world + w] >= seq for every w.
extern "C" int dewb_reduce_partials(const void* partials, const void* residual, void* out, long long rows, int N, int world,
                                    const void* my_flags, int slot, unsigned int seq, unsigned long long limit_ns, int* err,
                                    void* stream_ptr) {
  using namespace dewb::gemm_comm;
  if (N % 8 != 0 || rows <= 0) return rows == 0 ? 0 : -3;
  const long long total = rows * (N >> 3);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  reduce_partials_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_ptr)>>>(
      reinterpret_cast<const __nv_bfloat16*>(partials), reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(out), rows, N, N, world, reinterpret_cast<const uint32_t*>(my_flags), slot, seq, limit_ns, err);
  return static_cast<int>(cudaGetLastError());
}
