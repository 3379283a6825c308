// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a, bf16, fp32 accumulation).
//
//   all-gather -> GEMM   (column-parallel layer after a sequence-parallel region)
//       D[M, N] = A[M, K] * B[N, K]^T where rank s holds rows [s * M/W, (s+1) * M/W) of A in its symmetric buffer.
//       One kernel gathers and multiplies. A copier warp in every CTA pulls the peers' shards across NVLink exactly
//       once - TMA tile loads from the owning rank's memory (per-rank tensor maps, plain peer loads, no multicast)
//       into shared memory, TMA stores into a local staging copy - and counts each 128-row block in as it completes.
//       The GEMM tiles of the local shard go first and need nothing remote; a tile of a remote row block starts as soon
//       as that block's counter is full, so the transfer hides under the local products. (Reading A tiles straight
//       from peer memory in the main loop would move every tile across NVLink once per column block: peer memory is
//       not cached in the local L2.) The kernel itself announces "my shard is written" to the peers when it starts
//       and waits (bounded) for a peer's announcement before its first load from that peer.
//
//   GEMM -> reduce-scatter   (row-parallel layer before a sequence-parallel region)
//       every rank computes a partial P_r[M, N] = A_r * B_r^T over its slice of K; rank j owns rows
//       [j * M/W, (j+1) * M/W) of the sum. The epilogue stores each finished tile directly into slot `rank` of the
//       owner's symmetric partial buffer (peer st.global), so the transfer rides under the remaining tiles; the last
//       CTA to finish publishes a flag to every peer. `dewb_reduce_partials` on the owner waits for the W flags and
//       sums the W slots (+ optional residual).
//
// Kernel skeleton as the dense kernel: warp 0 TMA producer, warp 1 tcgen05 issuer, warps 2..5 epilogue, warp 6 copier,
// 4-stage ring, two TMEM accumulators. Every wait is bounded and reports through the status word. Buffers that peers
// read or write (the shard, the partial slots) are double-buffered by call parity, which makes a separate "done"
// handshake unnecessary: a rank can only reach call n + 1 after every peer has entered call n, i.e. left call n - 1.
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
constexpr int THREADS = 224;
constexpr int COPY_STAGES = 2;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + COPY_STAGES * A_BYTES + 1024 + 256;
constexpr int MAX_RANKS = 8;

struct alignas(64) TmaSet { CUtensorMap m[MAX_RANKS]; };
struct Peers { unsigned long long p[MAX_RANKS]; };

struct Shared {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], copy_full[COPY_STAGES];
  uint32_t tmem_base;
  int abort_flag;
  int epi_ok[4];             // MODE 1: each epilogue warp's verdict on the current tile's accumulator wait
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
  Peers flag_ptrs;               // every rank's flag array
  unsigned int* block_ready;     // MODE 0: per 128-row block of A, chunks staged so far (monotonic over calls)
  uint32_t ready_target;         // MODE 0: value a block's counter reaches when all its chunks of this call are staged
  Peers partials;                // MODE 1: every rank's partial buffer [W, M/W, N]
  int slot;
  uint32_t seq;
  unsigned long long limit_ns;
  unsigned int* counter;         // MODE 1: CTAs that have finished (reset by the last one)
};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_comm_kernel(const __grid_constant__ TmaSet maps, const __grid_constant__ TmaSet pmaps,
                 const __grid_constant__ CUtensorMap tma_stage, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Dptr,
                 int M, int N, int K, long long ldd, const CommArgs ca, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  {
    __shared__ int poisoned;
    if (threadIdx.x == 0) poisoned = *reinterpret_cast<volatile int*>(err);
    __syncthreads();
    if (poisoned != 0) return;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* cbuf = smem + STAGES * STAGE_BYTES;                 // copier staging: COPY_STAGES tiles of A
  Shared* sh = reinterpret_cast<Shared*>(cbuf + COPY_STAGES * A_BYTES);
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
    for (int c = 0; c < COPY_STAGES; ++c) mbar_init(&sh->copy_full[c], 1);
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
  if (MODE == 0 && blockIdx.x == 0 && threadIdx.x == 0) {
    // this kernel runs after whatever wrote the local shard (stream order): tell every peer it may read it
    __threadfence_system();
    for (int p = 0; p < ca.world; ++p)
      st_release_sys(reinterpret_cast<uint32_t*>(ca.flag_ptrs.p[p]) + ca.slot * ca.world + ca.rank, ca.seq);
  }

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_of(t, m_blk, n_blk);
        const int src = MODE == 0 ? m_blk / ca.tiles_per_shard : 0;
        const bool remote = MODE == 0 && src != ca.rank;
        // local rows come from the local shard; remote rows from the staging copy, indexed by the global row
        const int m0 = (MODE == 0 && !remote) ? (m_blk - src * ca.tiles_per_shard) * BM : m_blk * BM;
        const CUtensorMap* amap = remote ? &tma_stage : &maps.m[MODE == 0 ? ca.rank : 0];
        if (remote) {
          // bounded wait until the copier warps have staged this row block, then order the async-proxy reads after it
          const unsigned int* c = ca.block_ready + m_blk;
          const uint64_t t0 = globaltimer_ns();
          while (static_cast<int32_t>(*reinterpret_cast<const volatile unsigned int*>(c) - ca.ready_target) < 0) {
            if (*abort_flag != 0 || globaltimer_ns() - t0 > ca.limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); *abort_flag = 1; ok = false; break; }
            __nanosleep(32);
          }
          if (!ok) break;
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
          tma_load_2d(sa, amap, &sh->full[stage], k * BK, m0);
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
  } else if (warp == 6) {
    // ------------------------------------------------------------------ copier (MODE 0): peers' shards -> local staging
    if (MODE == 0 && lane == 0 && ca.world > 1) {
      const int kc = k_iters;                                  // 64-column chunks per row block
      const long long remote_blocks = static_cast<long long>(ca.world - 1) * ca.tiles_per_shard;
      const long long chunks = remote_blocks * kc;
      uint32_t have = 1u << ca.rank;
      int cs = 0; uint32_t cph = 0;
      int pend_blk[COPY_STAGES] = {-1, -1};
      bool ok = true;
      for (long long i = blockIdx.x; i < chunks && ok; i += gridDim.x) {
        const long long rb = i / kc;                           // remote row block in ring order from rank + 1
        const int k = static_cast<int>(i - rb * kc);
        const int src = (ca.rank + 1 + static_cast<int>(rb / ca.tiles_per_shard)) % ca.world;
        const int mb = static_cast<int>(rb % ca.tiles_per_shard);
        if (!((have >> src) & 1u)) {
          const uint32_t* f = ca.my_flags + ca.slot * ca.world + src;
          const uint64_t t0 = globaltimer_ns();
          while (static_cast<int32_t>(ld_acquire_sys(f) - ca.seq) < 0) {
            if (*abort_flag != 0 || globaltimer_ns() - t0 > ca.limit_ns) { atomicCAS(err, 0, ERR_WAIT_PEER); *abort_flag = 1; ok = false; break; }
            __nanosleep(64);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
          have |= 1u << src;
        }
        // the store that last used this staging stage must have read it; the block it belonged to is then published
        tma_store_wait_read<COPY_STAGES - 1>();
        uint8_t* dst = cbuf + cs * A_BYTES;
        mbar_expect_tx(&sh->copy_full[cs], A_BYTES);
        tma_load_2d(dst, &maps.m[src], &sh->copy_full[cs], k * BK, mb * BM);
        if (!mbar_wait(&sh->copy_full[cs], cph, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
        const int gblk = src * ca.tiles_per_shard + mb;        // global row block
        tma_store_2d(&tma_stage, dst, k * BK, gblk * BM);
        tma_store_commit();
        // publish the chunk stored one step earlier: at most one store group is still in flight after this wait
        tma_store_wait<COPY_STAGES - 1>();
        const int prev = pend_blk[cs ^ 1];
        if (prev >= 0) { asm volatile("fence.proxy.async;" ::: "memory"); __threadfence(); atomicAdd(ca.block_ready + prev, 1u); pend_blk[cs ^ 1] = -1; }
        pend_blk[cs] = gblk;
        if (++cs == COPY_STAGES) { cs = 0; cph ^= 1; }
      }
      tma_store_wait<0>();
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      for (int c = 0; c < COPY_STAGES; ++c) if (pend_blk[c] >= 0) atomicAdd(ca.block_ready + pend_blk[c], 1u);
    }
  } else if (MODE == 0) {
    // ------------------------------------------------------------------ epilogue, local output (warps 2..5)
    const int q = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m_blk, n_blk;
      tile_of(t, m_blk, n_blk);
      const int row = m_blk * BM + q * 32 + lane;
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
        if (row < M && col < N) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(Dptr) + static_cast<long long>(row) * ldd + col;
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
    // ------------------------------------------------------------------ epilogue, scattered to the owners (warps 2..5)
    // A tile leaves in four 128 x 64 pieces: TMEM -> registers -> bf16 in a swizzled shared-memory stage -> one TMA
    // store into slot `rank` of the owner's partial buffer. Bulk stores cross NVLink as large bursts; 64-byte
    // per-thread stores do not. The four warps meet at a named barrier at fixed points of every tile, whatever
    // their waits returned, so a timed-out wait can never strand the others there.
    const int q = warp & 3;
    const bool issuer = (warp == 2 && lane == 0);
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    int chunk = 0;                                     // running count of pieces: stage = chunk & 1
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m_blk, n_blk;
      tile_of(t, m_blk, n_blk);
      const int owner = m_blk / ca.tiles_per_shard;
      const int row0 = (m_blk - owner * ca.tiles_per_shard) * BM;     // row inside the owner's range
      const int n0 = n_blk * BN;
      bool got = ok && mbar_wait(&sh->tmem_full[acc], acc_phase, abort_flag);
      got = __all_sync(0xffffffffu, got);
      if (lane == 0) sh->epi_ok[q] = got ? 1 : 0;
      named_barrier_sync(1, 128);
      const bool all_got = (sh->epi_ok[0] & sh->epi_ok[1] & sh->epi_ok[2] & sh->epi_ok[3]) != 0;
      named_barrier_sync(1, 128);                      // everyone has read the verdicts before the next tile rewrites them
      if (!all_got) {
        if (ok && !got) atomicCAS(err, 0, ERR_WAIT_TMEM_FULL);
        ok = false;
        continue;                                      // keep the barrier count of the remaining tiles
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
      const int r_in = q * 32 + lane;                  // row of the tile this thread holds
#pragma unroll 1
      for (int c4 = 0; c4 < BN / 64; ++c4, ++chunk) {
        uint8_t* stage = cbuf + (chunk & 1) * A_BYTES;
        // the store that used this stage two pieces ago must have finished reading it
        if (issuer) tma_store_wait_read<1>();
        named_barrier_sync(1, 128);
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(taddr + c4 * 64, r0);
        tmem_ld_32x32b_x32(taddr + c4 * 64 + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t* src = j < 4 ? &r0[j * 8] : &r1[(j - 4) * 8];
          uint4 pk;
          pk.x = pack_bf16(__uint_as_float(src[0]), __uint_as_float(src[1]));
          pk.y = pack_bf16(__uint_as_float(src[2]), __uint_as_float(src[3]));
          pk.z = pack_bf16(__uint_as_float(src[4]), __uint_as_float(src[5]));
          pk.w = pack_bf16(__uint_as_float(src[6]), __uint_as_float(src[7]));
          *reinterpret_cast<uint4*>(stage + r_in * 128 + ((j ^ (r_in & 7)) << 4)) = pk;
        }
        fence_proxy_async();                           // generic-proxy writes of the stage -> visible to the bulk store
        named_barrier_sync(1, 128);
        if (issuer && n0 + c4 * 64 < N) {
          tma_store_2d(&pmaps.m[owner], stage, n0 + c4 * 64, row0);
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // every store of this CTA (most of them to peers) has completed and is visible system-wide before the CTA counts
    // itself done; the last CTA to finish publishes this rank's flag to every peer
    if (issuer) { tma_store_wait<0>(); asm volatile("fence.proxy.async;" ::: "memory"); }
    __threadfence_system();
    named_barrier_sync(1, 128);
    if (issuer) {
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
static int launch(const TmaSet& maps, const TmaSet& pmaps, const CUtensorMap& tstage, const CUtensorMap& tb, void* D, int M, int N, int K, long long ldd, const CommArgs& ca,
                  int* err, cudaStream_t stream) {
  auto kern = gemm_comm_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sms = sm_count();
  kern<<<tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, stream>>>(maps, pmaps, tstage, tb, D, M, N, K, ldd, ca, err);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm_comm
}  // namespace dewb

// D[M, N] (bf16, row stride ldd) = gather_rows(A) * B^T. a_ptrs[s]: rank s's shard [M / world, K] (row stride lda, the
// same on every rank; double-buffer it by call parity); B [N, K] local. staging: local scratch [M, K] bf16 (row stride
// lda) that receives the peers' shards; block_ready: M / 128 zero-initialised device words that persist across calls.
// flag_ptrs[p][slot * world + rank] = seq announces this rank's shard to rank p; my_flags is this rank's own flag array.
// calls: how many calls (including this one) have used `block_ready` - the counters are monotonic.
// M / world must be a multiple of 128 and K a multiple of 64.
extern "C" int dewb_ag_gemm_bf16(const unsigned long long* a_ptrs, const void* B, void* D, void* staging,
                                 unsigned int* block_ready, unsigned int calls, int M, int N, int K, long long lda,
                                 long long ldb, long long ldd, int rank, int world, const unsigned long long* flag_ptrs,
                                 const void* my_flags, int slot, unsigned int seq, unsigned long long limit_ns, int* err,
                                 void* stream_ptr) {
  using namespace dewb;
  using namespace dewb::gemm_comm;
  if (world < 1 || world > MAX_RANKS || M % (world * BM) != 0 || K % BK != 0 || (lda % 8) || (ldb % 8) || (ldd % 8)) return -3;
  TmaSet maps;
  const int Ms = M / world;
  for (int s = 0; s < world; ++s) {
    const int r = make_tmap_2d(&maps.m[s], reinterpret_cast<const void*>(a_ptrs[s]), Ms, K, lda, BM, BK, 2, true);
    if (r) return 1000 + r;
  }
  for (int s = world; s < MAX_RANKS; ++s) maps.m[s] = maps.m[0];
  CUtensorMap tb, tstage;
  int r = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2, true);
  if (r) return 2000 + r;
  r = make_tmap_2d(&tstage, staging, M, K, lda, BM, BK, 2, true);
  if (r) return 3000 + r;
  CommArgs ca{};
  ca.rank = rank; ca.world = world; ca.tiles_per_shard = Ms / BM;
  ca.my_flags = reinterpret_cast<const uint32_t*>(my_flags); ca.slot = slot; ca.seq = seq; ca.limit_ns = limit_ns;
  for (int p = 0; p < world; ++p) ca.flag_ptrs.p[p] = flag_ptrs[p];
  ca.block_ready = block_ready;
  ca.ready_target = calls * static_cast<unsigned int>(K / BK);
  return launch<0>(maps, maps, tstage, tb, D, M, N, K, ldd, ca, err, reinterpret_cast<cudaStream_t>(stream_ptr));
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
  // slot `rank` of every owner's partial buffer as a [M / world, N] tensor, stored in 128 x 64 pieces
  TmaSet pmaps;
  const int Ms = M / world;
  for (int p = 0; p < world; ++p) {
    const __nv_bfloat16* slot_base = reinterpret_cast<const __nv_bfloat16*>(partial_ptrs[p]) + static_cast<long long>(rank) * Ms * N;
    r = make_tmap_2d(&pmaps.m[p], slot_base, Ms, N, N, BM, 64, 2, true);
    if (r) return 3000 + r;
  }
  for (int p = world; p < MAX_RANKS; ++p) pmaps.m[p] = pmaps.m[0];
  return launch<1>(maps, pmaps, maps.m[0], tb, nullptr, M, N, K, N, ca, err, reinterpret_cast<cudaStream_t>(stream_ptr));
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
