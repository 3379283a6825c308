// Paged decode attention, streamed: a producer warp brings whole 64-key pages of K and V into a shared-memory ring with
// TMA (one [64 x 128] tile each, 128-byte swizzle, no multicast) while four consumer warps compute from shared memory
// on the tensor cores.  bf16 pools, head dimension 128, up to 8 query heads per KV head, page size a multiple of 64.
//
// grid = (row, kv head, key split), 160 threads.  Per 64-key tile each consumer warp owns 16 keys:
//   S   = Q K^T   mma.sync m16n8k16 (rows = the query heads of the group, padded to 16; K fragments by ldmatrix)
//   online softmax in the log2 domain, per head row, inside the warp (quad reductions)
//   O  += P V     the score accumulators re-packed as the A operand, V fragments by ldmatrix.trans
// The per-warp (max, sum, O) are merged in shared memory and written as one partial per (row, head, split); the
// combine kernel of decode_attention.cu finishes (splits, sinks, normalisation).  The producer runs up to three tiles
// ahead, so the memory latency is hidden by the ring rather than by occupancy.
// The query count per KV head is far below the 64 rows tcgen05 needs, which is why this kernel uses the warp-level MMA.
//
// Capability parity: src/dew/nn/kernels/decode_attention.py (attend_paged), src/dew/nn/kernels/templates/attention_decode.py.
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace dewb {
namespace decode2 {

constexpr int D = 128;
constexpr int TK = 64;                       // keys per tile (one page or a page-aligned part of one)
constexpr int STAGES = 3;
constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int TILE_BYTES = TK * D * 2;       // 16 KiB: two 64-column halves of [64 rows x 128 B]
constexpr int STAGE_BYTES = 2 * TILE_BYTES;  // K and V
constexpr int OFF_Q = STAGES * STAGE_BYTES;  // [8 heads][128] bf16
constexpr int OFF_BARS = OFF_Q + 8 * D * 2;
constexpr int SMEM = OFF_BARS + 128;
constexpr uint32_t FULL = 0xffffffffu;

struct Bars {
  uint64_t full[STAGES], empty[STAGES];
  int abort_flag, poisoned;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (+)= A B, A [16 x 16] row-major bf16 (a1, a3: rows 8..15), B [16 x 8] as two k-halves, fp32 accumulate
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16-byte piece `chunk` (8 values, 0..15) of row `r` of a [64 x 128] bf16 tile stored as two swizzled 64-column halves
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, int r, int chunk) {
  return tile + (chunk >> 3) * (TK * 128) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
}

__global__ void __launch_bounds__(THREADS, 2)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                        const __nv_bfloat16* __restrict__ q, const int* __restrict__ page_table,
                        const int* __restrict__ lengths, float* __restrict__ part_m, float* __restrict__ part_l,
                        float* __restrict__ part_acc, int Hq, int Hkv, int page_size, int max_pages, int splits,
                        float scale_log2, int window, long long q_row_stride, int* __restrict__ err,
                        __nv_bfloat16* __restrict__ out, const float* __restrict__ sinks, unsigned int* __restrict__ arrivals,
                        int chunk_tiles) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    return;
  }
  Bars* bars = reinterpret_cast<Bars*>(smem + OFF_BARS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) bars->poisoned = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (bars->poisoned != 0) return;
  const int row = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int len = lengths[row];
  // this split's keys, in whole 64-key tiles: [t_begin, t_end) tile indices of the row; keys outside [first, len) are masked
  const int first = (window > 0 && len > window) ? len - window : 0;
  const int tile_lo = first / TK, tile_hi = (len + TK - 1) / TK;
  // With `out` the kernel finishes the row itself: a row uses as many of the grid's splits as it has chunks of `chunk_tiles`
  // tiles (short rows take one CTA, the others leave at once), and the last split to arrive merges the partials.
  int eff = splits;
  if (out != nullptr) {
    eff = (max(0, tile_hi - tile_lo) + chunk_tiles - 1) / chunk_tiles;
    eff = max(1, min(splits, eff));
    if (split >= eff) return;
  }
  const int per_split = (tile_hi - tile_lo + eff - 1) / eff;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_hi, t_begin + per_split);
  const int ntiles = max(0, t_end - t_begin);

  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + OFF_Q);
  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], CONSUMERS); }
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  for (int i = tid; i < 8 * D; i += THREADS) {
    const int g = i / D, d = i - g * D;
    sQ[i] = g < G ? q[static_cast<long long>(row) * q_row_stride + (hk * G + g) * D + d] : __float2bfloat16(0.f);
  }
  __syncthreads();
  volatile int* abort_flag = &bars->abort_flag;
  const uint32_t ring = smem_u32(smem);

  // per-warp running state of the group's heads: this lane's head row is lane / 4
  float m_run = -INFINITY, l_run = 0.f;
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; o[n][2] = 0.f; o[n][3] = 0.f; }

  if (warp == CONSUMERS) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      const int* table = page_table + static_cast<long long>(row) * max_pages;
      for (int t = 0; t < ntiles; ++t) {
        const int s = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); break; }
        const int key0 = (t_begin + t) * TK;
        const int page = table[key0 / page_size];
        const int row0 = page * page_size + key0 % page_size;
        uint8_t* st = smem + s * STAGE_BYTES;
        mbar_expect_tx(&bars->full[s], STAGE_BYTES);
        tma_load_2d(st, &tk, &bars->full[s], hk * D, row0);
        tma_load_2d(st + TK * 128, &tk, &bars->full[s], hk * D + 64, row0);
        tma_load_2d(st + TILE_BYTES, &tv, &bars->full[s], hk * D, row0);
        tma_load_2d(st + TILE_BYTES + TK * 128, &tv, &bars->full[s], hk * D + 64, row0);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    // Q fragments: A operand rows = heads; rows 8..15 do not exist (a1 = a3 = 0)
    uint32_t qa0[8], qa2[8];
    {
      const int g = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa0[ks] = *reinterpret_cast<const uint32_t*>(sQ + g * D + ks * 16 + c);
        qa2[ks] = *reinterpret_cast<const uint32_t*>(sQ + g * D + ks * 16 + 8 + c);
      }
    }
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      const int s = t % STAGES;
      const uint32_t ph = (t / STAGES) & 1;
      {
        const bool got = mbar_wait(&bars->full[s], ph, abort_flag);
        if (!__all_sync(FULL, got)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; break; }
      }
      const uint32_t kt = ring + s * STAGE_BYTES, vt = kt + TILE_BYTES;
      const int kw = warp * 16;                           // this warp's 16 keys of the tile
      // scores: two blocks of 8 keys
      float sc[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) { sc[nb][0] = 0.f; sc[nb][1] = 0.f; sc[nb][2] = 0.f; sc[nb][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        // four 8x8 matrices: (keys 0..7, dims lo), (keys 0..7, dims hi), (keys 8..15, dims lo), (keys 8..15, dims hi)
        const int mat = lane >> 3, r8 = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(tile_addr(kt, kw + (mat >> 1) * 8 + r8, ks * 2 + (mat & 1)), b0, b1, b2, b3);
        mma_16816(sc[0], qa0[ks], 0u, qa2[ks], 0u, b0, b1);
        mma_16816(sc[1], qa0[ks], 0u, qa2[ks], 0u, b2, b3);
      }
      // mask and online softmax for head row lane / 4 (values of rows 8..15, sc[.][2..3], are ignored)
      const int key_base = (t_begin + t) * TK + kw + (lane & 3) * 2;
      float pv[4];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = key_base + (i >> 1) * 8 + (i & 1);
        const float v = (key >= first && key < len) ? sc[i >> 1][i & 1] * scale_log2 : -INFINITY;
        pv[i] = v;
        mx = fmaxf(mx, v);
      }
      mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
      float ps = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) { pv[i] = (m_new == -INFINITY) ? 0.f : exp2f(pv[i] - m_new); ps += pv[i]; }
      ps += __shfl_xor_sync(FULL, ps, 1);
      ps += __shfl_xor_sync(FULL, ps, 2);
      l_run = l_run * alpha + ps;
      m_run = m_new;
#pragma unroll
      for (int n = 0; n < 16; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
      // P as the A operand of the second product: keys 0..7 -> a0, keys 8..15 -> a2
      const uint32_t pa0 = pack_bf16(pv[0], pv[1]), pa2 = pack_bf16(pv[2], pv[3]);
#pragma unroll
      for (int nb2 = 0; nb2 < 8; ++nb2) {
        // four transposed 8x8 matrices: (keys lo, dims chunk 2 nb2), (keys hi, same chunk), (keys lo, chunk + 1), (keys hi, chunk + 1)
        const int mat = lane >> 3, r8 = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(tile_addr(vt, kw + (mat & 1) * 8 + r8, nb2 * 2 + (mat >> 1)), b0, b1, b2, b3);
        mma_16816(o[nb2 * 2], pa0, 0u, pa2, 0u, b0, b1);
        mma_16816(o[nb2 * 2 + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty[s]);
    }
  }
  // merge the four consumer warps (the ring is free: every tile has been consumed or the CTA is leaving)
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(smem);                      // [4][8]
  float* sm_l = sm_m + CONSUMERS * 8;                                // [4][8]
  float* sm_acc = sm_l + CONSUMERS * 8;                              // [4][8][128]
  if (warp < CONSUMERS) {
    const int g = lane >> 2, c = (lane & 3) * 2;
    if ((lane & 3) == 0) { sm_m[warp * 8 + g] = m_run; sm_l[warp * 8 + g] = l_run; }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      sm_acc[(warp * 8 + g) * D + n * 8 + c] = o[n][0];
      sm_acc[(warp * 8 + g) * D + n * 8 + c + 1] = o[n][1];
    }
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += THREADS) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) mm = fmaxf(mm, sm_m[w * 8 + g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) {
      const float f = sm_m[w * 8 + g] == -INFINITY ? 0.f : exp2f(sm_m[w * 8 + g] - mm);
      ll += sm_l[w * 8 + g] * f;
      a += sm_acc[(w * 8 + g) * D + d] * f;
    }
    if (out != nullptr && eff == 1) {
      // the only split of the row: finish here (sink, normalisation)
      if (sinks != nullptr && mm > -INFINITY) {
        const float sk = sinks[hk * G + g] * 1.4426950408889634f;
        const float mn = fmaxf(mm, sk), f = exp2f(mm - mn);
        ll = ll * f + exp2f(sk - mn);
        a *= f;
      }
      out[(static_cast<long long>(row) * Hq + hk * G + g) * D + d] = __float2bfloat16(ll > 0.f ? a / ll : 0.f);
      continue;
    }
    const long long oidx = (static_cast<long long>(row) * Hq + hk * G + g) * splits + split;
    part_acc[oidx * D + d] = a;
    if (d == 0) { part_m[oidx] = mm; part_l[oidx] = ll; }
  }
  if (out == nullptr || eff == 1) return;
  // the last of the row's splits to get here merges them (the counter wraps back to zero for the next launch)
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicInc(arrivals + static_cast<long long>(row) * Hkv + hk, static_cast<unsigned int>(eff - 1)) == static_cast<unsigned int>(eff - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int i = tid; i < G * D; i += THREADS) {
    const int g = i / D, d = i - g * D;
    const long long base = (static_cast<long long>(row) * Hq + hk * G + g) * splits;
    float M = -INFINITY;
    for (int sp = 0; sp < eff; ++sp) M = fmaxf(M, __ldcg(part_m + base + sp));
    float Lsum = 0.f, a = 0.f;
    for (int sp = 0; sp < eff; ++sp) {
      const float ms = __ldcg(part_m + base + sp);
      if (ms == -INFINITY) continue;
      const float f = exp2f(ms - M);
      Lsum += __ldcg(part_l + base + sp) * f;
      a += __ldcg(part_acc + (base + sp) * D + d) * f;
    }
    if (sinks != nullptr && M > -INFINITY) {
      const float sk = sinks[hk * G + g] * 1.4426950408889634f;
      const float mn = fmaxf(M, sk), f = exp2f(M - mn);
      Lsum = Lsum * f + exp2f(sk - mn);
      a *= f;
    }
    out[(static_cast<long long>(row) * Hq + hk * G + g) * D + d] = __float2bfloat16(Lsum > 0.f ? a / Lsum : 0.f);
  }
}


// ---------------------------------------------------------------------------------------------------------------------
// Persistent, balanced form.  All 64-key tiles of a decode step - KV head by KV head, row by row - form one sequence, of
// which CTA b takes the tiles [b Q, (b + 1) Q): every CTA moves the same number of tiles whatever the rows' lengths are.
// Every CTA computes the rows' tile counts and their prefix sum from `lengths` in its prologue and walks its range segment
// by segment (a segment = the part of one (row, KV head) inside the range) through ONE shared-memory ring, so the producer
// warp is already fetching the next segment's pages while the consumers merge the current one, and a CTA's set-up cost is
// paid once per launch.  A (row, head) that lies inside one CTA's range is finished there; otherwise every CTA that holds a
// part writes a partial and the last one to arrive merges them (self-resetting ticket).  Rows without keys are zeroed.
constexpr int P_MAXROWS = 1024;
constexpr int P_OFF_MERGE = STAGES * STAGE_BYTES;                    // [4 warps][8 heads][64] fp32: one half of the head dimension at a time
constexpr int P_OFF_ML = P_OFF_MERGE + CONSUMERS * 8 * 64 * 4;        // [2][4][8] fp32
constexpr int P_OFF_PREFIX = P_OFF_ML + 2 * CONSUMERS * 8 * 4;        // [P_MAXROWS + 1] int
constexpr int P_OFF_BARS = P_OFF_PREFIX + (P_MAXROWS + 4) * 4;
constexpr int P_SMEM = P_OFF_BARS + 128;

struct PBars {
  uint64_t full[STAGES], empty[STAGES];
  int abort_flag, poisoned, is_last, pad;
};

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Seg { int row, hk, part, eff, t_begin, ntiles, first, len; };

// the segment that starts at tile `u` of the sequence and ends with its (row, head) or with the CTA's range `u1`
__device__ __forceinline__ Seg locate(int u, int u1, const int* prefix, const int* __restrict__ lengths, int rows,
                                      int per_head, int Q, int window) {
  Seg sg;
  sg.hk = u / per_head;
  const int w = u - sg.hk * per_head;
  int lo = 0, hi = rows;                                   // largest r with prefix[r] <= w
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= w) lo = mid; else hi = mid;
  }
  sg.row = lo;
  const int start = sg.hk * per_head + prefix[lo];          // the (row, head)'s first tile in the sequence
  const int n = prefix[lo + 1] - prefix[lo];
  sg.len = lengths[lo];
  sg.first = (window > 0 && sg.len > window) ? sg.len - window : 0;
  sg.t_begin = sg.first / TK + (u - start);
  sg.ntiles = min(u1, start + n) - u;
  const int first_cta = start / Q;
  sg.part = u / Q - first_cta;
  sg.eff = (start + n - 1) / Q - first_cta + 1;
  return sg;
}

__global__ void __launch_bounds__(THREADS, 2)
paged_decode_persist_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                            const __nv_bfloat16* __restrict__ q, const int* __restrict__ page_table,
                            const int* __restrict__ lengths, float* __restrict__ part_m, float* __restrict__ part_l,
                            float* __restrict__ part_acc, int rows, int Hq, int Hkv, int page_size, int max_pages,
                            int max_parts, float scale_log2, int window, long long q_row_stride, int* __restrict__ err,
                            __nv_bfloat16* __restrict__ out, const float* __restrict__ sinks,
                            unsigned int* __restrict__ arrivals, int min_tiles) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    return;
  }
  PBars* bars = reinterpret_cast<PBars*>(smem + P_OFF_BARS);
  int* prefix = reinterpret_cast<int*>(smem + P_OFF_PREFIX);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) bars->poisoned = *reinterpret_cast<volatile int*>(err);
  __syncthreads();
  if (bars->poisoned != 0) return;
  const int G = Hq / Hkv;
  // tile counts of the rows, then their exclusive prefix sum (warp 0: each lane a contiguous run of rows)
  for (int r = tid; r < rows; r += THREADS) {
    const int len = lengths[r];
    const int first = (window > 0 && len > window) ? len - window : 0;
    const int tiles = max(0, (len + TK - 1) / TK - first / TK);
    prefix[r + 1] = tiles;
    if (tiles == 0 && (r % gridDim.x) == blockIdx.x)         // a row without keys: its output is zero
      for (int i = 0; i < Hq * D; ++i) out[static_cast<long long>(r) * Hq * D + i] = __float2bfloat16(0.f);
  }
  if (tid == 0) {
    prefix[0] = 0;
    for (int i = 0; i < STAGES; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], CONSUMERS); }
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (warp == 0) {
    const int per = (rows + 31) / 32;
    const int r0 = min(rows, lane * per), r1 = min(rows, r0 + per);
    int sum = 0;
    for (int r = r0; r < r1; ++r) sum += prefix[r + 1];
    int incl = sum;
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(FULL, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int r = r0; r < r1; ++r) { run += prefix[r + 1]; prefix[r + 1] = run; }
  }
  __syncthreads();
  const int per_head = prefix[rows];
  const int total = per_head * Hkv;
  // a (row, head) of n tiles meets at most (n - 1) / Q + 2 ranges: Q is kept large enough for the partial buffers' stride
  int Q = max(min_tiles, (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
  const int u0 = min(total, static_cast<int>(blockIdx.x) * Q), u1 = min(total, u0 + Q);
  if (u0 >= u1) return;
  volatile int* abort_flag = &bars->abort_flag;
  const uint32_t ring = smem_u32(smem);
  int tg = 0;                                                // tiles this CTA has moved through the ring so far

  if (warp == CONSUMERS) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      bool ok = true;
      for (int u = u0; u < u1 && ok;) {
        const Seg sg = locate(u, u1, prefix, lengths, rows, per_head, Q, window);
        const int* table = page_table + static_cast<long long>(sg.row) * max_pages;
        for (int t = 0; t < sg.ntiles; ++t, ++tg) {
          const int s = tg % STAGES;
          const uint32_t ph = (tg / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag)) { atomicCAS(err, 0, ERR_WAIT_EMPTY); ok = false; break; }
          const int key0 = (sg.t_begin + t) * TK;
          const int page = table[key0 / page_size];
          const int row0 = page * page_size + key0 % page_size;
          uint8_t* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&bars->full[s], STAGE_BYTES);
          tma_load_2d(st, &tk, &bars->full[s], sg.hk * D, row0);
          tma_load_2d(st + TK * 128, &tk, &bars->full[s], sg.hk * D + 64, row0);
          tma_load_2d(st + TILE_BYTES, &tv, &bars->full[s], sg.hk * D, row0);
          tma_load_2d(st + TILE_BYTES + TK * 128, &tv, &bars->full[s], sg.hk * D + 64, row0);
        }
        u += sg.ntiles;
      }
    }
    return;
  }
  // -------------------------------------------------------------------- consumers (128 threads, named barrier 1)
  float* sm_acc = reinterpret_cast<float*>(smem + P_OFF_MERGE);      // [4][8][64]
  float* sm_m = reinterpret_cast<float*>(smem + P_OFF_ML);           // [4][8]
  float* sm_l = sm_m + CONSUMERS * 8;                                // [4][8]
  const int g = lane >> 2, c = (lane & 3) * 2;
  bool ok = true;
  for (int u = u0; u < u1;) {
    const Seg it = locate(u, u1, prefix, lengths, rows, per_head, Q, window);
    u += it.ntiles;
    // Q fragments straight from global memory: A operand rows = heads; rows 8..15 do not exist (a1 = a3 = 0)
    uint32_t qa0[8], qa2[8];
    {
      const __nv_bfloat16* qp = q + static_cast<long long>(it.row) * q_row_stride + (it.hk * G + g) * D + c;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa0[ks] = g < G ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
        qa2[ks] = g < G ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
      }
    }
    float m_run = -INFINITY, l_run = 0.f;
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; o[n][2] = 0.f; o[n][3] = 0.f; }
    for (int t = 0; t < it.ntiles; ++t, ++tg) {
      if (!ok) continue;
      const int s = tg % STAGES;
      const uint32_t ph = (tg / STAGES) & 1;
      {
        const bool got = mbar_wait(&bars->full[s], ph, abort_flag);
        if (!__all_sync(FULL, got)) { if (lane == 0) atomicCAS(err, 0, ERR_WAIT_FULL); ok = false; continue; }
      }
      const uint32_t kt = ring + s * STAGE_BYTES, vt = kt + TILE_BYTES;
      const int kw = warp * 16;
      float sc[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) { sc[nb][0] = 0.f; sc[nb][1] = 0.f; sc[nb][2] = 0.f; sc[nb][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int mat = lane >> 3, r8 = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(tile_addr(kt, kw + (mat >> 1) * 8 + r8, ks * 2 + (mat & 1)), b0, b1, b2, b3);
        mma_16816(sc[0], qa0[ks], 0u, qa2[ks], 0u, b0, b1);
        mma_16816(sc[1], qa0[ks], 0u, qa2[ks], 0u, b2, b3);
      }
      const int key_base = (it.t_begin + t) * TK + kw + (lane & 3) * 2;
      float pv[4];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = key_base + (i >> 1) * 8 + (i & 1);
        const float v = (key >= it.first && key < it.len) ? sc[i >> 1][i & 1] * scale_log2 : -INFINITY;
        pv[i] = v;
        mx = fmaxf(mx, v);
      }
      mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
      float ps = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) { pv[i] = (m_new == -INFINITY) ? 0.f : exp2f(pv[i] - m_new); ps += pv[i]; }
      ps += __shfl_xor_sync(FULL, ps, 1);
      ps += __shfl_xor_sync(FULL, ps, 2);
      l_run = l_run * alpha + ps;
      m_run = m_new;
#pragma unroll
      for (int n = 0; n < 16; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
      const uint32_t pa0 = pack_bf16(pv[0], pv[1]), pa2 = pack_bf16(pv[2], pv[3]);
#pragma unroll
      for (int nb2 = 0; nb2 < 8; ++nb2) {
        const int mat = lane >> 3, r8 = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(tile_addr(vt, kw + (mat & 1) * 8 + r8, nb2 * 2 + (mat >> 1)), b0, b1, b2, b3);
        mma_16816(o[nb2 * 2], pa0, 0u, pa2, 0u, b0, b1);
        mma_16816(o[nb2 * 2 + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty[s]);
    }
    // ---- merge the four warps (each holds 16 of every tile's 64 keys), half of the head dimension at a time
    if ((lane & 3) == 0) { sm_m[warp * 8 + g] = m_run; sm_l[warp * 8 + g] = l_run; }
    const bool single = it.eff == 1;
    const long long head0 = static_cast<long long>(it.row) * Hq + it.hk * G;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        sm_acc[(warp * 8 + g) * 64 + n * 8 + c] = o[half * 8 + n][0];
        sm_acc[(warp * 8 + g) * 64 + n * 8 + c + 1] = o[half * 8 + n][1];
      }
      consumer_bar();
      for (int i = tid; i < G * 64; i += CONSUMERS * 32) {
        const int gg = i >> 6, d = (i & 63) + half * 64;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) mm = fmaxf(mm, sm_m[w * 8 + gg]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
          const float f = sm_m[w * 8 + gg] == -INFINITY ? 0.f : exp2f(sm_m[w * 8 + gg] - mm);
          ll += sm_l[w * 8 + gg] * f;
          a += sm_acc[(w * 8 + gg) * 64 + (i & 63)] * f;
        }
        if (single) {
          if (sinks != nullptr && mm > -INFINITY) {
            const float sk = sinks[it.hk * G + gg] * 1.4426950408889634f;
            const float mn = fmaxf(mm, sk), f = exp2f(mm - mn);
            ll = ll * f + exp2f(sk - mn);
            a *= f;
          }
          out[(head0 + gg) * D + d] = __float2bfloat16(ll > 0.f ? a / ll : 0.f);
        } else {
          const long long oidx = (head0 + gg) * max_parts + it.part;
          part_acc[oidx * D + d] = a;
          if (d == 0) { part_m[oidx] = mm; part_l[oidx] = ll; }
        }
      }
      consumer_bar();
    }
    if (single) continue;
    // ---- several parts: the last CTA of the (row, head) to get here merges the partials
    __threadfence();
    consumer_bar();
    if (tid == 0)
      bars->is_last = atomicInc(arrivals + static_cast<long long>(it.row) * Hkv + it.hk, static_cast<unsigned int>(it.eff - 1)) ==
                      static_cast<unsigned int>(it.eff - 1);
    consumer_bar();
    const bool last = bars->is_last != 0;
    consumer_bar();                                          // (is_last may be rewritten by the next segment only after everyone read it)
    if (!last) continue;
    __threadfence();
    for (int i = tid; i < G * D; i += CONSUMERS * 32) {
      const int gg = i / D, d = i - gg * D;
      const long long base = (head0 + gg) * max_parts;
      float M = -INFINITY;
      for (int sp = 0; sp < it.eff; ++sp) M = fmaxf(M, __ldcg(part_m + base + sp));
      float Lsum = 0.f, a = 0.f;
      for (int sp = 0; sp < it.eff; ++sp) {
        const float ms = __ldcg(part_m + base + sp);
        if (ms == -INFINITY) continue;
        const float f = exp2f(ms - M);
        Lsum += __ldcg(part_l + base + sp) * f;
        a += __ldcg(part_acc + (base + sp) * D + d) * f;
      }
      if (sinks != nullptr && M > -INFINITY) {
        const float sk = sinks[it.hk * G + gg] * 1.4426950408889634f;
        const float mn = fmaxf(M, sk), f = exp2f(M - mn);
        Lsum = Lsum * f + exp2f(sk - mn);
        a *= f;
      }
      out[(head0 + gg) * D + d] = __float2bfloat16(Lsum > 0.f ? a / Lsum : 0.f);
    }
  }
}

}  // namespace decode2
}  // namespace dewb

// The streamed form of the paged decode attention's first stage: writes the per-split partials (part_m, part_l in the log2
// domain, part_acc) exactly as the first-stage kernel of dewb_paged_decode does; the caller runs the same combine.
// kpool / vpool: bf16 [pool_tokens, Hkv, 128] (pool_tokens = pages * page_size), page_size a multiple of 64, Hq / Hkv <= 8.
// q_row_stride: elements between the query rows (0 = packed [rows, Hq, 128]); a packed projection output can be read in place.
extern "C" int dewb_paged_decode_stream(const void* q, const void* kpool, const void* vpool, long long pool_tokens,
                                        const int* page_table, const int* lengths, float* part_m, float* part_l,
                                        float* part_acc, int rows, int Hq, int Hkv, int page_size, int max_pages, int splits,
                                        float scale, int window, long long q_row_stride, int* err, void* stream_ptr) {
  using namespace dewb::decode2;
  if (rows <= 0) return 0;
  if (Hq % Hkv != 0 || Hq / Hkv > 8 || page_size % TK != 0 || splits < 1 || pool_tokens <= 0) return -3;
  CUtensorMap tk, tv;
  int r;
  const uint64_t cols = static_cast<uint64_t>(Hkv) * D;
  if ((r = dewb::make_tmap_2d(&tk, kpool, static_cast<uint64_t>(pool_tokens), cols, cols, TK, 64, 2, true))) return 1000 + r;
  if ((r = dewb::make_tmap_2d(&tv, vpool, static_cast<uint64_t>(pool_tokens), cols, cols, TK, 64, 2, true))) return 2000 + r;
  cudaError_t e = cudaFuncSetAttribute(paged_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(rows, Hkv, splits);
  paged_decode_tma_kernel<<<grid, THREADS, SMEM, reinterpret_cast<cudaStream_t>(stream_ptr)>>>(
      tk, tv, reinterpret_cast<const __nv_bfloat16*>(q), page_table, lengths, part_m, part_l, part_acc, Hq, Hkv, page_size,
      max_pages, splits, scale * 1.4426950408889634f, window, q_row_stride > 0 ? q_row_stride : static_cast<long long>(Hq) * D, err,
      nullptr, nullptr, nullptr, 0);
  return static_cast<int>(cudaGetLastError());
}

// The same kernel finishing the rows itself: out [rows, Hq, 128] bf16; `arrivals` uint32 [rows * Hkv], zero once (the kernel
// leaves it zero); `sinks` fp32 [Hq] or null.  The grid carries `splits` CTAs per (row, KV head), of which a row uses one per
// `chunk_tiles` 64-key tiles it holds: choose splits = ceil(longest possible row in tiles / chunk_tiles).
extern "C" int dewb_paged_decode_fused(const void* q, const void* kpool, const void* vpool, long long pool_tokens,
                                       const int* page_table, const int* lengths, float* part_m, float* part_l,
                                       float* part_acc, unsigned int* arrivals, const float* sinks, void* out, int rows, int Hq,
                                       int Hkv, int page_size, int max_pages, int splits, int chunk_tiles, float scale,
                                       int window, long long q_row_stride, int* err, void* stream_ptr) {
  using namespace dewb::decode2;
  if (rows <= 0) return 0;
  if (Hq % Hkv != 0 || Hq / Hkv > 8 || page_size % TK != 0 || splits < 1 || chunk_tiles < 1 || pool_tokens <= 0) return -3;
  CUtensorMap tk, tv;
  int r;
  const uint64_t cols = static_cast<uint64_t>(Hkv) * D;
  if ((r = dewb::make_tmap_2d(&tk, kpool, static_cast<uint64_t>(pool_tokens), cols, cols, TK, 64, 2, true))) return 1000 + r;
  if ((r = dewb::make_tmap_2d(&tv, vpool, static_cast<uint64_t>(pool_tokens), cols, cols, TK, 64, 2, true))) return 2000 + r;
  cudaError_t e = cudaFuncSetAttribute(paged_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(rows, Hkv, splits);
  paged_decode_tma_kernel<<<grid, THREADS, SMEM, reinterpret_cast<cudaStream_t>(stream_ptr)>>>(
      tk, tv, reinterpret_cast<const __nv_bfloat16*>(q), page_table, lengths, part_m, part_l, part_acc, Hq, Hkv, page_size,
      max_pages, splits, scale * 1.4426950408889634f, window, q_row_stride > 0 ? q_row_stride : static_cast<long long>(Hq) * D, err,
      reinterpret_cast<__nv_bfloat16*>(out), sinks, arrivals, chunk_tiles);
  return static_cast<int>(cudaGetLastError());
}

// Persistent, balanced form of the same operation (see the kernel's comment): one launch of `ctas` CTAs (two per SM) that
// share out the tiles evenly.  A CTA's range is at least `min_tiles` tiles, so a (row, head) of n tiles is cut into at most
// (n - 1) / min_tiles + 2 parts: `max_parts` (the stride of the partial buffers: part_m / part_l [rows * Hq * max_parts],
// part_acc [... * 128]) must be at least that for the longest row.  rows <= 1024; `arrivals` uint32 [rows * Hkv], zero once.
extern "C" int dewb_paged_decode_persist(const void* q, const void* kpool, const void* vpool, long long pool_tokens,
                                         const int* page_table, const int* lengths, float* part_m, float* part_l,
                                         float* part_acc, unsigned int* arrivals, const float* sinks, void* out, int rows, int Hq,
                                         int Hkv, int page_size, int max_pages, int max_parts, int min_tiles, float scale,
                                         int window, long long q_row_stride, int ctas, int* err, void* stream_ptr) {
  using namespace dewb::decode2;
  if (rows <= 0) return 0;
  if (Hq % Hkv != 0 || Hq / Hkv > 8 || page_size % TK != 0 || max_parts < 2 || min_tiles < 1 || pool_tokens <= 0 ||
      rows > P_MAXROWS || ctas < 1)
    return -3;
  CUtensorMap tk, tv;
  int r;
  const uint64_t cols = static_cast<uint64_t>(Hkv) * D;
  if ((r = dewb::make_tmap_2d(&tk, kpool, static_cast<uint64_t>(pool_tokens), cols, cols, TK, 64, 2, true))) return 1000 + r;
  if ((r = dewb::make_tmap_2d(&tv, vpool, static_cast<uint64_t>(pool_tokens), cols, cols, TK, 64, 2, true))) return 2000 + r;
  cudaError_t e = cudaFuncSetAttribute(paged_decode_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  paged_decode_persist_kernel<<<ctas, THREADS, P_SMEM, reinterpret_cast<cudaStream_t>(stream_ptr)>>>(
      tk, tv, reinterpret_cast<const __nv_bfloat16*>(q), page_table, lengths, part_m, part_l, part_acc, rows, Hq, Hkv, page_size,
      max_pages, max_parts, scale * 1.4426950408889634f, window, q_row_stride > 0 ? q_row_stride : static_cast<long long>(Hq) * D, err,
      reinterpret_cast<__nv_bfloat16*>(out), sinks, arrivals, min_tiles);
  return static_cast<int>(cudaGetLastError());
}
