// Mixture-of-experts routing and token exchange over peer memory.
//
//   moe_route_kernel   one warp per token: softmax / sigmoid scores over E experts, selection by score + bias, top-k,
//                      optional normalisation of the k weights.
//   moe_rank_kernel    one CTA per expert: the rank of every (token, choice) pair among the pairs of its expert, in
//                      pair order (deterministic: ballots and prefix counts, no atomics), and the expert's count.
//   moe_plan_kernel    every rank reads all ranks' counts from their symmetric memory (after a bounded wait for the
//                      "counts written" flags) and derives the same placement: on the owner of expert e the rows coming
//                      from rank r start at  aligned_offset[e] + sum_{r' < r} counts[r'][e]  of an expert-sorted buffer
//                      whose group starts are multiples of 128 - the layout the tcgen05 grouped GEMM consumes.  It
//                      writes each pair's (destination rank, destination row) and the owner-side layout of this rank.
//   moe_push_kernel    dispatch: one warp per token stores the token's row (bf16, optionally scaled per pair, or
//                      quantised to e4m3 with a per-row scale on the way) straight into the destination ranks' receive
//                      buffers with plain peer stores; the last block to finish raises the "rows pushed" flag on
//                      every peer.
//   moe_pull_kernel    combine: one warp per token loads the token's k result rows from the owners' output buffers
//                      (peer loads), weights and sums them in fp32; the last block raises the "rows pulled" flag.
// With one rank the same kernels run with the rank as its own only peer.
//
// Replaces the reference's exchange dispatch: per-expert count all-gather, ragged all-to-all dispatch and combine
// (src/dew/nn/moe.py:1131-1215) and the router's top-k (src/dew/nn/moe.py:316-586).
#include "../common/peer.cuh"
#include <cuda_fp8.h>

namespace dewb {
namespace moe {

using namespace dewb::peer;
using bf16 = __nv_bfloat16;

constexpr int MAX_E = 256;
constexpr int MAX_K = 16;
constexpr uint32_t FULL = 0xffffffffu;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ scores_out,
                 float* __restrict__ w_out, int* __restrict__ ids_out, int T, int E, int k, int sigmoid, int norm,
                 float scaling) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    float sc[MAX_E / 32], sel[MAX_E / 32];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAX_E / 32; ++i) {
      const int e = lane + 32 * i;
      sc[i] = e < E ? logits[static_cast<long long>(t) * E + e] : -INFINITY;
      mx = fmaxf(mx, sc[i]);
    }
    if (sigmoid) {
#pragma unroll
      for (int i = 0; i < MAX_E / 32; ++i) sc[i] = (lane + 32 * i) < E ? 1.f / (1.f + __expf(-sc[i])) : 0.f;
    } else {
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < MAX_E / 32; ++i) { sc[i] = (lane + 32 * i) < E ? __expf(sc[i] - mx) : 0.f; sum += sc[i]; }
      sum = warp_sum(sum);
      const float inv = 1.f / sum;
#pragma unroll
      for (int i = 0; i < MAX_E / 32; ++i) sc[i] *= inv;
    }
#pragma unroll
    for (int i = 0; i < MAX_E / 32; ++i) {
      const int e = lane + 32 * i;
      if (e < E) {
        scores_out[static_cast<long long>(t) * E + e] = sc[i];
        sel[i] = sc[i] + (bias != nullptr ? bias[e] : 0.f);
      } else {
        sel[i] = -INFINITY;
      }
    }
    float my_w = 0.f;
    int my_id = 0;
    float wsum = 0.f;
    for (int j = 0; j < k; ++j) {
      // this lane's best remaining candidate, then the warp's (ties go to the lower expert index)
      float bv = -INFINITY, bs = 0.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAX_E / 32; ++i) {
        if (sel[i] > bv) { bv = sel[i]; bi = lane + 32 * i; bs = sc[i]; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(FULL, bv, o);
        const int oi = __shfl_xor_sync(FULL, bi, o);
        const float os = __shfl_xor_sync(FULL, bs, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
      }
      if ((bi & 31) == lane) {
#pragma unroll
        for (int i = 0; i < MAX_E / 32; ++i) if (i == (bi >> 5)) sel[i] = -INFINITY;
      }
      wsum += bs;
      if (lane == j) { my_w = bs; my_id = bi; }
    }
    if (lane < k) {
      float w = my_w;
      if (norm) w = w / fmaxf(wsum, 1e-20f);
      w_out[static_cast<long long>(t) * k + lane] = w * scaling;
      ids_out[static_cast<long long>(t) * k + lane] = my_id;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_rank_kernel(const int* __restrict__ ids, int pairs, int* __restrict__ rank_in_group, int* __restrict__ counts) {
  __shared__ int warp_tot[8];
  __shared__ int running_s;
  const int e = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) running_s = 0;
  __syncthreads();
  for (int base = 0; base < pairs; base += 256) {
    const int p = base + tid;
    const bool flag = p < pairs && ids[p] == e;
    const uint32_t ballot = __ballot_sync(FULL, flag);
    const int before = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int off = running_s, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) { if (w < warp) off += warp_tot[w]; total += warp_tot[w]; }
    if (flag) rank_in_group[p] = off + before;
    __syncthreads();
    if (tid == 0) running_s += total;
    __syncthreads();
  }
  if (tid == 0) counts[e] = running_s;
}

// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_plan_kernel(Peers counts_ptrs, const uint32_t* __restrict__ my_flags, int slot, uint32_t seq, unsigned long long limit_ns,
                const int* __restrict__ ids, const int* __restrict__ rank_in_group, int pairs, int E, int rank, int world,
                int rows_cap, int* __restrict__ dest_rank, int* __restrict__ dest_pos, int* __restrict__ offsets,
                int* __restrict__ local_counts, int* __restrict__ tile_group, int* __restrict__ info, int* __restrict__ err) {
  __shared__ int cnt[MAX_RANKS][MAX_E];
  __shared__ int aligned[MAX_E], owner_off[MAX_E], src_base[MAX_E], total[MAX_E];
  __shared__ int owner_rows[MAX_RANKS];
  if (status_poisoned(err)) return;
  if (world > 1 && !wait_all_peers(my_flags, slot, world, seq, limit_ns, err)) return;
  const int tid = threadIdx.x;
  const int per = E / world;
  for (int i = tid; i < world * E; i += blockDim.x) {
    const int r = i / E, e = i - r * E;
    cnt[r][e] = ld_sys_s32(reinterpret_cast<const int*>(counts_ptrs.p[r]) + e);
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int r = 0; r < world; ++r) { tot += cnt[r][e]; if (r < rank) before += cnt[r][e]; }
    total[e] = tot;
    aligned[e] = (tot + 127) / 128 * 128;
    src_base[e] = before;
  }
  __syncthreads();
  if (tid < world) {
    int off = 0;
    for (int le = 0; le < per; ++le) { const int e = tid * per + le; owner_off[e] = off; off += aligned[e]; }
    owner_rows[tid] = off;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) src_base[e] += owner_off[e];
  __syncthreads();
  const int rows_mine = owner_rows[rank];
  if (blockIdx.x == 0) {
    // A receive buffer that is too small drops the pairs past its end (capacity semantics): the owner's layout is cut at the
    // buffer's end, the dropped pairs get position -1 (not sent, contribute zero to the combine), and the caller reads how many.
    for (int le = tid; le < per; le += blockDim.x) {
      const int o = owner_off[rank * per + le];
      offsets[le] = min(o, rows_cap);
      local_counts[le] = max(0, min(total[rank * per + le], rows_cap - o));
    }
    if (tid == 0) {
      offsets[per] = min(rows_mine, rows_cap);
      int worst = 0;
      long long dropped = 0;
      for (int r = 0; r < world; ++r) worst = max(worst, owner_rows[r]);
      for (int e = 0; e < E; ++e) {
        const int o = owner_off[e];                                  // rows of expert e past its owner's buffer end
        dropped += max(0, min(total[e], o + total[e] - rows_cap));
      }
      info[0] = min(rows_mine, rows_cap);
      info[1] = worst > rows_cap ? 1 : 0;
      info[2] = worst;                                               // rows (with group padding) the busiest owner was sent
      info[3] = static_cast<int>(dropped);                           // pairs dropped over all owners (the same number on every rank)
    }
  }
  const int stride = gridDim.x * blockDim.x;
  for (int p = blockIdx.x * blockDim.x + tid; p < pairs; p += stride) {
    const int e = ids[p];
    const int pos = src_base[e] + rank_in_group[p];
    dest_rank[p] = e / per;
    dest_pos[p] = pos < rows_cap ? pos : -1;
  }
  const int tiles = rows_cap / 128;
  for (int t = blockIdx.x * blockDim.x + tid; t < tiles; t += stride) {
    const int start = t * 128;
    int grp = -1;
    if (start < rows_mine) {
      for (int le = 0; le < per; ++le) {
        const int o = owner_off[rank * per + le];
        if (start >= o && start < o + aligned[rank * per + le]) { grp = le; break; }
      }
    }
    tile_group[t] = grp;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// FP8 = false: recv is bf16 [rows_cap, d];  FP8 = true: recv is e4m3 [rows_cap, d] and recv_scale fp32 [rows_cap].
template <bool FP8>
__global__ void __launch_bounds__(256)
moe_push_kernel(const bf16* __restrict__ x, const float* __restrict__ pair_scale, const int* __restrict__ dest_rank,
                const int* __restrict__ dest_pos, Peers recv, Peers recv_scale, Peers flags, const uint32_t* __restrict__ my_flags,
                int slot_ready, int slot_pushed, uint32_t seq, unsigned long long limit_ns, unsigned int* __restrict__ counter,
                int T, int d, int k, int rank, int world, int* __restrict__ err) {
  if (status_poisoned(err)) return;
  if (world > 1 && !wait_all_peers(my_flags, slot_ready, world, seq, limit_ns, err)) return;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = d >> 3;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * d);
    float inv = 1.f;
    if (FP8) {
      float mx = 0.f;
      for (int i = lane; i < nvec; i += 32) {
        float f[8]; unpack8(xr[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(f[j]));
      }
      mx = warp_max(mx);
      const float sc = mx > 0.f ? mx / 448.f : 1.f;
      inv = 1.f / sc;
      if (lane < k) {
        const int pos = dest_pos[static_cast<long long>(t) * k + lane];
        if (pos >= 0) reinterpret_cast<float*>(recv_scale.p[dest_rank[static_cast<long long>(t) * k + lane]])[pos] = sc;
      }
    }
    for (int i = lane; i < nvec; i += 32) {
      const uint4 v = xr[i];
      float f[8];
      uint2 q8 = make_uint2(0u, 0u);
      if (FP8) {
        unpack8(v, f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q8.x |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
          q8.y |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f[4 + j] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
        }
      } else if (pair_scale != nullptr) {
        unpack8(v, f);
      }
      for (int j = 0; j < k; ++j) {
        const long long p = static_cast<long long>(t) * k + j;
        const int pos = dest_pos[p];
        if (pos < 0) continue;
        uint8_t* base = reinterpret_cast<uint8_t*>(recv.p[dest_rank[p]]);
        if (FP8) {
          reinterpret_cast<uint2*>(base + static_cast<long long>(pos) * d)[i] = q8;
        } else if (pair_scale != nullptr) {
          const float s = pair_scale[p];
          float g[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) g[c] = f[c] * s;
          reinterpret_cast<uint4*>(base + static_cast<long long>(pos) * d * 2)[i] = pack8(g);
        } else {
          reinterpret_cast<uint4*>(base + static_cast<long long>(pos) * d * 2)[i] = v;
        }
      }
    }
  }
  if (world > 1) last_block_signals(counter, flags, slot_pushed, rank, world, seq);
}

// out[t] = sum_j w[t, j] * src(dest_rank, dest_pos)[.]  (w null: plain sum); gathered (optional) keeps the k rows.
__global__ void __launch_bounds__(256)
moe_pull_kernel(Peers src, const float* __restrict__ w, const int* __restrict__ dest_rank, const int* __restrict__ dest_pos,
                bf16* __restrict__ out, bf16* __restrict__ gathered, Peers flags, const uint32_t* __restrict__ my_flags,
                int slot_ready, int slot_pulled, uint32_t seq, unsigned long long limit_ns, unsigned int* __restrict__ counter,
                int T, int d, int k, int rank, int world, int* __restrict__ err) {
  if (status_poisoned(err)) return;
  if (world > 1 && !wait_all_peers(my_flags, slot_ready, world, seq, limit_ns, err)) return;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = d >> 3;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    for (int i = lane; i < nvec; i += 32) {
      float acc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = 0.f;
      for (int j = 0; j < k; ++j) {
        const long long p = static_cast<long long>(t) * k + j;
        const int pos = dest_pos[p];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (pos >= 0) v = ld_sys_u4(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(src.p[dest_rank[p]]) +
                                                                   static_cast<long long>(pos) * d * 2) + i);
        if (gathered != nullptr) reinterpret_cast<uint4*>(gathered + p * d)[i] = v;
        float f[8]; unpack8(v, f);
        const float wj = w != nullptr ? w[p] : 1.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = fmaf(wj, f[c], acc[c]);
      }
      reinterpret_cast<uint4*>(out + static_cast<long long>(t) * d)[i] = pack8(acc);
    }
  }
  if (world > 1) last_block_signals(counter, flags, slot_pulled, rank, world, seq);
}

static inline int warp_grid(int T) {
  long long b = (static_cast<long long>(T) * 32 + 255) / 256;
  if (b < 1) b = 1;
  return static_cast<int>(b < 148 * 8 ? b : 148 * 8);
}

}  // namespace moe
}  // namespace dewb

using namespace dewb::moe;
#define STREAM(p) reinterpret_cast<cudaStream_t>(p)

// logits [T, E] fp32, bias [E] fp32 or null -> scores [T, E] fp32, weights [T, k] fp32, ids [T, k] int32.
extern "C" int dewb_moe_route(const float* logits, const float* bias, float* scores, float* weights, int* ids, int T, int E,
                              int k, int sigmoid, int norm, float scaling, void* stream) {
  if (E <= 0 || E > MAX_E || k <= 0 || k > MAX_K || k > E) return -3;
  if (T <= 0) return 0;
  moe_route_kernel<<<warp_grid(T), 256, 0, STREAM(stream)>>>(logits, bias, scores, weights, ids, T, E, k, sigmoid, norm, scaling);
  return static_cast<int>(cudaGetLastError());
}

// ids [pairs] int32 in [0, E) -> rank_in_group [pairs], counts [E] (counts may live in symmetric memory).
extern "C" int dewb_moe_rank(const int* ids, int pairs, int E, int* rank_in_group, int* counts, void* stream) {
  if (E <= 0 || E > MAX_E) return -3;
  moe_rank_kernel<<<E, 256, 0, STREAM(stream)>>>(ids, pairs, rank_in_group, counts);
  return static_cast<int>(cudaGetLastError());
}

// counts_ptrs: the W ranks' count arrays.  Outputs: dest_rank / dest_pos [pairs]; offsets [E / W + 1], local_counts [E / W],
// tile_group [rows_cap / 128] (this rank's layout as an owner); info = {rows in use, overflow flag}.
extern "C" int dewb_moe_plan(const unsigned long long* counts_ptrs, const void* my_flags, int slot, unsigned int seq,
                             unsigned long long limit_ns, const int* ids, const int* rank_in_group, int pairs, int E, int rank,
                             int world, int rows_cap, int* dest_rank, int* dest_pos, int* offsets, int* local_counts,
                             int* tile_group, int* info, int* err, void* stream) {
  if (E <= 0 || E > MAX_E || world < 1 || world > MAX_RANKS || E % world != 0 || rows_cap % 128 != 0) return -3;
  int blocks = (pairs + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  moe_plan_kernel<<<blocks, 256, 0, STREAM(stream)>>>(make_peers(counts_ptrs, world), reinterpret_cast<const uint32_t*>(my_flags),
                                                      slot, seq, limit_ns, ids, rank_in_group, pairs, E, rank, world, rows_cap,
                                                      dest_rank, dest_pos, offsets, local_counts, tile_group, info, err);
  return static_cast<int>(cudaGetLastError());
}

// x [T, d] bf16 -> rows of the destination ranks' receive buffers.  fp8 = 0: recv bf16 [rows_cap, d], pair_scale [T * k]
// fp32 or null; fp8 = 1: recv e4m3 [rows_cap, d] + recv_scale fp32 [rows_cap] (pair_scale ignored).
extern "C" int dewb_moe_push(const void* x, const float* pair_scale, const int* dest_rank, const int* dest_pos,
                             const unsigned long long* recv_ptrs, const unsigned long long* recv_scale_ptrs,
                             const unsigned long long* flag_ptrs, const void* my_flags, int slot_ready, int slot_pushed,
                             unsigned int seq, unsigned long long limit_ns, unsigned int* counter, int T, int d, int k, int rank,
                             int world, int fp8, int* err, void* stream) {
  if (d % 8 != 0 || k <= 0 || k > MAX_K || world < 1 || world > MAX_RANKS) return -3;
  if (T <= 0) return 0;
  const Peers recv = make_peers(recv_ptrs, world), rs = make_peers(recv_scale_ptrs, world), fl = make_peers(flag_ptrs, world);
  if (fp8)
    moe_push_kernel<true><<<warp_grid(T), 256, 0, STREAM(stream)>>>(
        reinterpret_cast<const bf16*>(x), pair_scale, dest_rank, dest_pos, recv, rs, fl, reinterpret_cast<const uint32_t*>(my_flags),
        slot_ready, slot_pushed, seq, limit_ns, counter, T, d, k, rank, world, err);
  else
    moe_push_kernel<false><<<warp_grid(T), 256, 0, STREAM(stream)>>>(
        reinterpret_cast<const bf16*>(x), pair_scale, dest_rank, dest_pos, recv, rs, fl, reinterpret_cast<const uint32_t*>(my_flags),
        slot_ready, slot_pushed, seq, limit_ns, counter, T, d, k, rank, world, err);
  return static_cast<int>(cudaGetLastError());
}

// out [T, d] bf16 = sum over the k choices of w * (row of the owner's buffer, bf16 [rows_cap, d]); gathered [T * k, d] or null.
extern "C" int dewb_moe_pull(const unsigned long long* src_ptrs, const float* w, const int* dest_rank, const int* dest_pos,
                             void* out, void* gathered, const unsigned long long* flag_ptrs, const void* my_flags,
                             int slot_ready, int slot_pulled, unsigned int seq, unsigned long long limit_ns,
                             unsigned int* counter, int T, int d, int k, int rank, int world, int* err, void* stream) {
  if (d % 8 != 0 || k <= 0 || k > MAX_K || world < 1 || world > MAX_RANKS) return -3;
  if (T <= 0) return 0;
  moe_pull_kernel<<<warp_grid(T), 256, 0, STREAM(stream)>>>(
      make_peers(src_ptrs, world), w, dest_rank, dest_pos, reinterpret_cast<bf16*>(out), reinterpret_cast<bf16*>(gathered),
      make_peers(flag_ptrs, world), reinterpret_cast<const uint32_t*>(my_flags), slot_ready, slot_pulled, seq, limit_ns,
      counter, T, d, k, rank, world, err);
  return static_cast<int>(cudaGetLastError());
}
