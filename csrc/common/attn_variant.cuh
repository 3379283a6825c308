// Optional attention variants shared by the forward and backward flash kernels.  The plain causal / full kernels are
// compiled with VAR = false and contain none of this.
//   window   : query i sees keys in (i + T - S - window, i + T - S]  (0 = no window)
//   softcap  : scores become cap * tanh(score / cap)                 (0 = none)
//   sinks    : one learned logit per query head that joins the softmax denominator only (forward; the backward kernels
//              see it through the saved log-sum-exp)
//   segments : packed documents - a query sees a key only if both carry the same segment id; ids are non-decreasing
//              along the sequence (0 = padding, allowed after the last document), which is what lets whole tiles be skipped
#pragma once
#include <cuda_runtime.h>

namespace dewb {
namespace attn {

struct Variant {
  int window;
  float softcap;
  const float* sinks;      // [Hq] or null
  const int* q_seg;        // [B, S] or null
  const int* k_seg;        // [B, T] or null
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// First key tile (of `bn` keys) that a query tile starting at row q0 can see; `off` = T - S (bottom-right alignment).
__device__ __forceinline__ int first_key_tile(const Variant& v, int b, int q0, int S, int T, int bn, int n_tiles) {
  const int off = T - S;
  int lo = 0;
  if (v.window > 0) lo = max(0, (q0 + off - v.window + 1) / bn);
  if (v.q_seg != nullptr && v.k_seg != nullptr) {
    const int first = v.q_seg[static_cast<long long>(b) * S + min(q0, S - 1)];
    const int* ks = v.k_seg + static_cast<long long>(b) * T;
    // id 0 marks padding, which may follow the last document: a tile that ends in padding is never skipped
    while (lo < n_tiles) {
      const int last = ks[min(lo * bn + bn - 1, T - 1)];
      if (last == 0 || last >= first) break;
      ++lo;
    }
  }
  return min(lo, n_tiles);
}

// One past the last query block (of `bq` rows) that can see any key of the tile [kv0, kv0 + bkv).
__device__ __forceinline__ int end_query_block(const Variant& v, int b, int kv0, int bkv, int S, int T, int bq) {
  const int off = T - S;
  int hi = (S + bq - 1) / bq;
  if (v.window > 0) hi = min(hi, (min(S, kv0 + bkv - 1 + v.window - off) + bq - 1) / bq);
  if (v.q_seg != nullptr && v.k_seg != nullptr) {
    const int last = v.k_seg[static_cast<long long>(b) * T + min(kv0 + bkv - 1, T - 1)];
    const int* qs = v.q_seg + static_cast<long long>(b) * S;
    if (last != 0) {                   // a key tile that ends in padding (id 0) keeps every query block
      while (hi > 0 && qs[min((hi - 1) * bq, S - 1)] > last) --hi;
    }
  }
  return max(hi, 0);
}

}  // namespace attn
}  // namespace dewb
