/* dewb_noalloc.h - an RMSNorm backward entry point that allocates nothing.
 *
 * This entry point has no counterpart in the reference framework; it exists for callers of this library that are
 * not allowed to allocate device memory at the time they call it.
 *
 * Who cannot allocate, and why: code that runs inside a fixed memory plan - a serving process whose device memory
 * was carved up at start-up and handed out to model weights and the KV-cache pool, a real-time control loop where a
 * call into the allocator is an unbounded stall, a plugin loaded by a host application that owns the GPU's memory and
 * forbids cudaMalloc from plugin code, or an allocator hook itself.  The ordinary entry point
 * (dewb_rmsnorm_bwd) asks its caller for a scratch buffer of dewb_rmsnorm_bwd_blocks(rows) x d floats, which
 * such callers have no way to obtain on demand.
 *
 * What this one does instead: the partial sums of the weight gradient live in one file-scope
 *     static __device__ __align__(256) float  array of  DEWB_NOALLOC_MAX_SPLITS x DEWB_NOALLOC_MAX_D  floats
 * (148 x 4096 x 4 bytes = 2,424,832 bytes) inside the library.  Every GPU that loads the library holds that array
 * until the process exits.  The caller still passes every input and output.
 *
 * Rules of use:
 *   - d must be a multiple of 8 and at most DEWB_NOALLOC_MAX_D; larger rows are rejected with
 *     DEWB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and remembers it; make that first call before any stream capture begins.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left in it.  Every call
 *     overwrites the part it reads before reading it, so calls that run one after another are independent; two calls
 *     that overlap on the GPU (different streams without an ordering between them) race on the array and must be
 *     ordered by the caller.
 *   - `device` is made the current CUDA device for the whole call (the address look-up and every launch) and the
 *     caller's current device is put back before the call returns, so the caller need not have `device` current;
 *     `stream` must belong to `device` (null selects its default stream).
 *   - Host threads: the first calls on a device may come from several threads at once (they all store the same
 *     address); after that the entry point keeps no host-side state.  The rule on overlapping GPU work above still holds.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on the first call or any later one.
 */
#ifndef DEWB_NOALLOC_H_
#define DEWB_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define DEWB_NOALLOC_MAX_D 4096
#define DEWB_NOALLOC_MAX_SPLITS 148
#define DEWB_NOALLOC_ERR_TOO_LARGE (-20)
#define DEWB_NOALLOC_ERR_SYMBOL (-21)

/* Backward of y = x * rsqrt(mean(x^2) + eps) * w over `rows` rows of width `d` (bf16 tensors, fp32 rstd saved by the
 * forward).  Writes dx [rows, d] (bf16) and dw [d] (fp32 in dw_f32 and / or bf16 in dw_bf16; either may be null;
 * `accumulate` != 0 adds into them).  `dres` (optional, bf16 [rows, d]) is added into dx.  `device` is the CUDA device
 * the pointers live on; `stream` is a cudaStream_t.  Returns 0 on success, a negative DEWB_NOALLOC_ERR_* code for a
 * rejected call, or a positive cudaError_t. */
int dewb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                             void* dx, float* dw_f32, void* dw_bf16, int accumulate, long long rows, int d, int device,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DEWB_NOALLOC_H_ */
