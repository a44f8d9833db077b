/* Allocation-free entry point of libgllm_kernels.so.
 *
 * This entry point has no counterpart in the reference engine. It exists for callers that are not
 * allowed to allocate device memory at the moment they need attention: hosts that embed the library
 * behind a fixed memory plan (every byte of HBM is handed out at start-up, so a late cudaMalloc
 * either fails or breaks the plan), plug-ins running on a thread or callback where the owning
 * framework forbids calls into its allocator, and real-time loops where an allocator call is an
 * unbounded stall.
 *
 * gllm_paged_decode_noalloc() is the split-KV paged flash-decode kernel (same math as
 * gllm_paged_decode) whose scratch — the per-split partial outputs, their log-sum-exps and the ticket
 * counters — lives in a file-scope `static __device__` array inside the library instead of caller
 * memory. Every GPU that loads the library holds that array (about 8.3 MB) until the process exits.
 *
 * Limits:   batch * n_q_heads * max_splits <= GLLM_NOALLOC_MAX_UNITS
 *           batch * n_kv_heads             <= GLLM_NOALLOC_MAX_COUNTERS
 *           head_dim 128, 16-token pages, bf16 (as gllm_paged_decode)
 * A call beyond these limits returns -1 and gllm_last_error() says which limit was exceeded.
 *
 * The first call on a device looks up the device address of the scratch array
 * (cudaGetSymbolAddress) and raises the kernel's shared-memory limit; make that first call before any
 * stream capture begins. The call itself performs no cudaMalloc / cudaFree and calls no allocating
 * library routine. The ticket counters are cleared on the caller's stream at the start of every call.
 *
 * All calls on a device share the one scratch array, which keeps whatever the previous call left in
 * it: two calls whose kernels can overlap on the GPU (different streams, or graph branches) race on
 * it. Serialise them on one stream.
 *
 * Inputs and outputs are still caller memory (device pointers), exactly as for gllm_paged_decode:
 *   q, out        [batch, n_q_heads, 128] bf16
 *   kv_cache      [num_pages, 2, n_kv_heads, 16, 128] bf16
 *   block_tables  [batch, max_blocks] int32, ctx_lens [batch] int32 (<= 0 marks an empty slot)
 *   sinks         [n_q_heads] fp32 or NULL; window 0 = full attention; stream is a cudaStream_t
 * Returns 0 on success.
 *
 * Errors found by the kernel itself (a block-table entry outside the pool is redirected to page 0, a
 * context longer than the block table is cut to it, a page copy that never arrives is abandoned after a
 * bounded wait) do not show in that return value: the launch is asynchronous. They are recorded in a
 * status word of this path's own, separate from the one gllm_check_error() reads.
 * gllm_paged_decode_noalloc_status(stream) copies that word to the host on `stream`, WAITS for the
 * stream, and returns it (0 = no problem; otherwise one of the library's status codes: 1 page copy timed
 * out, 6 page id outside the pool, 9 context longer than the block table; -1 if the read itself failed).
 * A non-zero word is cleared by the read, so one bad call is reported once. It allocates nothing either.
 * Call it after the calls you want checked, outside any stream capture.
 *
 * The first call on a device may come from any thread: the one-time set-up is guarded by a mutex.
 */
#ifndef GLLM_NOALLOC_H_
#define GLLM_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define GLLM_NOALLOC_MAX_UNITS 16384    /* batch * n_q_heads * max_splits */
#define GLLM_NOALLOC_MAX_COUNTERS 4096  /* batch * n_kv_heads */

int gllm_paged_decode_noalloc(const void* q, void* out, const void* kv_cache, int num_pages,
                              const int* block_tables, int max_blocks, const int* ctx_lens, int batch,
                              int n_q_heads, int n_kv_heads, float scale, int pages_per_split, int max_splits,
                              int window, const float* sinks, void* stream);

int gllm_paged_decode_noalloc_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GLLM_NOALLOC_H_ */
