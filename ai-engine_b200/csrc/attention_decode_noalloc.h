/* Split-KV decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in einyx/ai-engine; it exists for users of
 * this library, not for parity with the reference.
 *
 * Who needs it.  Some programs that link this library cannot call cudaMalloc, or
 * any routine that allocates on the device, at the moment they need attention:
 * a host that sized every device buffer at start-up and gave the rest of the
 * GPU's memory away (an allocation there can fail, and even when it succeeds it
 * may synchronise the whole device and stall the other streams); a plain C or
 * C++ caller that has no torch allocator to borrow scratch from; a latency-bound
 * loop whose owner has ruled out allocator calls on its hot path.  The regular
 * entry point, aie_paged_attention_decode, asks such a caller for two scratch
 * buffers whenever the keys are cut into more than one part.  This variant asks
 * for none: its scratch is a fixed array that lives in the library's device image.
 *
 * What it computes.  Exactly what aie_paged_attention_decode computes, with the
 * same kernels: for every token listed in dec_tokens (a request that brings one
 * token), softmax(q.k * scale over the visible keys) . v, read through the block
 * table, written to out[t, h, :] in bfloat16.  Inputs and outputs are the
 * caller's own device buffers, as before.
 *
 * The limit.  The scratch holds AIE_NOALLOC_SCRATCH_FLOATS floats (16 MiB), and
 * every GPU whose context loads this library keeps those 16 MiB until the process
 * exits.  A call with S > 1 needs n_dec * H * S * (d + 1) floats; a call that
 * needs more returns AIE_TOO_LARGE (-3) and launches nothing.  S == 1 needs no
 * scratch and is never refused for size.
 *
 * First call on a device.  The first call made while a given device is current
 * looks up the device address of the scratch array (cudaGetSymbolAddress) and
 * keeps it; later calls on that device reuse it.  Make that first call before
 * any stream capture on the device, and not from two threads at once.
 *
 * Sharing.  Every call on a device uses the same array, and the array keeps what
 * the last call left in it.  Nothing in it has to start at zero: each call writes
 * every element that its own reduce step reads.  Two calls whose kernels can be
 * in flight on the GPU at the same time (different streams, or different host
 * threads) race on the array and give wrong results; issue them on one stream or
 * order them with events.
 *
 * It calls no cudaMalloc, cudaFree or other allocating routine.  Return value: 0,
 * a negative AIE_* refusal, or a positive cudaError_t.
 */
#pragma once
#include <cuda_runtime.h>

#define AIE_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define AIE_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif

int aie_paged_attention_decode_noalloc(
    const void* q,            /* bf16 [T, H, d] queries, already rotated */
    const void* k_pages,      /* bf16 [num_pages, K, P, d] */
    const void* v_pages,      /* bf16 [num_pages, K, P, d] */
    void* out,                /* bf16 [T, H, d]; rows of the listed tokens are written */
    const int* dec_tokens,    /* [n_dec] token indices t */
    int n_dec,
    const int* positions,     /* [T] absolute position of each token */
    const int* token_req,     /* [T] row of the block table for each token */
    const int* block_table,   /* [rows, bt_width] page ids, -1 where none */
    int bt_width, int num_pages, int P, int H, int K, int d,
    int window,               /* 0: all keys; w: keys in (pos - w, pos] */
    float scale,
    int S,                    /* parts each request's keys are cut into */
    unsigned* err,            /* device error word (AIE_DEV_* bits) */
    cudaStream_t stream);

#ifdef __cplusplus
}
#endif
