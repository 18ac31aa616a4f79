// The allocation-free variant of the split-KV decode attention: the same kernels
// as aie_paged_attention_decode, with the scratch for the parts in a static device
// array of this file instead of buffers from the caller.  See
// attention_decode_noalloc.h for who it is for, its limit and its rules of use.
#include "attention_decode_noalloc.h"

#include "attention_decode.cuh"

// The scratch.  In host code this name is only a stand-in for the symbol, not a
// device address: handing it to a kernel would make the kernel fault or, where the
// GPU can reach host memory, quietly use the wrong memory.  Host code below gets
// the real address once per device with cudaGetSymbolAddress and passes that.
static __device__ __align__(256) float g_decode_scratch[AIE_NOALLOC_SCRATCH_FLOATS];

#define AIE_NOALLOC_MAX_DEVICES 64
static float* g_scratch_addr[AIE_NOALLOC_MAX_DEVICES];   // per device, filled on first use

extern "C" int aie_paged_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                                  void* out, const int* dec_tokens, int n_dec,
                                                  const int* positions, const int* token_req,
                                                  const int* block_table, int bt_width, int num_pages, int P,
                                                  int H, int K, int d, int window, float scale, int S,
                                                  unsigned* err, cudaStream_t stream) {
    if (n_dec <= 0) return 0;
    if (K <= 0 || H <= 0 || H % K || S < 1) return AIE_BAD_ARG;
    if (d != 64 && d != 128) return AIE_UNSUPPORTED;
    const int G = H / K;
    const int GC = G >= DEC_HEADS ? DEC_HEADS : G;
    const int gchunks = (G + GC - 1) / GC;
    if (K * gchunks > 65535 || n_dec > 65535) return AIE_UNSUPPORTED;
    if ((bt_width + S - 1) / S + 2 > DEC_MAX_PAGES) return AIE_UNSUPPORTED;   // more splits needed
    if (S > DEC_MAX_SPLITS) return AIE_UNSUPPORTED;

    float* part_o = nullptr;
    float* part_lse = nullptr;
    if (S > 1) {
        const long long slots = (long long)n_dec * H * S;
        const long long need = slots * (d + 1);
        if (need > (long long)AIE_NOALLOC_SCRATCH_FLOATS) return AIE_TOO_LARGE;
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= AIE_NOALLOC_MAX_DEVICES) return AIE_UNSUPPORTED;
        if (g_scratch_addr[dev] == nullptr) {   // set-up: once per device, with that device current
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_decode_scratch);
            if (e != cudaSuccess) return (int)e;
            g_scratch_addr[dev] = static_cast<float*>(p);
        }
        part_o = g_scratch_addr[dev];            // [n_dec * H * S * d]
        part_lse = part_o + slots * d;           // [n_dec * H * S]
    }

    dim3 grid(S, K * gchunks, n_dec);
    int rc;
    if (d == 64)
        rc = launch_decode<64>(GC, grid, stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages,
                               (bf16*)out, part_o, part_lse, dec_tokens, positions, token_req, block_table,
                               bt_width, num_pages, P, H, K, G, window, scale, S, nullptr, err);
    else
        rc = launch_decode<128>(GC, grid, stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages,
                                (bf16*)out, part_o, part_lse, dec_tokens, positions, token_req, block_table,
                                bt_width, num_pages, P, H, K, G, window, scale, S, nullptr, err);
    if (rc) return rc;
    if (S > 1) {
        // every (token, head, part) slot of the scratch that this reduce reads was
        // written by the launch above, so stale contents of earlier calls are never seen
        dim3 rg(n_dec, H);
        launch_pdl(decode_reduce_kernel, rg, dim3(d < 128 ? 64 : 128), 0, stream, (const float*)part_o, (const float*)part_lse, (bf16*)out, dec_tokens, H, d, S);
    }
    return (int)cudaGetLastError();
}
