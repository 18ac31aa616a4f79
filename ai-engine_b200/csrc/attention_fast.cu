// bfloat16 paged attention for serving: a split-KV kernel for requests that bring
// one token (decode), and a reduce kernel that joins the splits.
//
// Decode.  One CTA handles one request, one kv head and up to eight of the query
// heads that share it (so each key and value is read once for the group), over
// one contiguous part of the request's keys (a "split"; the host picks the number
// of splits so that the grid fills the machine however few requests there are).
// Each of its four warps runs a pipeline of its own: 16-key tiles of keys and
// values are gathered page by page into the warp's ring of shared-memory stages
// with 16-byte cp.async copies (XOR-swizzled for ldmatrix), three or four tiles
// ahead of the arithmetic, so the memory system always has work in flight and no
// warp waits on a block-table lookup (the CTA reads its block-table entries once,
// up front).  The group's query heads are the rows of a 16-row mma.sync tile
// (bf16 in, float32 accumulate): q.k for a tile is 2 x D/16 multiplies, p.v D/8;
// the running maximum and sum are float32 (online softmax).  Warps and then splits
// are merged with the usual (max, sum) rescaling; all softmax arithmetic is float32.
// Formula: crates/ai-engine-runtime/src/arch/attention.rs:148-157,177-196,203-224.
#include "common.cuh"
#include "attention_decode.cuh"

// Scratch (S > 1): part_o [n_dec * H * S * D] floats, part_lse [n_dec * H * S] floats.
// counters (optional): n_dec * K * ceil(G / 8) ints that are zero; with them the parts are joined
// by whichever CTA finishes last (and the counters are zero again afterwards); without them a
// second kernel joins the parts.
extern "C" int aie_paged_attention_decode(const void* q, const void* k_pages, const void* v_pages, void* out,
                                          float* part_o, float* part_lse, const int* dec_tokens, int n_dec,
                                          const int* positions, const int* token_req, const int* block_table,
                                          int bt_width, int num_pages, int P, int H, int K, int d, int window,
                                          float scale, int S, int* counters, unsigned* err,
                                          cudaStream_t stream) {
    if (n_dec <= 0) return 0;
    if (K <= 0 || H % K || S < 1) return AIE_BAD_ARG;
    if (d != 64 && d != 128) return AIE_UNSUPPORTED;
    if (S > 1 && (!part_o || !part_lse)) return AIE_BAD_ARG;
    if (S > DEC_MAX_SPLITS) return AIE_UNSUPPORTED;
    const int G = H / K;
    const int GC = G >= DEC_HEADS ? DEC_HEADS : G;
    const int gchunks = (G + GC - 1) / GC;
    if (K * gchunks > 65535 || n_dec > 65535) return AIE_UNSUPPORTED;
    if ((bt_width + S - 1) / S + 2 > DEC_MAX_PAGES) return AIE_UNSUPPORTED;   // more splits needed
    dim3 grid(S, K * gchunks, n_dec);
    int rc;
    if (d == 64)
        rc = launch_decode<64>(GC, grid, stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages,
                               (bf16*)out, part_o, part_lse, dec_tokens, positions, token_req, block_table,
                               bt_width, num_pages, P, H, K, G, window, scale, S, counters, err);
    else
        rc = launch_decode<128>(GC, grid, stream, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages,
                                (bf16*)out, part_o, part_lse, dec_tokens, positions, token_req, block_table,
                                bt_width, num_pages, P, H, K, G, window, scale, S, counters, err);
    if (rc) return rc;
    if (S > 1 && counters == nullptr) {
        dim3 rg(n_dec, H);
        launch_pdl(decode_reduce_kernel, rg, dim3(d < 128 ? 64 : 128), 0, stream, (const float*)part_o, (const float*)part_lse, (bf16*)out, dec_tokens, H, d, S);
    }
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
#include "attention_prefill.cuh"

// tiles: [n_tiles][2] = (request row, offset of the 128-token tile within the request's tokens)
extern "C" int aie_paged_attention_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                                           const int* tiles, int n_tiles, const int* q_start, const int* q_len,
                                           const int* ctx_len, const int* block_table, int bt_width,
                                           int num_pages, int P, int H, int K, int d, int window, float scale,
                                           unsigned* err, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (K <= 0 || H % K) return AIE_BAD_ARG;
    if (d != 64 && d != 128) return AIE_UNSUPPORTED;
    if (n_tiles > 65535) return AIE_UNSUPPORTED;
    dim3 grid(H, n_tiles);
    if (d == 64) {
        const size_t smem = prefill_smem_bytes<64>();
        cudaFuncSetAttribute(paged_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        paged_prefill_kernel<64><<<grid, PF_WARPS * 32, smem, stream>>>(
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, tiles, q_start, q_len, ctx_len,
            block_table, bt_width, num_pages, P, H, K, window, scale, err);
    } else {
        const size_t smem = prefill_smem_bytes<128>();
        cudaFuncSetAttribute(paged_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        paged_prefill_kernel<128><<<grid, PF_WARPS * 32, smem, stream>>>(
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, tiles, q_start, q_len, ctx_len,
            block_table, bt_width, num_pages, P, H, K, window, scale, err);
    }
    AIE_LAUNCH_CHECK();
}
