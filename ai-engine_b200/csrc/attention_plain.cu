// Plain paged attention: one block per (query token, query head) — all T tokens of
// the step, or the T tokens named by `token_list`; keys are read
// from the layer's pages through the request's block table.  It serves the
// float32 path of the engine and is the reference the fast kernels are checked
// against.  Formula (crates/ai-engine-runtime/src/arch/attention.rs:148-157,
// 177-196, 203-224): query head h reads kv head h / (H/K); s = (q.k) * scale;
// key j is seen by a query at position p iff j <= p (and j > p - window when
// the layer has a window); softmax over keys in float32; out = p.v.
//
// Keys are taken in chunks of 128 that start at multiples of 128 of the
// absolute key position, with a running maximum and sum, so the order of every
// addition depends on the query's position only — not on how the prompt was cut
// into steps or on what else is in the batch.
#include "common.cuh"

#define PLAIN_CHUNK 128

template <typename A, typename C>
__global__ void __launch_bounds__(PLAIN_CHUNK)
paged_attention_plain_kernel(const A* __restrict__ q, const C* __restrict__ k_pages,
                             const C* __restrict__ v_pages, A* __restrict__ out,
                             const int* __restrict__ positions, const int* __restrict__ token_req,
                             const int* __restrict__ block_table, int bt_width, int num_pages,
                             int P, int H, int K, int d, int window, float scale,
                             const int* __restrict__ token_list, unsigned* err) {
    extern __shared__ __align__(16) float sm[];
    float* q_s = sm;                                  // d
    float* p_s = q_s + d;                             // CHUNK
    float* red = p_s + PLAIN_CHUNK;                   // 32
    long long* off_s = (long long*)(red + 32);        // CHUNK  (8-byte aligned: d is a multiple of 2)

    const int t = token_list ? token_list[blockIdx.x] : blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const int row = token_req[t];
    const int kvh = h / (H / K);
    for (int e = tid; e < d; e += blockDim.x) q_s[e] = to_f32<A>(q[((size_t)t * H + h) * d + e]);
    __syncthreads();

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;  // output elements tid and tid + 128 (d <= 256)

    for (int c0 = (lo / PLAIN_CHUNK) * PLAIN_CHUNK; c0 <= pos; c0 += PLAIN_CHUNK) {
        const int kp = c0 + tid;
        const bool valid = kp >= lo && kp <= pos;
        float s = -INFINITY;
        long long off = -1;
        if (valid) {
            const int pidx = kp / P;
            const int page = pidx < bt_width ? block_table[(size_t)row * bt_width + pidx] : -1;
            if (page < 0 || page >= num_pages) {
                atomicOr(err, AIE_DEV_PAGE_OOB);
            } else {
                off = (((long long)page * K + kvh) * P + (kp % P)) * d;
                const C* kr = k_pages + off;
                float dot = 0.f;
                for (int e = 0; e < d; ++e) dot += q_s[e] * to_f32<C>(kr[e]);
                s = dot * scale;
            }
        }
        off_s[tid] = off;
        const float cmax = block_max(s, red);
        const float m_new = fmaxf(m, cmax);
        // every chunk visited holds at least one visible key unless a page was bad
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        const float csum = block_sum(p, red);   // has __syncthreads inside: p_s, off_s visible
        l = l * corr + csum;
        m = m_new;
        acc0 *= corr;
        acc1 *= corr;
        const int n = min(PLAIN_CHUNK, pos - c0 + 1);
        for (int j = 0; j < n; ++j) {
            const long long o = off_s[j];
            if (o < 0) continue;
            const float pj = p_s[j];
            if (tid < d) acc0 += pj * to_f32<C>(v_pages[o + tid]);
            if (tid + PLAIN_CHUNK < d) acc1 += pj * to_f32<C>(v_pages[o + tid + PLAIN_CHUNK]);
        }
        __syncthreads();
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    A* o = out + ((size_t)t * H + h) * d;
    if (tid < d) o[tid] = from_f32<A>(acc0 * inv);
    if (tid + PLAIN_CHUNK < d) o[tid + PLAIN_CHUNK] = from_f32<A>(acc1 * inv);
}

extern "C" int aie_paged_attention_plain(const void* q, const void* k_pages, const void* v_pages,
                                         void* out, int dtype, const int* positions,
                                         const int* token_req, const int* block_table, int bt_width,
                                         int num_pages, int P, int T, int H, int K, int d, int window,
                                         float scale, const int* token_list, unsigned* err,
                                         cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > 2 * PLAIN_CHUNK || (d % 2) || K <= 0 || H % K) return AIE_UNSUPPORTED;
    const size_t smem = (size_t)(d + PLAIN_CHUNK + 32) * sizeof(float) + PLAIN_CHUNK * sizeof(long long);
    if (H > 65535) return AIE_UNSUPPORTED;
    dim3 grid(T, H);
    if (dtype == AIE_F32)
        paged_attention_plain_kernel<float, float><<<grid, PLAIN_CHUNK, smem, stream>>>(
            (const float*)q, (const float*)k_pages, (const float*)v_pages, (float*)out, positions,
            token_req, block_table, bt_width, num_pages, P, H, K, d, window, scale, token_list, err);
    else if (dtype == AIE_BF16)
        paged_attention_plain_kernel<bf16, bf16><<<grid, PLAIN_CHUNK, smem, stream>>>(
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, positions,
            token_req, block_table, bt_width, num_pages, P, H, K, d, window, scale, token_list, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
