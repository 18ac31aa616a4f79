// Rotary position encoding of q and k and the write of k, v into cache pages.
//
// Rotation (crates/ai-engine-runtime/src/arch/rope.rs:38-44,66-106), split halves:
//   ang = float(pos) * inv_freq[i]                      (float32)
//   out[i]        = x[i] * cos(ang) - x[i + d/2] * sin(ang)
//   out[i + d/2]  = x[i] * sin(ang) + x[i + d/2] * cos(ang)
// `inv_freq` (rot_dim/2 floats) is a parameter, so another scaling rule or a
// partial rotation (rot_dim < d) is another vector, not another kernel.
// k (rotated) and v go to page block_table[row][pos / P], slot pos % P of the
// layer's pool, laid out [page][kv_head][slot][d]
// (the reference writes them token by token, crates/ai-engine-candle/src/paged/attention.rs:59-83).
#include "common.cuh"

template <typename A, typename C>
__global__ void rope_kv_write_kernel(const A* __restrict__ qkv, A* __restrict__ q_out,
                                     C* __restrict__ k_pages, C* __restrict__ v_pages,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_req,
                                     const int* __restrict__ block_table, int bt_width,
                                     int num_pages, int P, int H, int K, int d, int rot_dim,
                                     const float* __restrict__ inv_freq, int write,
                                     unsigned* err) {
    extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        float s, c;
        sincosf(ang, &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    const int row = token_req[t];
    const int pidx = pos / P;
    int page = (write && pidx < bt_width && pos >= 0) ? block_table[(size_t)row * bt_width + pidx] : -1;
    const bool page_ok = page >= 0 && page < num_pages;   // write == 0: the pages are another run's, q only
    if (write && !page_ok && threadIdx.x == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
    const int slot = pos % P;
    const int qkv_w = (H + 2 * K) * d;
    const A* src = qkv + (size_t)t * qkv_w;

    // q heads and k heads: rotate pairs (i, i + half) for i < half, copy the rest
    const int hd2 = d - half;  // per head: `half` rotated pairs + (d - rot_dim) passthrough
    for (int idx = threadIdx.x; idx < (H + K) * hd2; idx += blockDim.x) {
        const int head = idx / hd2, i = idx % hd2;
        const A* x = src + (size_t)head * d;
        if (i < half) {
            const float x1 = to_f32<A>(x[i]), x2 = to_f32<A>(x[i + half]);
            const float c = cs[i], s = cs[half + i];
            const float o1 = x1 * c - x2 * s;
            const float o2 = x1 * s + x2 * c;
            if (head < H) {
                A* q = q_out + ((size_t)t * H + head) * d;
                q[i] = from_f32<A>(o1);
                q[i + half] = from_f32<A>(o2);
            } else if (page_ok) {
                C* k = k_pages + (((size_t)page * K + (head - H)) * P + slot) * d;
                k[i] = from_f32<C>(o1);
                k[i + half] = from_f32<C>(o2);
            }
        } else {
            const int e = rot_dim + (i - half);  // passthrough element
            const float v = to_f32<A>(x[e]);
            if (head < H)
                q_out[((size_t)t * H + head) * d + e] = from_f32<A>(v);
            else if (page_ok)
                k_pages[(((size_t)page * K + (head - H)) * P + slot) * d + e] = from_f32<C>(v);
        }
    }
    if (page_ok) {
        const A* vs = src + (size_t)(H + K) * d;
        for (int idx = threadIdx.x; idx < K * d; idx += blockDim.x) {
            const int kh = idx / d, e = idx % d;
            v_pages[(((size_t)page * K + kh) * P + slot) * d + e] = from_f32<C>(to_f32<A>(vs[idx]));
        }
    }
}

extern "C" int aie_rope_kv_write(const void* qkv, void* q_out, void* k_pages, void* v_pages,
                                 int dtype, const int* positions, const int* token_req,
                                 const int* block_table, int bt_width, int num_pages, int P, int T,
                                 int H, int K, int d, int rot_dim, const float* inv_freq,
                                 int write, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot_dim % 2 || rot_dim > d || rot_dim < 0) return AIE_BAD_ARG;
    const size_t smem = (size_t)rot_dim * sizeof(float);
    if (dtype == AIE_F32)
        rope_kv_write_kernel<float, float><<<T, 256, smem, stream>>>(
            (const float*)qkv, (float*)q_out, (float*)k_pages, (float*)v_pages, positions, token_req,
            block_table, bt_width, num_pages, P, H, K, d, rot_dim, inv_freq, write, err);
    else if (dtype == AIE_BF16)
        rope_kv_write_kernel<bf16, bf16><<<T, 256, smem, stream>>>(
            (const bf16*)qkv, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, positions, token_req,
            block_table, bt_width, num_pages, P, H, K, d, rot_dim, inv_freq, write, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
