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

// I: dtype of qkv (the compute dtype, or float32 parts of a split product that are added here);
// A: dtype of q_out; C: dtype of the cache.
template <typename I, typename A, typename C>
__global__ void rope_kv_write_kernel(const I* __restrict__ qkv, int parts, size_t part_stride,
                                     A* __restrict__ q_out,
                                     C* __restrict__ k_pages, C* __restrict__ v_pages,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_req,
                                     const int* __restrict__ block_table, int bt_width,
                                     int num_pages, int P, int H, int K, int d, int rot_dim,
                                     const float* __restrict__ inv_freq, int write,
                                     unsigned* err) {
    // one warp per (token, head slot): slots [0, H) are q heads, [H, H+K) k heads,
    // [H+K, H+2K) v heads; lanes walk the head's rotated pairs, then its other elements
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, slot_h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (slot_h >= H + 2 * K) return;
    const int lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int half = rot_dim / 2;
    const I* x = qkv + (size_t)t * (H + 2 * K) * d + (size_t)slot_h * d;
    auto in = [&](int e) {
        float v = to_f32<I>(x[e]);
        for (int p = 1; p < parts; ++p) v += to_f32<I>(x[p * part_stride + e]);
        return v;
    };
    const bool is_q = slot_h < H, is_v = slot_h >= H + K;
    if (!is_q && !write) return;     // the pages are another run's: q only
    A* qo = nullptr;
    C* ko = nullptr;
    if (is_q) {
        qo = q_out + ((size_t)t * H + slot_h) * d;
    } else {
        const int row = token_req[t];
        const int pidx = pos / P;
        const int page = (pidx < bt_width && pos >= 0) ? block_table[(size_t)row * bt_width + pidx] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
            return;
        }
        const int kh = is_v ? slot_h - H - K : slot_h - H;
        ko = (is_v ? v_pages : k_pages) + (((size_t)page * K + kh) * P + (pos % P)) * d;
    }
    if (is_v) {
        for (int e = lane; e < d; e += 32) ko[e] = from_f32<C>(in(e));
        return;
    }
    for (int i = lane; i < half; i += 32) {
        const float ang = (float)pos * inv_freq[i];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float x1 = in(i), x2 = in(i + half);
        const float o1 = x1 * cs - x2 * sn;
        const float o2 = x1 * sn + x2 * cs;
        if (is_q) {
            qo[i] = from_f32<A>(o1);
            qo[i + half] = from_f32<A>(o2);
        } else {
            ko[i] = from_f32<C>(o1);
            ko[i + half] = from_f32<C>(o2);
        }
    }
    for (int e = rot_dim + lane; e < d; e += 32) {      // elements that are not rotated
        const float v = in(e);
        if (is_q) qo[e] = from_f32<A>(v);
        else ko[e] = from_f32<C>(v);
    }
}

// Eight consecutive elements as floats (the address is 8-element aligned).
__device__ __forceinline__ void load8(const bf16* p, float* f) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&a);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(e[i]);
}
__device__ __forceinline__ void load8(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}
__device__ __forceinline__ void store8(bf16* p, const float* f) {
    uint4 o;
    bf16* e = reinterpret_cast<bf16*>(&o);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = __float2bfloat16_rn(f[i]);
    *reinterpret_cast<uint4*>(p) = o;
}

// Portions of prompts with a bfloat16 cache: one block per token.  The token's angles are computed once
// (float32, the same expression as above) and kept in shared memory; every thread rotates 8 pairs
// of one head with 16-byte loads and stores.  The projection comes in bfloat16 or in float32 (the
// product's accumulators, so that q and k are rounded once, after the rotation, as in small steps).
// Needs rot_dim % 16 == 0 and d % 8 == 0.
template <typename I>
__global__ void __launch_bounds__(256)
rope_kv_write_token_kernel(const I* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ k_pages,
                           bf16* __restrict__ v_pages, const int* __restrict__ positions,
                           const int* __restrict__ token_req, const int* __restrict__ block_table, int bt_width,
                           int num_pages, int P, int H, int K, int d, int rot_dim,
                           const float* __restrict__ inv_freq, int write, unsigned* err) {
    extern __shared__ float rope_cs[];       // [half] cosines, [half] sines
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[t];
    const int half = rot_dim / 2;
    for (int i = tid; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        rope_cs[i] = cs;
        rope_cs[half + i] = sn;
    }
    int page = -1;
    if (write) {
        const int pidx = pos / P;
        page = (pidx < bt_width && pos >= 0) ? block_table[(size_t)token_req[t] * bt_width + pidx] : -1;
        if (page < 0 || page >= num_pages) {
            if (tid == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
            page = -1;
        }
    }
    __syncthreads();
    const I* x = qkv + (size_t)t * (H + 2 * K) * d;
    const size_t slot = page >= 0 ? ((size_t)page * K * P + (pos % P)) * d : 0;      // + kv head * P * d
    const int cph = half / 8, heads = H + (page >= 0 ? K : 0);
    for (int w = tid; w < heads * cph; w += blockDim.x) {
        const int head = w / cph, c = (w % cph) * 8;
        const I* src = x + (size_t)head * d + c;
        bf16* dst = head < H ? q_out + ((size_t)t * H + head) * d + c : k_pages + slot + (size_t)(head - H) * P * d + c;
        float x1[8], x2[8], o1[8], o2[8];
        load8(src, x1);
        load8(src + half, x2);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float cs = rope_cs[c + e], sn = rope_cs[half + c + e];
            o1[e] = x1[e] * cs - x2[e] * sn;
            o2[e] = x1[e] * sn + x2[e] * cs;
        }
        store8(dst, o1);
        store8(dst + half, o2);
    }
    // what is not rotated: the tails of q and k heads, and the v heads
    const int tail = (d - rot_dim) / 8;
    for (int w = tid; w < heads * tail; w += blockDim.x) {
        const int head = w / tail, c = rot_dim + (w % tail) * 8;
        bf16* dst = head < H ? q_out + ((size_t)t * H + head) * d + c : k_pages + slot + (size_t)(head - H) * P * d + c;
        float v[8];
        load8(x + (size_t)head * d + c, v);
        store8(dst, v);
    }
    if (page >= 0) {
        const int dc = d / 8;
        for (int w = tid; w < K * dc; w += blockDim.x) {
            const int kh = w / dc, c = (w % dc) * 8;
            float v[8];
            load8(x + (size_t)(H + K + kh) * d + c, v);
            store8(v_pages + slot + (size_t)kh * P * d + c, v);
        }
    }
}

extern "C" int aie_rope_kv_write(const void* qkv, int in_dtype, int parts, long long part_stride,
                                 void* q_out, void* k_pages, void* v_pages, int dtype, const int* positions, const int* token_req,
                                 const int* block_table, int bt_width, int num_pages, int P, int T,
                                 int H, int K, int d, int rot_dim, const float* inv_freq,
                                 int write, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot_dim % 2 || rot_dim > d || rot_dim < 0) return AIE_BAD_ARG;
    if (T >= 64 && dtype == AIE_BF16 && parts == 1 && rot_dim % 16 == 0 && d % 8 == 0 &&
        !((size_t)qkv & 15) && !((size_t)q_out & 15) && !((size_t)k_pages & 15) && !((size_t)v_pages & 15))
    {
        // one pass over the token's rotated chunks when they fit a block: (H + K) heads x rot_dim / 16 chunks
        int threads = ((H + K) * (rot_dim / 16) + 31) / 32 * 32;
        threads = threads < 64 ? 64 : (threads > 256 ? ((threads + 1) / 2 + 31) / 32 * 32 : threads);
        if (threads > 256) threads = 256;
        if (in_dtype == AIE_BF16)
            return (int)launch_pdl(rope_kv_write_token_kernel<bf16>, dim3(T), dim3(threads), (size_t)rot_dim * sizeof(float),
                                   stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, positions,
                                   token_req, block_table, bt_width, num_pages, P, H, K, d, rot_dim, inv_freq, write, err);
        if (in_dtype == AIE_F32)
            return (int)launch_pdl(rope_kv_write_token_kernel<float>, dim3(T), dim3(threads), (size_t)rot_dim * sizeof(float),
                                   stream, (const float*)qkv, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, positions,
                                   token_req, block_table, bt_width, num_pages, P, H, K, d, rot_dim, inv_freq, write, err);
    }
    // few tokens: one warp per block, so that the work spreads over the machine; many: 8 warps
    const int warps = T >= 256 ? 8 : 1;
    if ((H + 2 * K + warps - 1) / warps > 65535) return AIE_UNSUPPORTED;
    const dim3 grid(T, (H + 2 * K + warps - 1) / warps);
    const int threads = 32 * warps;
    if (parts < 1 || (parts > 1 && in_dtype != AIE_F32)) return AIE_BAD_ARG;
#define ARGS positions, token_req, block_table, bt_width, num_pages, P, H, K, d, rot_dim, inv_freq, write, err
    cudaError_t e;
    if (dtype == AIE_F32 && in_dtype == AIE_F32)
        e = launch_pdl(rope_kv_write_kernel<float, float, float>, grid, dim3(threads), 0, stream, (const float*)qkv,
                       parts, (size_t)part_stride, (float*)q_out, (float*)k_pages, (float*)v_pages, ARGS);
    else if (dtype == AIE_BF16 && in_dtype == AIE_BF16)
        e = launch_pdl(rope_kv_write_kernel<bf16, bf16, bf16>, grid, dim3(threads), 0, stream, (const bf16*)qkv,
                       parts, (size_t)part_stride, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, ARGS);
    else if (dtype == AIE_BF16 && in_dtype == AIE_F32)
        e = launch_pdl(rope_kv_write_kernel<float, bf16, bf16>, grid, dim3(threads), 0, stream, (const float*)qkv,
                       parts, (size_t)part_stride, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, ARGS);
    else
        return AIE_BAD_ARG;
#undef ARGS
    return (int)e;
}
