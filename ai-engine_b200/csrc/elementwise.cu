// Memory-bound row kernels: embedding gather, residual add fused with RMSNorm,
// SiLU(gate) * up, dtype casts.  The residual stream is float32 in both compute
// dtypes; statistics and scaling are float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// x[t, :] = float(E[ids[t], :])        (crates/ai-engine-runtime/src/arch/embedding.rs:14-20)
// ---------------------------------------------------------------------------
template <typename W>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const W* __restrict__ table,
                                    float* __restrict__ x, int D, int vocab, unsigned* err) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_TOKEN_OOB);
        for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)t * D + i] = 0.f;
        return;
    }
    const W* row = table + (size_t)id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)t * D + i] = to_f32<W>(row[i]);
}

// bf16 table, D a multiple of 8: 16-byte loads, two float4 stores per thread
__global__ void embed_gather_vec_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                        float* __restrict__ x, int D, int vocab, unsigned* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(err, AIE_DEV_TOKEN_OOB);
    const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * D);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)t * D);
    for (int i = threadIdx.x; i < D / 8; i += blockDim.x) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (ok) {
            const uint4 raw = row[i];
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
            a = make_float4(__bfloat162float(e[0]), __bfloat162float(e[1]), __bfloat162float(e[2]), __bfloat162float(e[3]));
            b = make_float4(__bfloat162float(e[4]), __bfloat162float(e[5]), __bfloat162float(e[6]), __bfloat162float(e[7]));
        }
        dst[2 * i] = a;
        dst[2 * i + 1] = b;
    }
}

extern "C" int aie_embed_gather(const int* ids, const void* table, int table_dtype, float* x,
                                int T, int D, int vocab, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (table_dtype == AIE_F32)
        embed_gather_kernel<float><<<T, 256, 0, stream>>>(ids, (const float*)table, x, D, vocab, err);
    else if (table_dtype == AIE_BF16 && D % 8 == 0)
        launch_pdl(embed_gather_vec_kernel, dim3(T), dim3(D >= 4096 ? 512 : 128), 0, stream, ids, (const bf16*)table, x, D, vocab, err);
    else if (table_dtype == AIE_BF16)
        embed_gather_kernel<bf16><<<T, 256, 0, stream>>>(ids, (const bf16*)table, x, D, vocab, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ids[t] = last[src[t]] where src[t] >= 0: a token that the previous step sampled and that the host
// has not read yet is taken from the device buffer the sampler left it in (no counterpart in the
// reference, whose loop reads every token back before the next step: crates/ai-engine-candle/src/paged/engine.rs:150-170)
__global__ void take_sampled_ids_kernel(int* __restrict__ ids, const int* __restrict__ src,
                                        const int* __restrict__ last, int T, int n_last, unsigned* err) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int k = src[t];
    if (k < 0) return;
    if (k >= n_last) {
        atomicOr(err, AIE_DEV_TOKEN_OOB);
        return;
    }
    ids[t] = last[k];
}

extern "C" int aie_take_sampled_ids(int* ids, const int* src, const int* last, int T, int n_last, unsigned* err,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    take_sampled_ids_kernel<<<(T + 127) / 128, 128, 0, stream>>>(ids, src, last, T, n_last, err);
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm (crates/ai-engine-runtime/src/arch/rmsnorm.rs:29-42):
//   s = x[row] (+ delta[row], or the sum of `parts` deltas `part_stride` elements apart);  ms = mean(s^2);  r = 1/sqrt(ms + eps);
//   out[i] = (s * r) * w          with eps inside the root and the weight last.
// `rows` (optional) picks input rows; `write_back` stores s into x.
// ---------------------------------------------------------------------------
template <typename A, typename W, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const A* __restrict__ delta,
                                   const W* __restrict__ w, O* __restrict__ out,
                                   const int* __restrict__ rows, int D, float eps, int write_back,
                                   int parts, size_t part_stride) {
    extern __shared__ float srow[];   // D floats + 32
    float* red = srow + D;
    const int o = blockIdx.x;
    const size_t r = rows ? (size_t)rows[o] : (size_t)o;
    float* xr = x + r * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float s = xr[i];
        if (delta)
            for (int p = 0; p < parts; ++p) s += to_f32<A>(delta[p * part_stride + r * D + i]);
        srow[i] = s;
        ss += s * s;
    }
    ss = block_sum(ss, red);
    const float ms = ss / (float)D;
    const float rinv = 1.0f / sqrtf(ms + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float s = srow[i];
        if (write_back) xr[i] = s;
        out[(size_t)o * D + i] = from_f32<O>((s * rinv) * to_f32<W>(w[i]));
    }
}

// Fast path: D a multiple of 4 and at most 4 * 1024: the whole row lives in registers
// (one float4 per thread), read once and written once.  Same arithmetic and the same
// block reduction as the general kernel.
template <typename A, typename W, typename O>
__global__ void __launch_bounds__(1024)
add_rmsnorm_row_kernel(float* __restrict__ x, const A* __restrict__ delta, const W* __restrict__ w,
                       O* __restrict__ out, const int* __restrict__ rows, int D, float eps, int write_back,
                       int parts, size_t part_stride) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int o = blockIdx.x;
    const size_t r = rows ? (size_t)rows[o] : (size_t)o;
    const int i = threadIdx.x;
    const bool on = i < D / 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) {
        s = reinterpret_cast<const float4*>(x + r * D)[i];
        if (delta) {
            // parts of a split product, added in order; four loads are in flight at a time
            const A* dp = delta + r * D + 4 * i;
            int p = 0;
            for (; p + 4 <= parts; p += 4) {
                float4 dl[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) dl[u] = load4<A>(dp + (size_t)(p + u) * part_stride);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    s.x += dl[u].x;
                    s.y += dl[u].y;
                    s.z += dl[u].z;
                    s.w += dl[u].w;
                }
            }
            for (; p < parts; ++p) {
                const float4 dl = load4<A>(dp + (size_t)p * part_stride);
                s.x += dl.x;
                s.y += dl.y;
                s.z += dl.z;
                s.w += dl.w;
            }
        }
    }
    float ss = s.x * s.x;
    ss += s.y * s.y;
    ss += s.z * s.z;
    ss += s.w * s.w;
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
    if (on) {
        if (write_back) reinterpret_cast<float4*>(x + r * D)[i] = s;
        const float4 wv = load4<W>(w + 4 * i);
        store4<O>(out + (size_t)o * D + 4 * i,
                  make_float4((s.x * rinv) * wv.x, (s.y * rinv) * wv.y, (s.z * rinv) * wv.z, (s.w * rinv) * wv.w));
    }
}

// Many rows (portions of prompts, bfloat16 out): a quarter of the threads per row, four float4 each, all loads
// issued before the first use, so that eight blocks sit on an SM and keep 128 KB of loads in flight (with a
// thread per float4 two blocks of 1,024 threads fit, and the memory system idles through their reductions).
template <typename A, typename W, typename O>
__global__ void __launch_bounds__(256)
add_rmsnorm_row4_kernel(float* __restrict__ x, const A* __restrict__ delta, const W* __restrict__ w,
                        O* __restrict__ out, const int* __restrict__ rows, int D, float eps, int write_back) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int o = blockIdx.x;
    const size_t r = rows ? (size_t)rows[o] : (size_t)o;
    const int i = threadIdx.x, nt = blockDim.x;       // D == 16 * nt
    float4 s[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) s[k] = reinterpret_cast<const float4*>(x + r * D)[i + k * nt];
    if (delta) {
        float4 dl[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) dl[k] = load4<A>(delta + r * D + 4 * (i + k * nt));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            s[k].x += dl[k].x;
            s[k].y += dl[k].y;
            s[k].z += dl[k].z;
            s[k].w += dl[k].w;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        ss += s[k].x * s[k].x;
        ss += s[k].y * s[k].y;
        ss += s[k].z * s[k].z;
        ss += s[k].w * s[k].w;
    }
    ss = block_sum(ss, red);
    const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (write_back) reinterpret_cast<float4*>(x + r * D)[i + k * nt] = s[k];
        const float4 wv = load4<W>(w + 4 * (i + k * nt));
        store4<O>(out + (size_t)o * D + 4 * (i + k * nt),
                  make_float4((s[k].x * rinv) * wv.x, (s[k].y * rinv) * wv.y, (s[k].z * rinv) * wv.z, (s[k].w * rinv) * wv.w));
    }
}

template <typename A, typename W>
static int launch_rmsnorm_o(float* x, const void* delta, const void* w, void* out, int out_dtype,
                            const int* rows, int n, int D, float eps, int write_back, int parts,
                            size_t part_stride, cudaStream_t stream) {
    if (n >= 256 && parts == 1 && out_dtype == AIE_BF16 && D % 512 == 0 && D <= 4096) {
        launch_pdl(add_rmsnorm_row4_kernel<A, W, bf16>, dim3(n), dim3(D / 16), 0, stream, x, (const A*)delta, (const W*)w,
                   (bf16*)out, rows, D, eps, write_back);
        AIE_LAUNCH_CHECK();
    }
    if (D % 4 == 0 && D <= 4096) {
        const int threads = ((D / 4) + 31) / 32 * 32;
        if (out_dtype == AIE_F32)
            launch_pdl(add_rmsnorm_row_kernel<A, W, float>, dim3(n), dim3(threads), 0, stream, x, (const A*)delta, (const W*)w, (float*)out, rows, D, eps, write_back, parts, part_stride);
        else if (out_dtype == AIE_BF16)
            launch_pdl(add_rmsnorm_row_kernel<A, W, bf16>, dim3(n), dim3(threads), 0, stream, x, (const A*)delta, (const W*)w, (bf16*)out, rows, D, eps, write_back, parts, part_stride);
        else
            return AIE_BAD_ARG;
        AIE_LAUNCH_CHECK();
    }
    const size_t smem = (size_t)(D + 32) * sizeof(float);
    if (smem > 200 * 1024) return AIE_UNSUPPORTED;
    const int threads = D >= 1024 ? 512 : 256;
    if (out_dtype == AIE_F32) {
        auto k = add_rmsnorm_kernel<A, W, float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<n, threads, smem, stream>>>(x, (const A*)delta, (const W*)w, (float*)out, rows, D, eps, write_back, parts, part_stride);
    } else if (out_dtype == AIE_BF16) {
        auto k = add_rmsnorm_kernel<A, W, bf16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<n, threads, smem, stream>>>(x, (const A*)delta, (const W*)w, (bf16*)out, rows, D, eps, write_back, parts, part_stride);
    } else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

extern "C" int aie_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* w,
                               int w_dtype, void* out, int out_dtype, const int* rows, int n, int D,
                               float eps, int write_back, int parts, long long part_stride,
                               cudaStream_t stream) {
    if (n <= 0) return 0;
    if (delta == nullptr) delta_dtype = AIE_F32;
    if (parts < 1) return AIE_BAD_ARG;
#define GO(A, W) return launch_rmsnorm_o<A, W>(x, delta, w, out, out_dtype, rows, n, D, eps, write_back, parts, (size_t)part_stride, stream)
    if (delta_dtype == AIE_F32 && w_dtype == AIE_F32) GO(float, float);
    if (delta_dtype == AIE_F32 && w_dtype == AIE_BF16) GO(float, bf16);
    if (delta_dtype == AIE_BF16 && w_dtype == AIE_F32) GO(bf16, float);
    if (delta_dtype == AIE_BF16 && w_dtype == AIE_BF16) GO(bf16, bf16);
#undef GO
    return AIE_BAD_ARG;
}

// ---------------------------------------------------------------------------
// a[t, f] = silu(gate) * up   (crates/ai-engine-runtime/src/arch/ffn.rs:50-54), silu(z) = z * sigmoid(z)
// in float32.  block == 0: gu[t] = [gate (F) | up (F)].  block > 0: gu[t] is in groups of
// 2 * block columns, `block` gate columns followed by their `block` up columns.
// ---------------------------------------------------------------------------
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ a, int F, int block, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t t = i / F, f = i % F;
        const size_t gc = block ? (f / block) * 2 * block + f % block : f;
        const size_t uc = block ? gc + block : F + f;
        const float g = to_f32<A>(gu[t * 2 * F + gc]);
        const float u = to_f32<A>(gu[t * 2 * F + uc]);
        const float s = g * (1.0f / (1.0f + expf(-g)));
        a[i] = from_f32<A>(s * u);
    }
}

// Eight outputs per thread with 16-byte accesses (bfloat16) when F and the group size are
// multiples of 8.
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ a, int F, int block,
                                     size_t total8) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const unsigned F8 = (unsigned)(F / 8);
    for (; i < total8; i += stride) {
        const size_t t = i / F8;
        const unsigned f = (unsigned)(i - t * F8) * 8u;
        const unsigned gc = block ? (f / (unsigned)block) * 2u * (unsigned)block + f % (unsigned)block : f;
        const unsigned uc = block ? gc + (unsigned)block : (unsigned)F + f;
        const uint4 gr = *reinterpret_cast<const uint4*>(gu + t * 2 * F + gc);
        const uint4 ur = *reinterpret_cast<const uint4*>(gu + t * 2 * F + uc);
        const bf16* ge = reinterpret_cast<const bf16*>(&gr);
        const bf16* ue = reinterpret_cast<const bf16*>(&ur);
        uint4 o;
        bf16* oe = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // sigmoid by ex2.approx and rcp.approx (relative error about 1e-6, far below the bf16 rounding of
            // the result): with expf and a division the kernel was bound by instruction issue, not by memory
            const float g = __bfloat162float(ge[j]), u = __bfloat162float(ue[j]);
            float e, r;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
            oe[j] = __float2bfloat16_rn((g * r) * u);
        }
        *reinterpret_cast<uint4*>(a + t * F + f) = o;
    }
}

extern "C" int aie_silu_mul(const void* gu, void* a, int dtype, int T, int F, int block, cudaStream_t stream) {
    if (block < 0 || (block && F % block)) return AIE_BAD_ARG;
    if (T <= 0) return 0;
    const size_t total = (size_t)T * F;
    int blocks = (int)((total + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    if (dtype == AIE_BF16 && F % 8 == 0 && block % 8 == 0 && !((size_t)gu & 15) && !((size_t)a & 15)) {
        const size_t total8 = total / 8;
        int b8 = (int)((total8 + 255) / 256);
        if (b8 > aie_sm_count() * 16) b8 = aie_sm_count() * 16;
        launch_pdl(silu_mul_vec8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)gu, (bf16*)a, F, block, total8);
        AIE_LAUNCH_CHECK();
    }
    if (dtype == AIE_F32)
        launch_pdl(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)a, F, block, total);
    else if (dtype == AIE_BF16)
        launch_pdl(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)a, F, block, total);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// casts between float32 and bfloat16 (a 32-bit weight under bf16 activations)
// ---------------------------------------------------------------------------
template <typename I, typename O>
__global__ void cast_kernel(const I* __restrict__ in, O* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = from_f32<O>(to_f32<I>(in[i]));
}

extern "C" int aie_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                        cudaStream_t stream) {
    if (n <= 0) return 0;
    int blocks = (int)((n + 255) / 256);
    if (blocks > aie_sm_count() * 16) blocks = aie_sm_count() * 16;
    if (in_dtype == AIE_F32 && out_dtype == AIE_BF16)
        cast_kernel<float, bf16><<<blocks, 256, 0, stream>>>((const float*)in, (bf16*)out, (size_t)n);
    else if (in_dtype == AIE_BF16 && out_dtype == AIE_F32)
        cast_kernel<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)in, (float*)out, (size_t)n);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
