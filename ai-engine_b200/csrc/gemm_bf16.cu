// bfloat16 matrix products for steps with few tokens (decode): C[M, N] = X[M, K] . W[N, K]^T
// with M <= 16.  Such a product only streams the weights once, so the kernel is
// built around the memory system, not the tensor cores: the weight matrix is the
// 16-row operand of mma.sync.m16n8k16 ("swap A and B": D^T = W . X^T), every lane
// fetches its slice of two weight rows straight from global memory with 16-byte
// loads, several steps ahead of the multiply, and the tokens are the 8 columns.
// The hardware's k order inside one multiply does not matter to a dot product, so
// each lane feeds 8 consecutive k of a row to two multiplies and the tokens'
// fragments are permuted the same way; no shared-memory staging is needed.
// A CTA has 8 warps = RG groups of 16 weight rows x (8 / RG) parts of K; the parts
// are summed through shared memory in a fixed order, so a token's result does not
// depend on the other tokens of the batch.  Accumulation is float32.
// Epilogues: plain store (bf16 or float32), or SwiGLU for the fused gate/up matrix
// [2F, K] (rows [0, F) gate, [F, 2F) up): a[t, f] = silu(g) * u in float32
// (crates/ai-engine-runtime/src/arch/ffn.rs:50-54).
#include "common.cuh"

#define SM_WARPS 8
#define SM_UNROLL 4

__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const bf16* p) {
    uint4 v;   // weights are read once: do not keep them in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <typename OT> __device__ __forceinline__ void store_out(OT* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// MT: 8-token tiles (1 or 2).  RG: row groups per CTA (1, 2, 4, 8).  SWIGLU: fused gate/up epilogue.
template <int MT, int RG, bool SWIGLU, typename OT>
__global__ void __launch_bounds__(SM_WARPS * 32)
gemm_small_m_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, OT* __restrict__ C,
                    int M, int N, int K, int ldc, int F) {
    constexpr int KSPLIT = SM_WARPS / RG;
    __shared__ float red[KSPLIT][RG][16][MT * 8 + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int rg = warp % RG, ks = warp / RG;
    // weight rows of this warp
    int wrow;
    if (SWIGLU) wrow = ((rg & 1) ? F : 0) + blockIdx.x * (8 * RG) + (rg >> 1) * 16;
    else wrow = blockIdx.x * (16 * RG) + rg * 16;
    const int row_limit = SWIGLU ? ((rg & 1) ? 2 * F : F) : N;
    const bool rows_ok = wrow < row_limit;      // N and F are multiples of 16: a group is whole or absent
    const int Kw = K / KSPLIT, kbeg = ks * Kw;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

    if (rows_ok) {
        const bf16* w0 = W + (size_t)(wrow + g) * K + kbeg + c * 8;
        const bf16* w1 = w0 + (size_t)8 * K;
        const bf16* xp[MT];
        bool xok[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int tok = mt * 8 + g;
            xok[mt] = tok < M;
            xp[mt] = X + (size_t)(xok[mt] ? tok : 0) * K + kbeg + c * 8;
        }
        const int steps = Kw / 32;
        int s = 0;
        for (; s + SM_UNROLL <= steps; s += SM_UNROLL) {
            uint4 a_lo[SM_UNROLL], a_hi[SM_UNROLL], b[SM_UNROLL][MT];
#pragma unroll
            for (int u = 0; u < SM_UNROLL; ++u) {
                a_lo[u] = ldg_stream(w0 + (s + u) * 32);
                a_hi[u] = ldg_stream(w1 + (s + u) * 32);
            }
#pragma unroll
            for (int u = 0; u < SM_UNROLL; ++u)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    b[u][mt] = xok[mt] ? *reinterpret_cast<const uint4*>(xp[mt] + (s + u) * 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < SM_UNROLL; ++u)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16(acc[mt], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b[u][mt].x, b[u][mt].y);
                    mma_bf16(acc[mt], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b[u][mt].z, b[u][mt].w);
                }
        }
        for (; s < steps; ++s) {
            const uint4 a_lo = ldg_stream(w0 + s * 32), a_hi = ldg_stream(w1 + s * 32);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint4 b = xok[mt] ? *reinterpret_cast<const uint4*>(xp[mt] + s * 32) : make_uint4(0, 0, 0, 0);
                mma_bf16(acc[mt], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
                mma_bf16(acc[mt], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
            }
        }
    }
    // partial sums of this warp: rows g and g + 8, tokens 2c and 2c + 1 of each tile
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        red[ks][rg][g][mt * 8 + 2 * c] = acc[mt][0];
        red[ks][rg][g][mt * 8 + 2 * c + 1] = acc[mt][1];
        red[ks][rg][g + 8][mt * 8 + 2 * c] = acc[mt][2];
        red[ks][rg][g + 8][mt * 8 + 2 * c + 1] = acc[mt][3];
    }
    __syncthreads();
    if (!SWIGLU) {
        // outputs of the CTA: 16 * RG rows x M tokens; adjacent threads take adjacent rows
        for (int idx = tid; idx < 16 * RG * MT * 8; idx += SM_WARPS * 32) {
            const int r = idx % (16 * RG), tok = idx / (16 * RG);
            const int n = blockIdx.x * (16 * RG) + r;
            if (tok >= M || n >= N) continue;
            float v = 0.f;
#pragma unroll
            for (int k = 0; k < KSPLIT; ++k) v += red[k][r / 16][r % 16][tok];
            store_out<OT>(C + (size_t)tok * ldc + n, v);
        }
    } else {
        for (int idx = tid; idx < 8 * RG * MT * 8; idx += SM_WARPS * 32) {
            const int r = idx % (8 * RG), tok = idx / (8 * RG);
            const int f = blockIdx.x * (8 * RG) + r;
            if (tok >= M || f >= F) continue;
            float gv = 0.f, uv = 0.f;
#pragma unroll
            for (int k = 0; k < KSPLIT; ++k) {
                gv += red[k][(r / 16) * 2][r % 16][tok];
                uv += red[k][(r / 16) * 2 + 1][r % 16][tok];
            }
            const float sv = gv * (1.0f / (1.0f + expf(-gv)));
            store_out<OT>(C + (size_t)tok * ldc + f, sv * uv);
        }
    }
}

template <int MT, int RG, bool SWIGLU, typename OT>
static void launch_one(const bf16* X, const bf16* W, void* C, int M, int N, int K, int ldc, int F, cudaStream_t st) {
    const int rows_per_cta = SWIGLU ? 8 * RG : 16 * RG;
    const int rows = SWIGLU ? F : N;
    const int ctas = (rows + rows_per_cta - 1) / rows_per_cta;
    gemm_small_m_kernel<MT, RG, SWIGLU, OT><<<ctas, SM_WARPS * 32, 0, st>>>(X, W, (OT*)C, M, N, K, ldc, F);
}

template <int MT, bool SWIGLU, typename OT>
static int launch_rg(int RG, const bf16* X, const bf16* W, void* C, int M, int N, int K, int ldc, int F, cudaStream_t st) {
    switch (RG) {
        case 1: if (SWIGLU) return AIE_BAD_ARG; launch_one<MT, 1, false, OT>(X, W, C, M, N, K, ldc, F, st); break;
        case 2: launch_one<MT, 2, SWIGLU, OT>(X, W, C, M, N, K, ldc, F, st); break;
        case 4: launch_one<MT, 4, SWIGLU, OT>(X, W, C, M, N, K, ldc, F, st); break;
        case 8: launch_one<MT, 8, SWIGLU, OT>(X, W, C, M, N, K, ldc, F, st); break;
        default: return AIE_BAD_ARG;
    }
    return 0;
}

// swiglu != 0: W is the fused [2F, K] gate/up matrix (N = 2F) and C is [M, F].
// Refuses (AIE_UNSUPPORTED) what it does not take: M > 16, N or F not a multiple of 16,
// K not a multiple of 32 * (8 / row_groups); the caller then uses the library product.
extern "C" int aie_gemm_small_m(const void* X, const void* W, void* C, int out_dtype, int M, int N, int K,
                                int ldc, int swiglu, int row_groups, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0) return AIE_UNSUPPORTED;
    const int RG = row_groups;
    if (RG != 1 && RG != 2 && RG != 4 && RG != 8) return AIE_BAD_ARG;
    if (N % 16 || K % (32 * (SM_WARPS / RG))) return AIE_UNSUPPORTED;
    const int F = N / 2;
    if (swiglu && (N % 32 || RG < 2)) return AIE_UNSUPPORTED;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    int rc;
#define GO(MTV)                                                                                              \
    if (swiglu) {                                                                                            \
        rc = out_dtype == AIE_BF16 ? launch_rg<MTV, true, bf16>(RG, x, w, C, M, N, K, ldc, F, stream)        \
                                   : launch_rg<MTV, true, float>(RG, x, w, C, M, N, K, ldc, F, stream);      \
    } else {                                                                                                 \
        rc = out_dtype == AIE_BF16 ? launch_rg<MTV, false, bf16>(RG, x, w, C, M, N, K, ldc, F, stream)       \
                                   : launch_rg<MTV, false, float>(RG, x, w, C, M, N, K, ldc, F, stream);     \
    }
    if (out_dtype != AIE_BF16 && out_dtype != AIE_F32) return AIE_BAD_ARG;
    if (M <= 8) { GO(1) } else { GO(2) }
#undef GO
    if (rc) return rc;
    AIE_LAUNCH_CHECK();
}
