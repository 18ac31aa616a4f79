// Device code of the bfloat16 split-KV decode attention and the reduce that joins
// the splits, with the host-side dispatch over head size and group size.  Included
// by attention_fast.cu (scratch given by the caller) and by
// attention_decode_noalloc.cu (scratch in a static device array).
#pragma once
#include "common.cuh"

#define DEC_WARPS 4
#define DEC_TILE 16          // keys a warp stages and consumes at a time
#define DEC_MAX_PAGES 2048   // block-table entries of one CTA's part of the keys

__device__ __forceinline__ void dec_cp_async16(void* dst, const void* src, bool pred) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int n = pred ? 16 : 0;   // 0 source bytes: the destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}

// Shared memory of the decode kernel for head size D with NST stages per warp.
template <int D, int NST> struct DecodeSmem {
    static constexpr size_t stage_bytes = (size_t)2 * DEC_TILE * D * sizeof(bf16);      // keys + values
    static constexpr size_t bytes = DEC_WARPS * NST * stage_bytes + DEC_MAX_PAGES * sizeof(int);
};

template <int D, int GC, int NST>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                    const bf16* __restrict__ v_pages, bf16* __restrict__ out,
                    float* __restrict__ part_o, float* __restrict__ part_lse,
                    const int* __restrict__ dec_tokens, const int* __restrict__ positions,
                    const int* __restrict__ token_req, const int* __restrict__ block_table,
                    int bt_width, int num_pages, int P, int H, int K, int G, int window,
                    float scale, int S, unsigned* err) {
    constexpr int EPL = D / 8;      // elements of a key each of its 8 lanes holds
    constexpr int NCH = EPL / 8;    // 16-byte chunks per lane
    constexpr int VPL = D / 32;     // output elements per lane
    constexpr int CH = D / 8;       // 16-byte chunks per row
    constexpr int KPL = 32 / CH;    // keys one round of 32 copies covers
    static_assert(D % 64 == 0, "head size of the fast path");
    extern __shared__ __align__(128) unsigned char dec_smem[];
    __shared__ float p_s[DEC_WARPS][DEC_TILE][GC];
    __shared__ int ok_s[DEC_WARPS][NST][DEC_TILE];
    __shared__ float mrg_m[DEC_WARPS][GC], mrg_l[DEC_WARPS][GC];

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.x, di = blockIdx.z;
    const int gchunks = (G + GC - 1) / GC;
    const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * GC;
    const int ng = min(GC, G - g0);
    const int t = dec_tokens[di];
    const int pos = positions[t], row = token_req[t];
    const int hbase = kvh * G + g0;
    const int sub = lane & 7, kg = lane >> 3;

    bf16* stage0 = reinterpret_cast<bf16*>(dec_smem) + (size_t)warp * NST * 2 * DEC_TILE * D;
    int* bt_s = reinterpret_cast<int*>(dec_smem + DEC_WARPS * NST * DecodeSmem<D, NST>::stage_bytes);

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const int hi = pos + 1;
    const int tiles_total = (hi - lo + DEC_TILE - 1) / DEC_TILE;
    const int tps = (tiles_total + S - 1) / S;
    const int tile_begin = s * tps, tile_end = min((s + 1) * tps, tiles_total);

    // the block-table entries of this CTA's keys, once
    const int pg0 = (lo + tile_begin * DEC_TILE) / P;
    {
        const int last_key = min(hi, lo + tile_end * DEC_TILE) - 1;
        const int npg = tile_end > tile_begin ? last_key / P - pg0 + 1 : 0;
        const int* bt = block_table + (size_t)row * bt_width;
        for (int i = tid; i < npg && i < DEC_MAX_PAGES; i += DEC_WARPS * 32)
            bt_s[i] = (pg0 + i < bt_width) ? bt[pg0 + i] : -1;
    }

    // this lane's slice of every query head, float32
    float qr[GC][EPL];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        const bf16* qp = q + ((size_t)t * H + hbase + (g < ng ? g : 0)) * D;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const uint4 raw = *reinterpret_cast<const uint4*>(qp + (sub + 8 * j) * 8);
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) qr[g][j * 8 + i] = g < ng ? __bfloat162float(e[i]) : 0.f;
        }
    }
    __syncthreads();

    float m[GC], l[GC], acc[GC][VPL];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < VPL; ++e) acc[g][e] = 0.f;
    }

    const int first = tile_begin + warp;
    const int n_my = first < tile_end ? (tile_end - first + DEC_WARPS - 1) / DEC_WARPS : 0;

    // stage the keys and values of this warp's i-th tile (zero-filled where there is no key)
    auto issue = [&](int i) {
        if (i < n_my) {
            const int st = i % NST;
            const int kbase = lo + (first + i * DEC_WARPS) * DEC_TILE;
            int prow = -1;
            if (lane < DEC_TILE) {
                const int key = kbase + lane;
                if (key < hi) {
                    const int pidx = key / P;
                    const int page = (pidx - pg0 < DEC_MAX_PAGES) ? bt_s[pidx - pg0] : -1;
                    if (page >= 0 && page < num_pages) prow = (page * K + kvh) * P + (key - pidx * P);
                    else atomicOr(err, AIE_DEV_PAGE_OOB);
                }
                ok_s[warp][st][lane] = prow >= 0;
            }
            bf16* ks = stage0 + (size_t)st * 2 * DEC_TILE * D;
            bf16* vs = ks + DEC_TILE * D;
            const int cc = lane % CH, kq = lane / CH;
#pragma unroll
            for (int r = 0; r < DEC_TILE / KPL; ++r) {
                const int kidx = kq + r * KPL;
                const int pr = __shfl_sync(0xffffffffu, prow, kidx);
                const size_t off = (size_t)(pr >= 0 ? pr : 0) * D + cc * 8;
                dec_cp_async16(ks + kidx * D + cc * 8, k_pages + off, pr >= 0);
                dec_cp_async16(vs + kidx * D + cc * 8, v_pages + off, pr >= 0);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

#pragma unroll
    for (int i = 0; i < NST - 1; ++i) issue(i);

    for (int i = 0; i < n_my; ++i) {
        issue(i + NST - 1);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(NST - 1));
        __syncwarp();
        const int st = i % NST;
        const bf16* ks = stage0 + (size_t)st * 2 * DEC_TILE * D;
        const bf16* vs = ks + DEC_TILE * D;

        float sc[DEC_TILE / 4][GC];
        float tmax[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) tmax[g] = -INFINITY;
#pragma unroll
        for (int it = 0; it < DEC_TILE / 4; ++it) {
            const int kidx = it * 4 + kg;
            const bool valid = ok_s[warp][st][kidx] != 0;
            float dot[GC];
#pragma unroll
            for (int g = 0; g < GC; ++g) dot[g] = 0.f;
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                const uint4 raw = *reinterpret_cast<const uint4*>(ks + kidx * D + (sub + 8 * j) * 8);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    const float kv = __bfloat162float(e[x]);
#pragma unroll
                    for (int g = 0; g < GC; ++g) dot[g] = fmaf(qr[g][j * 8 + x], kv, dot[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                float d = dot[g];
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                sc[it][g] = valid ? d * scale : -INFINITY;
                tmax[g] = fmaxf(tmax[g], sc[it][g]);
            }
        }
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            float tm = tmax[g];
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
            const float m_new = fmaxf(m[g], tm);
            const float corr = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int it = 0; it < DEC_TILE / 4; ++it) {
                const float p = (sc[it][g] == -INFINITY) ? 0.f : __expf(sc[it][g] - m_new);
                psum += p;
                if (sub == 0) p_s[warp][it * 4 + kg][g] = p;
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 8);
            psum += __shfl_xor_sync(0xffffffffu, psum, 16);
            l[g] = l[g] * corr + psum;
            m[g] = m_new;
#pragma unroll
            for (int e = 0; e < VPL; ++e) acc[g][e] *= corr;
        }
        __syncwarp();
#pragma unroll
        for (int kk = 0; kk < DEC_TILE; ++kk) {
            float v[VPL];
            if (VPL == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(vs + kk * D + lane * VPL);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int x = 0; x < VPL; ++x) v[x] = __bfloat162float(e[x]);
            } else {
                const unsigned raw = *reinterpret_cast<const unsigned*>(vs + kk * D + lane * VPL);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int x = 0; x < VPL; ++x) v[x] = __bfloat162float(e[x]);
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                const float p = p_s[warp][kk][g];     // 0 for a key that is not there (its row is zero too)
#pragma unroll
                for (int e = 0; e < VPL; ++e) acc[g][e] = fmaf(p, v[e], acc[g][e]);
            }
        }
        __syncwarp();      // the stage and p_s are free again
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();

    // merge the warps of the CTA (the staging memory is free now: reuse it for the partial outputs)
    float* mrg_o = reinterpret_cast<float*>(dec_smem);      // [DEC_WARPS][GC][D]
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        if (lane == 0) { mrg_m[warp][g] = m[g]; mrg_l[warp][g] = l[g]; }
#pragma unroll
        for (int e = 0; e < VPL; ++e) mrg_o[((size_t)warp * GC + g) * D + lane * VPL + e] = acc[g][e];
    }
    __syncthreads();
    for (int idx = tid; idx < ng * D; idx += DEC_WARPS * 32) {
        const int g = idx / D, e = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mrg_m[w][g]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = (mrg_m[w][g] == -INFINITY) ? 0.f : __expf(mrg_m[w][g] - M);
            L += mrg_l[w][g] * f;
            A += mrg_o[((size_t)w * GC + g) * D + e] * f;
        }
        const float o = L > 0.f ? A / L : 0.f;
        const int h = hbase + g;
        if (S == 1) {
            out[((size_t)t * H + h) * D + e] = __float2bfloat16_rn(o);
        } else {
            const size_t pi = ((size_t)di * H + h) * S + s;
            part_o[pi * D + e] = o;
            if (e == 0) part_lse[pi] = L > 0.f ? M + __logf(L) : -INFINITY;
        }
    }
}

// out[t, h, :] = sum_s w_s * part_o[s] / sum_s w_s with w_s = exp(lse_s - max lse)
__global__ void decode_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                     bf16* __restrict__ out, const int* __restrict__ dec_tokens,
                                     int H, int D, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int di = blockIdx.x, h = blockIdx.y;
    const int t = dec_tokens[di];
    const size_t base = ((size_t)di * H + h) * S;
    float M = -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, part_lse[base + s]);
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float A = 0.f, W = 0.f;
        for (int s = 0; s < S; ++s) {
            const float lse = part_lse[base + s];
            const float w = (lse == -INFINITY) ? 0.f : __expf(lse - M);
            W += w;
            A += w * part_o[(base + s) * D + e];
        }
        out[((size_t)t * H + h) * D + e] = __float2bfloat16_rn(W > 0.f ? A / W : 0.f);
    }
}

template <int D>
static int launch_decode(int GC, dim3 grid, cudaStream_t st, const bf16* q, const bf16* kp, const bf16* vp,
                         bf16* out, float* po, float* pl, const int* dt, const int* pos, const int* tr,
                         const int* bt, int btw, int np, int P, int H, int K, int G, int window, float scale,
                         int S, unsigned* err) {
    constexpr int NST = D >= 128 ? 3 : 4;
    constexpr size_t smem = DecodeSmem<D, NST>::bytes;
#define GO(GCV)                                                                                                   \
    do {                                                                                                          \
        auto kern = paged_decode_kernel<D, GCV, NST>;                                                             \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
        launch_pdl(kern, grid, dim3(DEC_WARPS * 32), smem, st, q, kp, vp, out, po, pl, dt, pos, tr, bt, btw, np, \
                   P, H, K, G, window, scale, S, err);                                                            \
    } while (0)
    switch (GC) {
        case 1: GO(1); break;
        case 2: GO(2); break;
        case 3: GO(3); break;
        case 4: GO(4); break;
        default: return AIE_UNSUPPORTED;
    }
#undef GO
    return 0;
}
