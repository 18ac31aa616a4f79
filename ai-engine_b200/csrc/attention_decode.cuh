// Device code of the bfloat16 split-KV decode attention and the reduce that joins
// the splits, with the host-side dispatch over head size and group size.  Included
// by attention_fast.cu (scratch given by the caller) and by
// attention_decode_noalloc.cu (scratch in a static device array).
#pragma once
#include "common.cuh"

#define DEC_WARPS 4
#define DEC_TILE 32

template <int D, int GC>
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
    static_assert(D % 64 == 0, "head size of the fast path");
    __shared__ float p_s[DEC_WARPS][DEC_TILE][GC];
    __shared__ int row_s[DEC_WARPS][DEC_TILE];
    __shared__ float mrg_o[DEC_WARPS][GC][D];
    __shared__ float mrg_m[DEC_WARPS][GC], mrg_l[DEC_WARPS][GC];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.x, di = blockIdx.z;
    const int gchunks = (G + GC - 1) / GC;
    const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * GC;
    const int ng = min(GC, G - g0);
    const int t = dec_tokens[di];
    const int pos = positions[t], row = token_req[t];
    const int hbase = kvh * G + g0;
    const int sub = lane & 7, kg = lane >> 3;

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

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const int hi = pos + 1;
    const int tiles_total = (hi - lo + DEC_TILE - 1) / DEC_TILE;
    const int tps = (tiles_total + S - 1) / S;
    const int tile_end = min((s + 1) * tps, tiles_total);

    float m[GC], l[GC], acc[GC][VPL];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < VPL; ++e) acc[g][e] = 0.f;
    }
    const int* bt = block_table + (size_t)row * bt_width;

    for (int tile = s * tps + warp; tile < tile_end; tile += DEC_WARPS) {
        const int kbase = lo + tile * DEC_TILE;
        float sc[DEC_TILE / 4][GC];
        float tmax[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) tmax[g] = -INFINITY;
#pragma unroll
        for (int it = 0; it < DEC_TILE / 4; ++it) {
            const int key = kbase + it * 4 + kg;
            const bool valid = key < hi;
            int prow = -1;
            if (valid) {
                const int pidx = key / P;
                const int page = pidx < bt_width ? bt[pidx] : -1;
                if (page >= 0 && page < num_pages) prow = (page * K + kvh) * P + (key - pidx * P);
                else if (sub == 0) atomicOr(err, AIE_DEV_PAGE_OOB);
            }
            float dot[GC];
#pragma unroll
            for (int g = 0; g < GC; ++g) dot[g] = 0.f;
            if (prow >= 0) {
                const bf16* kp = k_pages + (size_t)prow * D;
#pragma unroll
                for (int j = 0; j < NCH; ++j) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(kp + (sub + 8 * j) * 8);
                    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float kv = __bfloat162float(e[i]);
#pragma unroll
                        for (int g = 0; g < GC; ++g) dot[g] = fmaf(qr[g][j * 8 + i], kv, dot[g]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                float d = dot[g];
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                sc[it][g] = prow >= 0 ? d * scale : -INFINITY;
                tmax[g] = fmaxf(tmax[g], sc[it][g]);
            }
            if (sub == 0) row_s[warp][it * 4 + kg] = prow;
        }
        float corr[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            float tm = tmax[g];
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
            const float m_new = fmaxf(m[g], tm);
            corr[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int it = 0; it < DEC_TILE / 4; ++it) {
                const float p = (sc[it][g] == -INFINITY || m_new == -INFINITY) ? 0.f : __expf(sc[it][g] - m_new);
                psum += p;
                if (sub == 0) p_s[warp][it * 4 + kg][g] = p;
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 8);
            psum += __shfl_xor_sync(0xffffffffu, psum, 16);
            l[g] = l[g] * corr[g] + psum;
            m[g] = m_new;
#pragma unroll
            for (int e = 0; e < VPL; ++e) acc[g][e] *= corr[g];
        }
        __syncwarp();
        const int nk = min(DEC_TILE, hi - kbase);
#pragma unroll 8
        for (int kk = 0; kk < nk; ++kk) {
            const int prow = row_s[warp][kk];
            if (prow < 0) continue;
            const bf16* vp = v_pages + (size_t)prow * D + lane * VPL;
            float v[VPL];
            if (VPL == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(vp);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int i = 0; i < VPL; ++i) v[i] = __bfloat162float(e[i]);
            } else {
                const unsigned raw = *reinterpret_cast<const unsigned*>(vp);
                const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int i = 0; i < VPL; ++i) v[i] = __bfloat162float(e[i]);
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                const float p = p_s[warp][kk][g];
#pragma unroll
                for (int e = 0; e < VPL; ++e) acc[g][e] = fmaf(p, v[e], acc[g][e]);
            }
        }
        __syncwarp();
    }

    // merge the warps of the CTA
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        if (lane == 0) { mrg_m[warp][g] = m[g]; mrg_l[warp][g] = l[g]; }
#pragma unroll
        for (int e = 0; e < VPL; ++e) mrg_o[warp][g][lane * VPL + e] = acc[g][e];
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
            A += mrg_o[w][g][e] * f;
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
#define GO(GCV) paged_decode_kernel<D, GCV><<<grid, DEC_WARPS * 32, 0, st>>>(q, kp, vp, out, po, pl, dt, pos, tr, bt, btw, np, P, H, K, G, window, scale, S, err)
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
