// Device code of the bfloat16 split-KV decode attention and the reduce that joins
// the splits, with the host-side dispatch over head size and group size.  Included
// by attention_fast.cu (scratch given by the caller) and by
// attention_decode_noalloc.cu (scratch in a static device array).
#pragma once
#include "common.cuh"

#define DEC_WARPS 4
#define DEC_TILE 16          // keys a warp stages and consumes at a time
#define DEC_MAX_PAGES 2048   // block-table entries of one CTA's part of the keys
#define DEC_HEADS 8          // query heads of one kv head that a CTA takes (rows of the 16-row MMA)

__device__ __forceinline__ void dec_cp_async16(void* dst, const void* src, bool pred) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int n = pred ? 16 : 0;   // 0 source bytes: the destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void dec_ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void dec_ldsm_x4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void dec_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                        unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned dec_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// A stage of a warp's ring holds SUB tiles of 16 keys: two at head size 64, so that a stage is 8 KB at both head
// sizes (what a warp pays per stage — index arithmetic, the wait, the hand-over — does not depend on the
// stage's bytes: with 4 KB stages the head-size-64 kernel ran at 3.3 TB/s where head size 128 ran at 4.9).
template <int D> struct DecodeSub { static constexpr int value = D <= 64 ? 2 : 1; };

// Shared memory of the decode kernel for head size D with NST stages per warp.
template <int D, int NST> struct DecodeSmem {
    static constexpr size_t stage_bytes = (size_t)2 * DecodeSub<D>::value * DEC_TILE * D * sizeof(bf16);      // keys + values
    static constexpr size_t bytes = DEC_WARPS * NST * stage_bytes + DEC_MAX_PAGES * sizeof(int);
};

// row r, 16-byte chunk c of a [16][D] bf16 tile, XOR-swizzled so that ldmatrix reads without conflicts
template <int D> __device__ __forceinline__ bf16* dec_at(bf16* base, int row, int chunk) {
    return base + row * D + ((chunk ^ (row & 7)) << 3);
}

// The query heads are rows 0 .. ng-1 of a 16-row mma.sync tile (rows up to 15 are padding): per
// 16-key tile, q.k is 2 x D/16 multiplies and p.v is D/8, both bf16 in / float32 accumulate.
template <int D, int NST>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                    const bf16* __restrict__ v_pages, bf16* __restrict__ out,
                    float* __restrict__ part_o, float* __restrict__ part_lse,
                    const int* __restrict__ dec_tokens, const int* __restrict__ positions,
                    const int* __restrict__ token_req, const int* __restrict__ block_table,
                    int bt_width, int num_pages, int P, int H, int K, int G, int GC, int window,
                    float scale, int S, int* __restrict__ counters, unsigned* err) {
    constexpr int CH = D / 8;       // 16-byte chunks per row
    constexpr int KPL = 32 / CH;    // keys one round of 32 copies covers
    constexpr int KS = D / 16;      // k-steps of q.k
    constexpr int SUB = DecodeSub<D>::value;       // 16-key tiles per stage
    constexpr int STILE = SUB * DEC_TILE;          // keys per stage
    static_assert(D % 64 == 0, "head size of the fast path");
    extern __shared__ __align__(128) unsigned char dec_smem[];
    __shared__ float mrg_m[DEC_WARPS][DEC_HEADS], mrg_l[DEC_WARPS][DEC_HEADS];

    // Everything up to the first use of q reads only what earlier steps left (the step's index
    // arrays, the block table, keys and values of earlier tokens), so it runs before
    // griddepcontrol.wait, while the kernel that writes q and this token's key is still running.
    pdl_launch_dependents();
    bool waited = false;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = blockIdx.x, di = blockIdx.z;
    const int gchunks = (G + GC - 1) / GC;
    const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * GC;
    const int ng = min(GC, G - g0);
    const int t = dec_tokens[di];
    const int pos = positions[t], row = token_req[t];
    const int hbase = kvh * G + g0;
    const int qrow = lane >> 2, qcol = (lane & 3) * 2;      // this lane's row and column pair of an MMA tile

    bf16* stage0 = reinterpret_cast<bf16*>(dec_smem) + (size_t)warp * NST * 2 * STILE * D;
    int* bt_s = reinterpret_cast<int*>(dec_smem + DEC_WARPS * NST * DecodeSmem<D, NST>::stage_bytes);

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const int hi = pos + 1;
    const int tiles_total = (hi - lo + STILE - 1) / STILE;       // stages' worth of keys
    const int tps = (tiles_total + S - 1) / S;
    const int tile_begin = s * tps, tile_end = min((s + 1) * tps, tiles_total);

    // the block-table entries of this CTA's keys, once
    const int pg0 = (lo + tile_begin * STILE) / P;
    {
        const int last_key = min(hi, lo + tile_end * STILE) - 1;
        const int npg = tile_end > tile_begin ? last_key / P - pg0 + 1 : 0;
        const int* bt = block_table + (size_t)row * bt_width;
        for (int i = tid; i < npg && i < DEC_MAX_PAGES; i += DEC_WARPS * 32)
            bt_s[i] = (pg0 + i < bt_width) ? bt[pg0 + i] : -1;
    }
    __syncthreads();

    const int first = tile_begin + warp;
    const int n_my = first < tile_end ? (tile_end - first + DEC_WARPS - 1) / DEC_WARPS : 0;

    // stage the keys and values of this warp's i-th stage (zero-filled where there is no key)
    auto issue = [&](int i) {
        if (i < n_my) {
            const int st = i % NST;
            const int kbase0 = lo + (first + i * DEC_WARPS) * STILE;
            if (!waited && kbase0 + STILE > pos) {      // this stage holds the token written in this step
                pdl_wait();
                waited = true;
            }
            bf16* ks = stage0 + (size_t)st * 2 * STILE * D;
            bf16* vs = ks + STILE * D;
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub) {
                const int kbase = kbase0 + sub * DEC_TILE;
                int prow = -1;
                if (lane < DEC_TILE) {
                    const int key = kbase + lane;
                    if (key < hi) {
                        const int pidx = key / P;
                        const int page = (pidx - pg0 < DEC_MAX_PAGES) ? bt_s[pidx - pg0] : -1;
                        if (page >= 0 && page < num_pages) prow = (page * K + kvh) * P + (key - pidx * P);
                        else atomicOr(err, AIE_DEV_PAGE_OOB);
                    }
                }
                const int cc = lane % CH, kq = lane / CH;
#pragma unroll
                for (int r = 0; r < DEC_TILE / KPL; ++r) {
                    const int kidx = kq + r * KPL;
                    const int pr = __shfl_sync(0xffffffffu, prow, kidx);
                    const size_t off = (size_t)(pr >= 0 ? pr : 0) * D + cc * 8;
                    dec_cp_async16(dec_at<D>(ks + sub * DEC_TILE * D, kidx, cc), k_pages + off, pr >= 0);
                    dec_cp_async16(dec_at<D>(vs + sub * DEC_TILE * D, kidx, cc), v_pages + off, pr >= 0);
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

#pragma unroll
    for (int i = 0; i < NST - 1; ++i) issue(i);
    if (!waited) {
        pdl_wait();
        waited = true;
    }

    // q as the A operand: row = head, rows >= ng (and 8..15) are zero
    unsigned qa[KS][2];
    {
        const bf16* qp = q + ((size_t)t * H + hbase + (qrow < ng ? qrow : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const unsigned lo2 = *reinterpret_cast<const unsigned*>(qp + ks * 16 + qcol);
            const unsigned hi2 = *reinterpret_cast<const unsigned*>(qp + ks * 16 + 8 + qcol);
            qa[ks][0] = qrow < ng ? lo2 : 0u;
            qa[ks][1] = qrow < ng ? hi2 : 0u;
        }
    }
    float m_run = -INFINITY, l_run = 0.f;      // of row qrow (valid when qrow < ng)
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;

    for (int i = 0; i < n_my; ++i) {
        issue(i + NST - 1);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(NST - 1));
        __syncwarp();
        const int st = i % NST;
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
        const int kb_tile = lo + (first + i * DEC_WARPS) * STILE + sub * DEC_TILE;      // first key of this 16-key tile
        bf16* ks_t = stage0 + (size_t)st * 2 * STILE * D + sub * DEC_TILE * D;
        bf16* vs_t = stage0 + (size_t)st * 2 * STILE * D + STILE * D + sub * DEC_TILE * D;

        // scores of the 16 keys: two 8-key column tiles
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
        const int mid = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            unsigned b0, b1, b2, b3;
            dec_ldsm_x4(b0, b1, b2, b3, dec_at<D>(ks_t, (mid >> 1) * 8 + (lane & 7), ks * 2 + (mid & 1)));
            dec_mma(sc[0], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
            dec_mma(sc[1], qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
        }
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                // a key is there when it lies before the end of the sequence (a page that is missing was flagged
                // when its copy was left out; its keys read as zeros)
                const bool valid = kb_tile + j * 8 + qcol + e < hi;
                sc[j][e] = valid ? sc[j][e] * scale : -INFINITY;
                tmax = fmaxf(tmax, sc[j][e]);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_use);
        float p[2][2], psum = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[j][e] = __expf(sc[j][e] - m_use);       // exp(-inf) = 0 for a key that is not there
                psum += p[j][e];
            }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l_run = l_run * corr + psum;
        m_run = m_new;
        const unsigned pa0 = dec_pack(p[0][0], p[0][1]), pa2 = dec_pack(p[1][0], p[1][1]);
#pragma unroll
        for (int jd = 0; jd < D / 8; jd += 2) {
            o[jd][0] *= corr;
            o[jd][1] *= corr;
            o[jd + 1][0] *= corr;
            o[jd + 1][1] *= corr;
            unsigned b0, b1, b2, b3;
            dec_ldsm_x4_t(b0, b1, b2, b3, dec_at<D>(vs_t, (mid & 1) * 8 + (lane & 7), jd + (mid >> 1)));
            dec_mma(o[jd], pa0, 0u, pa2, 0u, b0, b1);
            dec_mma(o[jd + 1], pa0, 0u, pa2, 0u, b2, b3);
        }
        }
        __syncwarp();      // the stage is free again
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();

    // merge the warps of the CTA (the staging memory is free now: reuse it for the partial outputs)
    float* mrg_o = reinterpret_cast<float*>(dec_smem);      // [DEC_WARPS][DEC_HEADS][D]
    if (qrow < DEC_HEADS) {
        if ((lane & 3) == 0) { mrg_m[warp][qrow] = m_run; mrg_l[warp][qrow] = l_run; }
#pragma unroll
        for (int jd = 0; jd < D / 8; ++jd) {
            mrg_o[((size_t)warp * DEC_HEADS + qrow) * D + jd * 8 + qcol] = o[jd][0];
            mrg_o[((size_t)warp * DEC_HEADS + qrow) * D + jd * 8 + qcol + 1] = o[jd][1];
        }
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
            A += mrg_o[((size_t)w * DEC_HEADS + g) * D + e] * f;
        }
        const float ov = L > 0.f ? A / L : 0.f;
        const int h = hbase + g;
        if (S == 1) {
            out[((size_t)t * H + h) * D + e] = __float2bfloat16_rn(ov);
        } else {
            const size_t pi = ((size_t)di * H + h) * S + s;
            part_o[pi * D + e] = ov;
            if (e == 0) part_lse[pi] = L > 0.f ? M + __logf(L) : -INFINITY;
        }
    }
    if (S > 1 && counters != nullptr) {
        // the CTA that finishes last among the S parts of this (request, kv head, head chunk)
        // joins them: out = sum_s w_s * part_o[s] / sum_s w_s with w_s = exp(lse_s - max lse)
        __shared__ int last_s;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int* c = counters + (size_t)di * gridDim.y + blockIdx.y;
            const int ticket = atomicAdd(c, 1);
            last_s = ticket == S - 1;
            if (last_s) *c = 0;                       // ready for the next launch
        }
        __syncthreads();
        if (last_s) {
            __threadfence();
            for (int idx = tid; idx < ng * D; idx += DEC_WARPS * 32) {
                const int g = idx / D, e = idx % D;
                const int h = hbase + g;
                const size_t base = ((size_t)di * H + h) * S;
                float M = -INFINITY;
                for (int sp = 0; sp < S; ++sp) M = fmaxf(M, __ldcg(part_lse + base + sp));
                float A = 0.f, W = 0.f;
                for (int sp = 0; sp < S; ++sp) {
                    const float lse = __ldcg(part_lse + base + sp);
                    const float w = (lse == -INFINITY) ? 0.f : __expf(lse - M);
                    W += w;
                    A += w * __ldcg(part_o + (base + sp) * D + e);
                }
                out[((size_t)t * H + h) * D + e] = __float2bfloat16_rn(W > 0.f ? A / W : 0.f);
            }
        }
    }
}

// out[t, h, :] = sum_s w_s * part_o[s] / sum_s w_s with w_s = exp(lse_s - max lse).  One block per
// (request, head).  The weights are worked out once (the first warp, lanes over the parts) and kept in
// shared memory; then every thread sums its element over the parts with eight loads in flight (a loop
// of one dependent load after another took 12 us at 37 parts, more than the bytes of the keys it joins).
#define DEC_MAX_SPLITS 64
__global__ void decode_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                     bf16* __restrict__ out, const int* __restrict__ dec_tokens,
                                     int H, int D, int S) {
    __shared__ float w_s[DEC_MAX_SPLITS];
    __shared__ float wsum_s;
    pdl_launch_dependents();
    const int di = blockIdx.x, h = blockIdx.y;
    const int t = dec_tokens[di];
    const size_t base = ((size_t)di * H + h) * S;
    pdl_wait();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float l0 = lane < S ? part_lse[base + lane] : -INFINITY;
        const float l1 = lane + 32 < S ? part_lse[base + lane + 32] : -INFINITY;
        float M = fmaxf(l0, l1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float w0 = (l0 == -INFINITY) ? 0.f : __expf(l0 - M);
        const float w1 = (l1 == -INFINITY) ? 0.f : __expf(l1 - M);
        if (lane < S) w_s[lane] = w0;
        if (lane + 32 < S) w_s[lane + 32] = w1;
        float W = w0 + w1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) W += __shfl_xor_sync(0xffffffffu, W, o);
        if (lane == 0) wsum_s = W;
    }
    __syncthreads();
    const float W = wsum_s;
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        const float* src = part_o + base * D + e;
        float A = 0.f;
        int s = 0;
        for (; s + 8 <= S; s += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = src[(size_t)(s + u) * D];
#pragma unroll
            for (int u = 0; u < 8; ++u) A += w_s[s + u] * v[u];
        }
        for (; s < S; ++s) A += w_s[s] * src[(size_t)s * D];
        out[((size_t)t * H + h) * D + e] = __float2bfloat16_rn(W > 0.f ? A / W : 0.f);
    }
}

template <int D>
static int launch_decode(int GC, dim3 grid, cudaStream_t st, const bf16* q, const bf16* kp, const bf16* vp,
                         bf16* out, float* po, float* pl, const int* dt, const int* pos, const int* tr,
                         const int* bt, int btw, int np, int P, int H, int K, int G, int window, float scale,
                         int S, int* counters, unsigned* err) {
    if (GC < 1 || GC > DEC_HEADS) return AIE_UNSUPPORTED;
    // stages of 8 KB (two 16-key tiles at head size 64, one at 128), rings of 3, two CTAs to an SM (at head size 64,
    // rings of 2 with three CTAs to an SM were measured 2 % slower in a whole step)
    constexpr int NST = 3;
    constexpr size_t smem = DecodeSmem<D, NST>::bytes;
    auto kern = paged_decode_kernel<D, NST>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(kern, grid, dim3(DEC_WARPS * 32), smem, st, q, kp, vp, out, po, pl, dt, pos, tr, bt, btw, np,
                           P, H, K, G, GC, window, scale, S, counters, err);
}
