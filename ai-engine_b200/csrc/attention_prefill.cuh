// bfloat16 paged attention for portions of prompts: tiles of 128 query tokens of one
// head against 64-key tiles of the request's cache, tensor-core products
// (mma.sync m16n8k16, bf16 in, float32 accumulate), online softmax in float32.
//
// One CTA of eight warps owns one (request, 128-token tile, query head); each warp
// owns 16 query rows.  Keys and values are gathered page by page through the block
// table into shared memory with 16-byte cp.async copies (two buffers: the next tile
// loads while this one is multiplied), in an XOR-swizzled layout that ldmatrix
// reads without bank conflicts.  Keys past the request's last token, and rows of a
// page that were never written, are zero-filled by the copy, so a masked
// probability of 0 never meets a NaN.  Tiles wholly above the diagonal (or below a
// window) are skipped; masks are applied only on tiles that straddle an edge.
// Formula: crates/ai-engine-runtime/src/arch/attention.rs:148-157,177-196,203-224.
#pragma once
#include "common.cuh"

#define PF_M 128
#define PF_N 64
#define PF_WARPS 8

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    const unsigned d = smem_u32(dst);
    const int n = pred ? 16 : 0;   // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// element (row, 16-byte chunk) of a [rows][D] bf16 tile -> swizzled address
template <int D> __device__ __forceinline__ bf16* tile_at(bf16* base, int row, int chunk) {
    return base + row * D + ((chunk ^ (row & 7)) << 3);
}

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32)
paged_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                     const bf16* __restrict__ v_pages, bf16* __restrict__ out,
                     const int* __restrict__ tiles,      // [n_tiles][2]: request row, offset of the tile in its tokens
                     const int* __restrict__ q_start, const int* __restrict__ q_len,
                     const int* __restrict__ ctx_len, const int* __restrict__ block_table,
                     int bt_width, int num_pages, int P, int H, int K, int window, float scale,
                     unsigned* err) {
    constexpr int CH = D / 8;       // 16-byte chunks per row
    constexpr int KS = D / 16;      // k-steps of q.k
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [128][D]
    bf16* k_s = q_s + PF_M * D;                                // [2][64][D]
    bf16* v_s = k_s + 2 * PF_N * D;                            // [2][64][D]
    int* row_s = reinterpret_cast<int*>(v_s + 2 * PF_N * D);   // [2][64] page rows of the tile's keys

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the list holds the tiles fewest keys first: start the longest, for all heads (heads run fastest in the grid)
    const int tile_i = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int r = tiles[2 * tile_i], q_off = tiles[2 * tile_i + 1];
    const int h = blockIdx.x, kvh = h / (H / K);
    const int t0 = q_start[r] + q_off;
    const int rows_valid = min(PF_M, q_len[r] - q_off);
    const int p0 = ctx_len[r] + q_off;              // position of the tile's first query
    const int p_last = p0 + rows_valid - 1;         // and of its last valid one
    const int* bt = block_table + (size_t)r * bt_width;

    // queries of this tile (rows past the portion are zero)
    for (int i = tid; i < PF_M * CH; i += PF_WARPS * 32) {
        const int row = i / CH, c = i % CH;
        const bool ok = row < rows_valid;
        const bf16* src = q + ((size_t)(t0 + (ok ? row : 0)) * H + h) * D + c * 8;
        cp_async16(tile_at<D>(q_s, row, c), src, ok);
    }
    cp_async_commit();

    int lo_min = 0;
    if (window > 0 && p0 - window + 1 > 0) lo_min = p0 - window + 1;
    const int kt_lo = lo_min / PF_N, kt_hi = p_last / PF_N;

    auto load_tile = [&](int kt, int buf) {
        // page rows of the 64 keys, then the copies
        if (tid < PF_N) {
            const int key = kt * PF_N + tid;
            int prow = -1;
            if (key <= p_last) {
                const int pidx = key / P;
                const int page = pidx < bt_width ? bt[pidx] : -1;
                if (page >= 0 && page < num_pages) prow = (page * K + kvh) * P + (key - pidx * P);
                else if (key >= lo_min) atomicOr(err, AIE_DEV_PAGE_OOB);   // behind a window a page may be gone
            }
            row_s[buf * PF_N + tid] = prow;
        }
        __syncthreads();
        bf16* kd = k_s + buf * PF_N * D;
        bf16* vd = v_s + buf * PF_N * D;
        for (int i = tid; i < PF_N * CH; i += PF_WARPS * 32) {
            const int row = i / CH, c = i % CH;
            const int prow = row_s[buf * PF_N + row];
            const bool ok = prow >= 0;
            const size_t off = (size_t)(ok ? prow : 0) * D + c * 8;
            cp_async16(tile_at<D>(kd, row, c), k_pages + off, ok);
            cp_async16(tile_at<D>(vd, row, c), v_pages + off, ok);
        }
        cp_async_commit();
    };

    load_tile(kt_lo, 0);

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    unsigned qf[KS][4];
    const int qrow0 = p0 + warp * 16 + (lane >> 2);     // position of this thread's first row; second is +8

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        if (kt < kt_hi) {
            load_tile(kt + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kt == kt_lo) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int mid = lane >> 3;
                ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                        tile_at<D>(q_s, warp * 16 + (mid & 1) * 8 + (lane & 7), ks * 2 + (mid >> 1)));
            }
        }
        const bf16* kb = k_s + buf * PF_N * D;
        const bf16* vb = v_s + buf * PF_N * D;

        // scores of 16 rows x 64 keys
        float s[PF_N / 8][4];
#pragma unroll
        for (int j = 0; j < PF_N / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int j = 0; j < PF_N / 8; j += 2) {
                const int mid = lane >> 3;
                unsigned b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3,
                        tile_at<D>(const_cast<bf16*>(kb), (j + (mid >> 1)) * 8 + (lane & 7), ks * 2 + (mid & 1)));
                mma16816(s[j], qf[ks], b0, b1);
                mma16816(s[j + 1], qf[ks], b2, b3);
            }
        }
        // scale, mask (only tiles that touch the diagonal, the end, or a window's edge)
        const int kbase = kt * PF_N;
        const bool edge = (kbase + PF_N - 1 > p0) || (window > 0 && kbase < p_last - window + 1 + PF_M);
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < PF_N / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * scale;
                if (edge) {
                    const int key = kbase + j * 8 + 2 * (lane & 3) + (e & 1);
                    const int qp = qrow0 + (e >> 1) * 8;
                    bool ok = key <= qp;
                    if (window > 0) ok = ok && key > qp - window;
                    if (!ok) v = -INFINITY;
                }
                s[j][e] = v;
                tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float tm = tmax[i];
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
            const float m_new = fmaxf(m_run[i], tm);
            m_use[i] = (m_new == -INFINITY) ? 0.f : m_new;          // a row with nothing visible yet
            corr[i] = (m_run[i] == -INFINITY) ? 0.f : __expf(m_run[i] - m_use[i]);
            m_run[i] = m_new;
        }
        float psum[2] = {0.f, 0.f};
        unsigned pf[PF_N / 16][4];
#pragma unroll
        for (int j = 0; j < PF_N / 8; ++j) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = __expf(s[j][e] - m_use[e >> 1]);     // exp(-inf) = 0 for masked keys
                psum[e >> 1] += p[e];
            }
            pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 1);
            psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 2);
            l_run[i] = l_run[i] * corr[i] + psum[i];
        }
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            o[j][0] *= corr[0];
            o[j][1] *= corr[0];
            o[j][2] *= corr[1];
            o[j][3] *= corr[1];
        }
        // o += p . v
#pragma unroll
        for (int kk = 0; kk < PF_N / 16; ++kk) {
#pragma unroll
            for (int jd = 0; jd < D / 8; jd += 2) {
                const int mid = lane >> 3;
                unsigned b0, b1, b2, b3;
                ldsm_x4_t(b0, b1, b2, b3,
                          tile_at<D>(const_cast<bf16*>(vb), kk * 16 + (mid & 1) * 8 + (lane & 7), jd + (mid >> 1)));
                mma16816(o[jd], pf[kk], b0, b1);
                mma16816(o[jd + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();     // everyone is done with this buffer before it is loaded again
    }

    // write the valid rows
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + (lane >> 2) + i * 8;
        if (row >= rows_valid) continue;
        const float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
        bf16* dst = out + ((size_t)(t0 + row) * H + h) * D + 2 * (lane & 3);
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(o[j][i * 2] * inv, o[j][i * 2 + 1] * inv);
        }
    }
}

template <int D> static size_t prefill_smem_bytes() {
    return (size_t)(PF_M * D + 4 * PF_N * D) * sizeof(bf16) + 2 * PF_N * sizeof(int);
}
