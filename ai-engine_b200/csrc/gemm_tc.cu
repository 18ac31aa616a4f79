// bfloat16 matrix product on the fifth-generation tensor cores:
//     C[T, N] = X[T, K] . W[N, K]^T          (weights as stored: [out, in])
// computed as D^T = W . X^T so that the weight matrix is the 128-row operand of
// tcgen05.mma and the tokens are its N dimension (16 .. 256).  Few tokens (decode)
// make this a pure weight stream, many tokens (prompts) a compute-bound product;
// the kernel is the same, only the token tile BN differs.
//
// One CTA owns one 128-row tile of W, one tile of BN tokens and one part of K
// (split-K across gridDim.z when the grid would otherwise not fill the machine).
// Warp roles:
//   warp 0 (one lane)  producer: TMA (cp.async.bulk.tensor.2d) loads of the W tile
//                      [128 x 64] and the X tile [BN x 64] of each K block into a
//                      ring of shared-memory stages, 128-byte swizzled, completion
//                      counted in bytes on the stage's "full" mbarrier;
//   warp 1 (one lane)  issues four tcgen05.mma (K = 16 each) per stage from shared-
//                      memory descriptors into the float32 accumulator in tensor
//                      memory, then tcgen05.commit, which releases the stage ("empty"
//                      mbarrier) when those products have read it; warp 1 also owns
//                      the tensor-memory allocation;
//   warps 2-5          epilogue: after the last commit, tcgen05.ld their quarter of
//                      the accumulator (lane = weight row, column = token) and store
//                      C[token][row] (32 lanes write 32 consecutive rows of a token).
// Split K: the CTAs that share an output tile form a thread-block cluster along z.
// Each stores its float32 partial tile in its own shared memory; after a cluster
// barrier every CTA adds, for its share of the tile, the tiles of all through distributed
// shared memory in rank order (so the sum does not depend on timing), applies the
// epilogue and stores.  Or the parts are left unjoined (`raw_parts`: float32
// [parts, T, N]) for a consumer that adds them (the norm and rotary kernels).
// Epilogues: plain store (bf16 or float32); SwiGLU on a weight whose 128-row tiles
// hold 64 gate rows followed by their 64 up rows: a[t, f] = silu(g) * u in float32
// (crates/ai-engine-runtime/src/arch/ffn.rs:50-54); or, for the fused q/k/v projection
// of a small step, the rotation of q and k by position and the write of k and v into
// their cache pages (a 128-row tile holds whole heads).
// The kernel is launched as a programmatic dependent: barriers, tensor memory and the
// first weight tiles of the ring are set up and requested before griddepcontrol.wait,
// while the previous kernel is still finishing; only the token tiles wait for it.
// Every wait is bounded: after WAIT_LIMIT polls a thread raises the CTA's abort
// flag and the device error word, the other roles leave their loops, copies in
// flight are waited for (bounded), tensor memory is freed and the CTA returns.
#include "tc_common.cuh"

#define TC_BM 128           // weight rows per tile (the MMA's M)
#define TC_BK 64            // K elements per stage (128 bytes: one swizzle row)
#define TC_THREADS 192

template <typename OT> __device__ __forceinline__ void tc_store(OT* p, float v);
template <> __device__ __forceinline__ void tc_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void tc_store<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int BN> struct TcSmem {
    static constexpr int stage_bytes = TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    static constexpr int max_stages = BN <= 64 ? 8 : (BN <= 128 ? 6 : 4);     // what 227 KB hold
    // the ring depth is chosen per launch: a grid of at most one CTA per SM takes the deepest ring
    // (one CTA must keep its SM's share of the memory system busy); a larger grid takes the deepest
    // ring with which its CTAs still share an SM and cover each other's start and end
    static constexpr int tile_bytes = BN * TC_BM * 4;      // the float32 tile staged for joining parts
    // [alignment slack | 1024 bytes of barriers | ring of stages, reused for the staged tile]
    static constexpr int bytes_for(int stages) {
        return 2048 + (stages * stage_bytes > tile_bytes ? stages * stage_bytes : tile_bytes);
    }
};

#define TC_EPI_STORE 0
#define TC_EPI_SWIGLU 1
#define TC_EPI_ROPE 2       // the fused q/k/v projection: rotate q and k by position, write k and v into their pages

// What the rotary epilogue needs beside the product: the step's positions and block table, the pages of
// the layer and the rotation's frequencies (rotation: crates/ai-engine-runtime/src/arch/rope.rs:38-44,66-106;
// cache write: crates/ai-engine-candle/src/paged/attention.rs:59-83).  The output columns are
// [H q heads | K k heads | K v heads] x d with d dividing 128, so a 128-row weight tile holds whole heads.
struct TcRope {
    bf16* q_out;              // [T, H, d]
    bf16* k_pages;            // [num_pages, K, P, d]
    bf16* v_pages;
    const int* positions;     // [T]
    const int* token_req;     // [T] row of the block table
    const int* block_table;   // [R, bt_width]
    const float* inv_freq;    // [d / 2]
    int bt_width, num_pages, P, H, K, d, write;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the float at `addr` (a shared-memory address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ float ld_peer(unsigned addr, unsigned rank) {
    unsigned peer;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(peer) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(peer) : "memory");
    return v;
}
// the sum over the cluster's CTAs, in rank order, of the float at `addr` in each: all loads are issued before
// the first is used (a load from another CTA's shared memory takes some hundred cycles)
__device__ __forceinline__ float sum_peers(unsigned addr, int parts) {
    float v[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) v[p] = p < parts ? ld_peer(addr, p) : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) acc += v[p];
    return acc;
}

template <int BN, int EPI, typename OT>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               OT* __restrict__ C, int T, int N, int K, int ldc, int kb_per_split, int STAGES, int raw_parts,
               unsigned* err, const TcRope rope) {
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ unsigned char tc_raw[];
    unsigned char* bars = reinterpret_cast<unsigned char*>(((size_t)tc_raw + 1023) & ~(size_t)1023);
    unsigned char* base = bars + 1024;                    // the ring, 1024-byte aligned
    unsigned long long* full = reinterpret_cast<unsigned long long*>(bars);
    unsigned long long* empty = full + 8;
    unsigned long long* accum = empty + 8;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(accum + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* tile_s = reinterpret_cast<float*>(base);      // [BN][128] partial tile, after the ring is idle

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * TC_BM, t0 = blockIdx.y * BN;
    // parts of K: joined inside a cluster (parts == cluster size), or left to the consumer
    // (raw_parts: part z is stored as it is at C + z * T * ldc and the next kernel adds them)
    const int parts = raw_parts ? 1 : gridDim.z;
    if (raw_parts) C += (size_t)blockIdx.z * T * ldc;
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(kb_begin + kb_per_split, kb_total);
    const int nkb = max(kb_end - kb_begin, 0);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {   // tensor memory for the accumulator: 128 lanes x TMEM_COLS columns of float32
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_d = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // weights do not depend on the previous kernel: request the first ring of W tiles now
            const int pre = min(nkb, STAGES);
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&full[i], TcSmem<BN>::stage_bytes);
                tma_load_2d(base + i * TcSmem<BN>::stage_bytes, &map_w, &full[i], (kb_begin + i) * TC_BK, n0);
            }
            pdl_wait();        // the tokens are the previous kernel's output
            for (int i = 0; i < pre; ++i)
                tma_load_2d(base + i * TcSmem<BN>::stage_bytes + TC_BM * TC_BK * 2, &map_x, &full[i],
                            (kb_begin + i) * TC_BK, t0);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES;
                const unsigned ph = (i / STAGES) & 1;
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err)) break;
                unsigned char* st = base + s * TcSmem<BN>::stage_bytes;
                mbar_expect_tx(&full[s], TcSmem<BN>::stage_bytes);
                const int k = (kb_begin + i) * TC_BK;
                tma_load_2d(st, &map_w, &full[s], k, n0);
                tma_load_2d(st + TC_BM * TC_BK * 2, &map_x, &full[s], k, t0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && nkb > 0) {
            const unsigned idesc = umma_idesc(BN);
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const unsigned ph = (i / STAGES) & 1;
                ok = mbar_wait(&full[s], ph, abort_flag, err);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                unsigned char* st = base + s * TcSmem<BN>::stage_bytes;
                const unsigned long long da = umma_desc(st), db = umma_desc(st + TC_BM * TC_BK * 2);
#pragma unroll
                for (int j = 0; j < TC_BK / 16; ++j)     // 32 bytes further along K inside the swizzled row
                    umma(tmem_d, da + 2 * j, db + 2 * j, idesc, (i > 0 || j > 0) ? 1u : 0u);
                umma_commit(&empty[s]);                  // the stage is free once these products have read it
            }
            if (ok) umma_commit(accum);                  // the accumulator is complete
        }
    } else {
        // epilogue warps 2..5 read lanes 32 * (warp % 4) .. + 31 of tensor memory: lane = weight row
        const int quarter = warp & 3;
        bool ok = nkb > 0;
        if (ok) ok = mbar_wait(accum, 0, abort_flag, err);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;      // the whole warp follows lane 0's verdict
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        pdl_wait();             // nothing is stored before the previous kernel is done with its buffers
        const int r = quarter * 32 + lane;               // row of the tile
        const bool direct = parts == 1 && EPI == TC_EPI_STORE;
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 16) {
            unsigned v[16];
            if (ok) {
                const unsigned taddr = tmem_d + ((unsigned)(quarter * 32) << 16) + (unsigned)c0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                               "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
                               "=r"(v[14]), "=r"(v[15])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;      // a part without K blocks (or an abort) adds nothing
            }
            if (direct) {
                if (n0 + r < N) {        // a part without K blocks stores zeros: its consumer adds every part
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c0 + j;
                        if (t >= T) break;
                        tc_store<OT>(C + (size_t)t * ldc + n0 + r, __uint_as_float(v[j]));
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) tile_s[(c0 + j) * TC_BM + r] = __uint_as_float(v[j]);
            }
        }
    }

    if (parts > 1 || EPI != TC_EPI_STORE) {
        // join the parts: every CTA of the cluster has its tile in shared memory; each CTA sums
        // and stores its share of the tile's tokens, reading the others' tiles in rank order
        __syncwarp();
        if (parts > 1) cluster_sync_all(); else __syncthreads();
        if (warp >= 2 && !*abort_flag) {
            const int e = tid - 64;                        // 0 .. 127
            const unsigned tile_addr = tc_smem(tile_s);
            const int rank = (int)cluster_rank();
            const int tokens = min(BN, T - t0);
            constexpr int COLS = EPI == TC_EPI_STORE ? TC_BM : TC_BM / 2;      // outputs per token
            const int total = tokens * COLS;
            const int share = (total + parts - 1) / parts;
            const int f0 = blockIdx.x * COLS, width = EPI == TC_EPI_STORE ? N : N / 2;
            for (int idx = rank * share + e; idx < min((rank + 1) * share, total); idx += 128) {
                const int tt = idx / COLS, j = idx % COLS;
                if (EPI == TC_EPI_ROPE) {
                    // pair (i, i + d/2) of head slot `slot`: columns c1, c2 of the tile
                    const int hd = rope.d, half = hd / 2;
                    const int hh = j / half, i = j % half;
                    const int c1 = hh * hd + i, c2 = c1 + half;
                    const int slot = blockIdx.x * (TC_BM / hd) + hh;
                    float x1 = sum_peers(tile_addr + (tt * TC_BM + c1) * 4, parts);
                    float x2 = sum_peers(tile_addr + (tt * TC_BM + c2) * 4, parts);
                    const int t = t0 + tt;
                    const int pos = rope.positions[t];
                    if (slot >= rope.H + 2 * rope.K) continue;
                    if (slot < rope.H + rope.K) {        // q and k heads are rotated; the angle in float32
                        float sn, cs;
                        sincosf((float)pos * rope.inv_freq[i], &sn, &cs);
                        const float o1 = x1 * cs - x2 * sn, o2 = x1 * sn + x2 * cs;
                        x1 = o1;
                        x2 = o2;
                    }
                    bf16* dst;
                    if (slot < rope.H) {
                        dst = rope.q_out + ((size_t)t * rope.H + slot) * hd;
                    } else {
                        if (!rope.write) continue;           // the pages are another run's
                        const int pidx = pos / rope.P;
                        const int page = (pidx < rope.bt_width && pos >= 0)
                                             ? rope.block_table[(size_t)rope.token_req[t] * rope.bt_width + pidx] : -1;
                        if (page < 0 || page >= rope.num_pages) {
                            atomicOr(err, AIE_DEV_PAGE_OOB);
                            continue;
                        }
                        const bool is_v = slot >= rope.H + rope.K;
                        const int kh = slot - rope.H - (is_v ? rope.K : 0);
                        dst = (is_v ? rope.v_pages : rope.k_pages) +
                              (((size_t)page * rope.K + kh) * rope.P + (pos - pidx * rope.P)) * hd;
                    }
                    dst[i] = __float2bfloat16_rn(x1);
                    dst[i + half] = __float2bfloat16_rn(x2);
                    continue;
                }
                float out;
                if (EPI == TC_EPI_STORE) {
                    out = sum_peers(tile_addr + (tt * TC_BM + j) * 4, parts);
                } else {     // rows 0..63 of the tile are gate rows, rows 64..127 their up rows
                    const float g = sum_peers(tile_addr + (tt * TC_BM + j) * 4, parts);
                    const float u = sum_peers(tile_addr + (tt * TC_BM + 64 + j) * 4, parts);
                    // sigmoid by ex2.approx and rcp.approx (relative error about 1e-6; the result is rounded to bf16)
                    float e, r;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
                    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
                    out = (g * r) * u;
                }
                if (f0 + j < width) tc_store<OT>(C + (size_t)(t0 + tt) * ldc + f0 + j, out);
            }
        }
        __syncwarp();
        if (parts > 1) cluster_sync_all();       // every CTA keeps its tile until the others have read it
    }

    // leave together; on an abort, give copies in flight a bounded time to land first
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {
        for (int s = 0; s < STAGES; ++s)
            for (unsigned i = 0; i < (1u << 16) && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i) {}
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(TMEM_COLS));
    }
}

// a [rows, K] bf16 row-major matrix, tiles of [box_rows, 64], 128-byte swizzle, zeros outside
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    return tc_make_map_2d(map, ptr, (unsigned long long)rows, (unsigned long long)K, (unsigned long long)K * 2,
                          box_rows, TC_BK);
}

template <int BN, int EPI, typename OT>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int T, int N, int K, int ldc,
                     int splits, int raw_parts, unsigned* err, cudaStream_t st, const TcRope& rope = TcRope()) {
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    const int kbps = (kb_total + splits - 1) / splits;
    auto kern = gemm_tc_kernel<BN, EPI, OT>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + TC_BM - 1) / TC_BM, (T + BN - 1) / BN, splits);
    const long long ctas = (long long)cfg.gridDim.x * cfg.gridDim.y * cfg.gridDim.z;
    // the deepest ring that still lets the grid's CTAs sit beside each other: one, two or three to an SM
    // (228 KB of shared memory an SM, 1 KB of it reserved per CTA); a grid of more than three waves
    // takes the ring for three
    const int sms = aie_sm_count();
    const int per_sm = ctas <= sms ? 1 : (ctas <= 2 * sms ? 2 : 3);
    int stages = (aie_smem_per_sm() / per_sm - 1024 - 2048) / TcSmem<BN>::stage_bytes;
    if (stages > TcSmem<BN>::max_stages) stages = TcSmem<BN>::max_stages;
    if (stages < 2) stages = 2;
    if (stages > kbps) stages = kbps < 2 ? 2 : kbps;
    const int smem = TcSmem<BN>::bytes_for(stages);
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<BN>::bytes_for(TcSmem<BN>::max_stages));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    ++na;
    if (splits > 1 && !raw_parts) {      // the parts of one output tile are one cluster
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = splits;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mw, mx, (OT*)C, T, N, K, ldc, kbps, stages, raw_parts, err, rope);
    return (int)e;
}

// bn: token tile (16, 32, 64, 128, 256).  splits: parts of K: 1 .. 8 joined in a cluster, or, with
// raw_parts (float32 output only, no swiglu), any number stored one after the other: C is [splits, T, N].
// swiglu: W is [2F, K] in 128-row tiles of 64 gate rows + their 64 up rows (N = 2F), C is [T, F].
// Requires K % 8 == 0 (16-byte rows) and 16-byte aligned X and W.
extern "C" int aie_gemm_tc(const void* X, const void* W, void* C, int out_dtype, int T, int N, int K, int ldc,
                           int bn, int splits, int swiglu, int raw_parts, unsigned* err, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((size_t)X & 15) || ((size_t)W & 15)) return AIE_UNSUPPORTED;
    if (splits < 1 || (!raw_parts && splits > 8) || splits > 65535) return AIE_BAD_ARG;
    if (raw_parts && (swiglu || out_dtype != AIE_F32)) return AIE_BAD_ARG;
    if (out_dtype != AIE_BF16 && out_dtype != AIE_F32) return AIE_BAD_ARG;
    if (swiglu && N % 128) return AIE_UNSUPPORTED;
    if ((T + bn - 1) / bn > 65535) return AIE_UNSUPPORTED;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, N, K, TC_BM);
    if (rc) return rc;
    rc = make_map(&mx, X, T, K, bn);
    if (rc) return rc;
#define GO(BNV)                                                                                                   \
    if (swiglu)                                                                                                   \
        rc = out_dtype == AIE_BF16 ? launch_tc<BNV, TC_EPI_SWIGLU, bf16>(mw, mx, C, T, N, K, ldc, splits, raw_parts, err, stream)  \
                                   : launch_tc<BNV, TC_EPI_SWIGLU, float>(mw, mx, C, T, N, K, ldc, splits, raw_parts, err, stream); \
    else                                                                                                          \
        rc = out_dtype == AIE_BF16 ? launch_tc<BNV, TC_EPI_STORE, bf16>(mw, mx, C, T, N, K, ldc, splits, raw_parts, err, stream)   \
                                   : launch_tc<BNV, TC_EPI_STORE, float>(mw, mx, C, T, N, K, ldc, splits, raw_parts, err, stream)
    switch (bn) {
        case 16: GO(16); break;
        case 32: GO(32); break;
        case 64: GO(64); break;
        case 128: GO(128); break;
        case 256: GO(256); break;
        default: return AIE_BAD_ARG;
    }
#undef GO
    return rc;
}

// The fused q/k/v projection of a small step: qkv = X . W^T with K cut into `splits` parts (1 .. 8) joined in a
// cluster, then, in the same kernel, q and k rotated by position (full rotation: inv_freq has d / 2 entries),
// q written to q_out [T, H, d] and k, v into their cache pages.  d must divide 128 and N = (H + 2 K) d be a
// multiple of 128; float32 sums, float32 angles.
extern "C" int aie_gemm_tc_rope(const void* X, const void* W, int T, int N, int K, int bn, int splits, void* q_out,
                                void* k_pages, void* v_pages, const int* positions, const int* token_req,
                                const int* block_table, int bt_width, int num_pages, int P, int H, int Kh, int d,
                                const float* inv_freq, int write, unsigned* err, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (K <= 0 || K % 8 || ((size_t)X & 15) || ((size_t)W & 15)) return AIE_UNSUPPORTED;
    if (d < 2 || d % 2 || TC_BM % d || N != (H + 2 * Kh) * d || N % TC_BM) return AIE_UNSUPPORTED;
    if (splits < 1 || splits > 8) return AIE_BAD_ARG;
    if ((T + bn - 1) / bn > 65535) return AIE_UNSUPPORTED;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, N, K, TC_BM);
    if (rc) return rc;
    rc = make_map(&mx, X, T, K, bn);
    if (rc) return rc;
    TcRope r;
    r.q_out = (bf16*)q_out; r.k_pages = (bf16*)k_pages; r.v_pages = (bf16*)v_pages;
    r.positions = positions; r.token_req = token_req; r.block_table = block_table; r.inv_freq = inv_freq;
    r.bt_width = bt_width; r.num_pages = num_pages; r.P = P; r.H = H; r.K = Kh; r.d = d; r.write = write;
    switch (bn) {
        case 16: return launch_tc<16, TC_EPI_ROPE, float>(mw, mx, nullptr, T, N, K, N, splits, 0, err, stream, r);
        case 32: return launch_tc<32, TC_EPI_ROPE, float>(mw, mx, nullptr, T, N, K, N, splits, 0, err, stream, r);
        case 64: return launch_tc<64, TC_EPI_ROPE, float>(mw, mx, nullptr, T, N, K, N, splits, 0, err, stream, r);
        default: return AIE_BAD_ARG;
    }
}

// A wait that nothing will ever satisfy, with a short limit: shows that a bounded wait gives up,
// raises the device error word (AIE_DEV_WAIT_TIMEOUT) and lets the kernel return.
__global__ void tc_wait_selftest_kernel(unsigned* err, int polls) {
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        bool done = false;
        for (int i = 0; i < polls && !done; ++i) done = mbar_try_wait(&bar, 0);
        if (!done) atomicOr(err, AIE_DEV_WAIT_TIMEOUT);
    }
}

extern "C" int aie_tc_wait_selftest(unsigned* err, int polls, cudaStream_t stream) {
    if (polls < 1 || polls > (1 << 20)) return AIE_BAD_ARG;
    tc_wait_selftest_kernel<<<1, 32, 0, stream>>>(err, polls);
    AIE_LAUNCH_CHECK();
}
