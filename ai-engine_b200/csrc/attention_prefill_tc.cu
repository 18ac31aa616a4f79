// bfloat16 paged attention for portions of prompts on the fifth-generation tensor cores
// (head sizes 64 and 128): scores and outputs live in tensor memory, operands come from shared memory
// filled by TMA, softmax is float32 in registers.
//
// One CTA owns 128 query tokens of one head.  For each tile of 128 keys:
//   warp 0             loads the key tile and the value tile page by page with TMA: one box per page,
//                      lane i issuing the box of the tile's page i (the pool of a layer is seen as
//                      [groups of 8 rows][2 halves of the head][8 rows][64], so a box lands as 1 KB
//                      128-byte-swizzled atoms, the two halves of a group side by side), a ring of
//                      three buffers for keys and one of three for values (four at head size 64: a
//                      tile is requested when its buffer is freed, and a ring of two left the
//                      products waiting for loads), one mbarrier per stage counting the bytes of both;
//                      the loop has no division and
//                      reads the next tile's page id while this tile's boxes are issued;
//   warp 1 (one lane)  issues S = Q . K^T (8 x tcgen05.mma of K = 16) into one of two score buffers in
//                      tensor memory — the scores of the next tile are computed while the softmax of
//                      this one runs, so the softmax warps never wait for a round trip — later
//                      O += P . V (8 x tcgen05.mma; P is read from tensor memory, where the softmax
//                      wrote it over the scores; V is the MN-major operand: its rows are keys), and
//                      commits to the mbarriers the others wait on;
//   warps 2-5          softmax, one thread per query row: the row of S in registers (tcgen05.ld), masked
//                      on tiles that touch the diagonal or the sequence's end, its maximum; then
//                      the probabilities and their running sum (float32; the scale-and-subtract and
//                      the sum as packed f32x2 instructions), written as bf16 pairs into tensor
//                      memory.  The reference
//                      maximum of a row moves only when the new maximum exceeds it by more than 8
//                      (in units of log2 e): P stays below 2^8 and the row of O in tensor memory is
//                      rescaled on few tiles; the final division by the running sum makes the
//                      result the same softmax.
// The value rows of keys past the sequence's last token are zeroed in shared memory before the
// last tile's P . V, so a probability of 0 never meets what an unwritten cache slot holds.
// The softmax warps hand a tile's probabilities to the issuing warp at a named hardware barrier (bar.arrive /
// bar.sync); every mbarrier wait is bounded (see tc_common.cuh) and a wait that runs out raises the device error
// word; a softmax warp whose wait ran out still arrives at the named barrier for every tile, so the issuing warp's
// bar.sync always returns.
// Formula: crates/ai-engine-runtime/src/arch/attention.rs:148-157,177-196,203-224.
#include "tc_common.cuh"

#define AT_M 128          // query rows per CTA
#define AT_N 128          // keys per tile
#define AT_THREADS 192      // loader warp, MMA warp, 4 softmax warps
#define AT_HALF_BYTES (128 * 64 * 2)      // one [128 x 64] bf16 swizzle atom column: 16 KB

#define AT_BAR_P 1            // named barriers 1, 2: the probabilities of an even / odd key tile are in tensor memory
                              // (two, because a softmax warp may be a tile ahead of another: its arrival for
                              // tile j + 1 must not count for tile j)
#define AT_RESCALE_STEP 8.0f     // a row's reference maximum moves in steps of more than this (log2 units)

// HD: head size, HD / 64 halves of 64 columns.  A tile of 128 keys (or queries) holds 16 KB per half.
template <int HD> struct AtSmem {
    static constexpr int HV = HD / 64;
    static constexpr int tile = HV * AT_HALF_BYTES;
    // [alignment slack | 1 KB: barriers | Q | K x NST | V x NST]
    // rings of NST key tiles and NST value tiles: as deep as 227 KB allow (3 at head size 128), because a
    // tile is requested when its buffer is freed and a ring of two leaves the products waiting for loads
    static constexpr int NST = HD >= 128 ? 3 : 4;
    static constexpr int q_off = 1024, k_off = q_off + tile, v_off = k_off + NST * tile, end = v_off + NST * tile;
    static constexpr int bytes = 1024 + end;
};

// shared-memory descriptor of an MN-major operand: rows of 64 elements (128 bytes) along MN,
// groups of 8 K-rows `sbo` bytes apart, blocks of 64 MN elements `lbo` bytes apart
__device__ __forceinline__ unsigned long long umma_desc_mn(const void* tile, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((tc_smem(tile) >> 4) & 0x3FFFu);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}

#define AT_ST16(v, taddr)                                                                                             \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" \
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), \
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory")

__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ unsigned long long at_pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ float at_lo(unsigned long long v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo;
}
__device__ __forceinline__ float at_hi(unsigned long long v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return hi;
}

// 32 consecutive columns of this thread's lane of tensor memory
#define AT_LD32(v, taddr)                                                                                             \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                            \
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n" \
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),  \
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), \
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), \
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]) \
                 : "r"(taddr))
#define AT_ST32(v, taddr)                                                                                             \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                      \
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" \
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), \
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),     \
                   "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),   \
                   "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory")

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                        const int* __restrict__ tiles, int n_tiles, const int* __restrict__ q_start,
                        const int* __restrict__ q_len, const int* __restrict__ ctx_len,
                        const int* __restrict__ block_table, int bt_width, int num_pages, int P, int H, int K,
                        float scale, unsigned* err) {
    extern __shared__ unsigned char at_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>(((size_t)at_raw + 1023) & ~(size_t)1023);
    unsigned long long* q_full = reinterpret_cast<unsigned long long*>(sm);
    constexpr int NST = AtSmem<HD>::NST;           // stages of the key ring and of the value ring
    unsigned long long* kv_full = q_full + 1;      // [NST] keys and values of a tile have landed
    unsigned long long* k_empty = kv_full + NST;   // [NST] the scores have read the keys
    unsigned long long* v_empty = k_empty + NST;   // [NST] P . V has read the values
    unsigned long long* s_full = v_empty + NST;    // [2] score buffers
    unsigned long long* p_ready = s_full + 2;
    unsigned long long* o_done = p_ready + 1;
    unsigned long long* v_fixed = o_done + 1;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(v_fixed + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    constexpr int HV = HD / 64;                    // halves of 64 columns
    constexpr int TILE = AtSmem<HD>::tile;         // bytes of a 128-row tile
    constexpr int GROUP = HV * 1024;               // bytes of 8 rows (all halves) of a key or value tile
    unsigned char* q_s = sm + AtSmem<HD>::q_off;
    unsigned char* k_s = sm + AtSmem<HD>::k_off;   // stage st at + st * TILE
    unsigned char* v_s = sm + AtSmem<HD>::v_off;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // later tiles hold more keys: start them first, for all heads (heads run fastest in the grid, so the heads
    // of a group, which read the same keys, start side by side)
    const int tile_i = n_tiles - 1 - (int)blockIdx.y;
    const int r = tiles[2 * tile_i], q_off = tiles[2 * tile_i + 1];
    const int h = blockIdx.x, kvh = h / (H / K);
    const int t0 = q_start[r] + q_off;
    const int rows_valid = min(AT_M, q_len[r] - q_off);
    const int p0 = ctx_len[r] + q_off;                 // position of the tile's first query
    const int p_last = p0 + rows_valid - 1;            // and of its last valid one
    const int n_kt = p_last / AT_N + 1;                // key tiles 0 .. n_kt - 1
    const int ppt = AT_N / P;                          // pages per key tile

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(o_done, 1);
        mbar_init(v_fixed, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {    // tensor memory: score buffer b at columns [128 b, 128 b + 128) (P over its first 64),
                        // outputs at [256, 256 + head size)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
            if (lane == 0) {
            // queries of this tile: rows t0 .. t0 + 127 of q [T, H * 128], columns of head h
            mbar_expect_tx(q_full, TILE);
            for (int hv = 0; hv < HV; ++hv) tma_load_2d(q_s + hv * AT_HALF_BYTES, &map_q, q_full, h * HD + hv * 64, t0);
        }
        // lane i owns page i of every key tile: one box per page (all 128 columns of its P keys); the id of
        // the next tile's page is read while this tile's boxes are issued
        const int* bt = block_table + (size_t)r * bt_width;
        const int lp = 31 - __clz(P);                      // P is a power of two
        auto page_of = [&](int jj) {
            const int pidx = jj * ppt + lane;
            return (lane < ppt && (pidx << lp) <= p_last && pidx < bt_width) ? bt[pidx] : -1;
        };
        int page = page_of(0);
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int st = j % NST;
            const int page_next = j + 1 < n_kt ? page_of(j + 1) : -1;
            const int n_pages = min(ppt, ((p_last - j * AT_N) >> lp) + 1);      // pages of this tile that hold keys
            const bool have = lane < n_pages;
            const bool valid = have && page >= 0 && page < num_pages;
            if (have && !valid) atomicOr(err, AIE_DEV_PAGE_OOB);
            // a missing page is flagged; page 0 stands in for it so that the byte count of the barrier holds
            const int group0 = (((valid ? page : 0) * K + kvh) << lp) >> 3;     // first group of 8 rows of the page
            // one barrier counts the bytes of the tile's keys and values: the products wait once per tile
            if (lane == 0) {
                const unsigned ph = ((j / NST) & 1) ^ 1;
                ok = mbar_wait(&k_empty[st], ph, abort_flag, err) && mbar_wait(&v_empty[st], ph, abort_flag, err);
                if (ok) mbar_expect_tx(&kv_full[st], 2u * (unsigned)n_pages * (unsigned)P * (unsigned)(HD * 2));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (have) {
                tma_load_4d(k_s + st * TILE + lane * P * (HD * 2), &map_k, &kv_full[st], 0, 0, 0, group0);
                tma_load_4d(v_s + st * TILE + lane * P * (HD * 2), &map_v, &kv_full[st], 0, 0, 0, group0);
            }
            __syncwarp();
            page = page_next;
        }
        __syncwarp();
        // the last tile: zero the value rows of keys past the sequence's end (whole warp)
        {
            const int j = n_kt - 1, st = j % NST;
            const int first_bad = p_last + 1 - j * AT_N;       // rows [first_bad, 128) are not keys
            bool ok2 = true;
            if (first_bad < AT_N) {
                if (lane == 0) ok2 = mbar_wait(&kv_full[st], (j / NST) & 1, abort_flag, err);
                ok2 = __shfl_sync(0xffffffffu, ok2 ? 1 : 0, 0) != 0;
                if (ok2) {
                    unsigned char* vd = v_s + st * TILE;
                    const int n_bad = AT_N - first_bad;
                    for (int i = lane; i < n_bad * HV * 8; i += 32) {      // 8 chunks of 16 bytes per row and half
                        const int row = first_bad + i / (HV * 8), c = i % (HV * 8);
                        *reinterpret_cast<uint4*>(vd + (row >> 3) * GROUP + (c >> 3) * 1024 + (row & 7) * 128 + (c & 7) * 16) =
                            make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(v_fixed);
        }
    } else if (warp == 1) {
        // the whole warp walks the tiles (it meets the softmax warps at a named barrier); lane 0 issues
        {
            const unsigned idesc_s = umma_idesc(AT_N), idesc_o = umma_idesc(HD, true);
            // descriptors of the first step of each operand, built once; a step or a stage further along is an
            // addition to the descriptor's address field (bytes / 16)
            const unsigned long long dq0 = umma_desc(q_s), dk0 = umma_desc(k_s, GROUP), dv0 = umma_desc_mn(v_s, 1024, GROUP);
            // S(j) = Q . K(j)^T over the head size into score buffer j & 1: steps of 16; keys from stage `st`
            auto issue_scores = [&](int j, int st) {
                const unsigned long long dk = dk0 + (unsigned long long)((st * TILE) >> 4);
                const unsigned ts = tmem_base + (unsigned)((j & 1) * AT_N);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma(ts, dq0 + (unsigned long long)((((ks >> 2) * AT_HALF_BYTES) >> 4) + 2 * (ks & 3)),
                         dk + (unsigned long long)((((ks >> 2) * 1024) >> 4) + 2 * (ks & 3)), idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(&k_empty[st]);
                umma_commit(&s_full[j & 1]);
            };
            bool ok = true;                 // lane 0's; once false, the warp only keeps its appointments at the barrier
            if (lane == 0) {
                ok = mbar_wait(q_full, 0, abort_flag, err);
                if (ok) ok = mbar_wait(&kv_full[0], 0, abort_flag, err);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    issue_scores(0, 0);
                }
            }
            int st = 0, ph = 0;             // stage and phase of tile j in the rings
            for (int j = 0; j < n_kt; ++j) {
                const int st1 = st + 1 == NST ? 0 : st + 1, ph1 = st + 1 == NST ? ph ^ 1 : ph;      // of tile j + 1
                if (lane == 0 && ok && j + 1 < n_kt) {
                    // the next tile's scores, while this tile's softmax runs.  They go over the P of tile
                    // j - 1, which the P . V issued before them has read: the tensor pipe runs what one thread
                    // issues in order.
                    ok = mbar_wait(&kv_full[st1], ph1, abort_flag, err);
                    if (ok) {
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        issue_scores(j + 1, st1);
                    }
                }
                if (lane == 0 && ok && j == n_kt - 1) ok = mbar_wait(v_fixed, 0, abort_flag, err);
                // the tile's probabilities are written: the 128 softmax threads arrive, this warp waits.  A hardware
                // barrier: an mbarrier test costs the issuing thread some hundred cycles while the tensor pipe reads
                // shared memory, and this hand-over is on the tile's critical path (P . V, then the scores of the tile
                // after the next, which the softmax warps wait for).  (The tile's values landed with its keys.)
                asm volatile("bar.sync %0, %1;\n" ::"r"(AT_BAR_P + (j & 1)), "r"(AT_M + 32) : "memory");
                st = st1;
                ph = ph1;
                if (lane != 0 || !ok) continue;
                const int st0 = st == 0 ? NST - 1 : st - 1;      // the stage of tile j again
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // O += P . V over 128 keys: 8 steps of 16 keys; P is in tensor memory (two keys to a column),
                // V is MN-major: 16 keys = two groups of 8 rows, the halves of the head 1 KB apart
                const unsigned long long dv = dv0 + (unsigned long long)((st0 * TILE) >> 4);
                const unsigned tp = tmem_base + (unsigned)((j & 1) * AT_N);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_a_tmem(tmem_base + 256u, tp + (unsigned)(ks * 8), dv + (unsigned long long)((ks * 2 * GROUP) >> 4),
                                idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&v_empty[st0]);
                umma_commit(o_done);
            }
        }
    } else {
        // softmax: one thread per query row (warp w reads lanes 32 * (w % 4) .. + 31 of tensor memory)
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int qpos = p0 + row;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned tmem_o = tmem_base + 256u;
        const float sl2 = scale * 1.4426950408889634f;      // scores in units of log2(e): exp2 below
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kt; ++j) {
            // (a warp that gave up still arrives at the barrier for every tile: the issuing warp waits there
            // without a limit)
            const unsigned tmem_s = tmem_base + (unsigned)((j & 1) * AT_N);
            if (ok) {
                if (lane == 0) ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, err);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (!ok) {
                asm volatile("bar.arrive %0, %1;\n" ::"r"(AT_BAR_P + (j & 1)), "r"(AT_M + 32) : "memory");
                continue;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int kbase = j * AT_N;
            const bool edge = kbase + AT_N - 1 > p0;     // the tile touches the diagonal or the sequence's end
            // the row of scores in registers (all four loads in flight at once), masked; its maximum
            unsigned sv[128];
            AT_LD32((sv + 0), tmem_s + lane_addr + 0);
            AT_LD32((sv + 32), tmem_s + lane_addr + 32);
            AT_LD32((sv + 64), tmem_s + lane_addr + 64);
            AT_LD32((sv + 96), tmem_s + lane_addr + 96);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (edge) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (kbase + i > qpos) sv[i] = 0xff800000u;      // -inf: not visible
            }
            float tmax = -INFINITY, tmax2 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 128; i += 4) {
                tmax = at_max3(tmax, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
                tmax2 = at_max3(tmax2, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
            }
            tmax = fmaxf(tmax, tmax2) * sl2;
            // the row's reference maximum moves only by more than AT_RESCALE_STEP
            float m_new = m_run, corr = 1.0f;
            if (tmax > m_run + AT_RESCALE_STEP) {
                m_new = tmax;
                corr = (m_run == -INFINITY) ? 0.f : exp2f(m_run - tmax);
            }
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            m_run = m_new;
            // rows whose reference maximum moved rescale their row of O once the previous P . V has landed
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                if (lane == 0) ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, err);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) {
                    asm volatile("bar.arrive %0, %1;\n" ::"r"(AT_BAR_P + (j & 1)), "r"(AT_M + 32) : "memory");
                    continue;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    unsigned ov[32];
                    AT_LD32(ov, tmem_o + lane_addr + c0);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    AT_ST32(ov, tmem_o + lane_addr + c0);
                }
            }
            // probabilities exp2(s * sl2 - m), their sum, packed to bf16 and written over the scores, 32 columns
            // at a time: two keys to a column, so the P of columns [32 c, 32 c + 32) lands on [16 c, 16 c + 16)
            const unsigned long long sl2_2 = at_pack2(sl2, sl2), negm_2 = at_pack2(-m_use, -m_use);
            unsigned long long psum2 = 0ull, psum2b = 0ull;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                unsigned pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    unsigned long long x2;
                    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(x2) : "l"(at_pack2(__uint_as_float(sv[32 * c + i]), __uint_as_float(sv[32 * c + i + 1]))), "l"(sl2_2), "l"(negm_2));
                    float e0, e1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(at_lo(x2)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(at_hi(x2)));
                    if (i & 2) asm("add.rn.f32x2 %0, %1, %2;" : "=l"(psum2b) : "l"(psum2b), "l"(at_pack2(e0, e1)));
                    else asm("add.rn.f32x2 %0, %1, %2;" : "=l"(psum2) : "l"(psum2), "l"(at_pack2(e0, e1)));
                    __nv_bfloat162 bb = __floats2bfloat162_rn(e0, e1);
                    pk[i >> 1] = *reinterpret_cast<unsigned*>(&bb);
                }
                AT_ST16(pk, tmem_s + lane_addr + (unsigned)(16 * c));
            }
            asm("add.rn.f32x2 %0, %1, %2;" : "=l"(psum2) : "l"(psum2), "l"(psum2b));
            l_run = l_run * corr + (at_lo(psum2) + at_hi(psum2));
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            asm volatile("bar.arrive %0, %1;\n" ::"r"(AT_BAR_P + (j & 1)), "r"(AT_M + 32) : "memory");
        }
        // the last P . V, then this row of O divided by the row's sum
        if (ok) {
            if (lane == 0) ok = mbar_wait(o_done, (n_kt - 1) & 1, abort_flag, err);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            bf16* dst = out + ((size_t)(t0 + row) * H + h) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                unsigned ov[32];
                AT_LD32(ov, tmem_o + lane_addr + c0);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row < rows_valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        unsigned pk[4];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(ov[i + e]) * inv,
                                                                     __uint_as_float(ov[i + e + 1]) * inv);
                            pk[e >> 1] = *reinterpret_cast<unsigned*>(&b);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {      // give copies in flight a bounded time to land
        for (int s = 0; s < NST; ++s) {
            for (unsigned i = 0; i < (1u << 16) && !mbar_try_wait(&kv_full[s], 0) && !mbar_try_wait(&kv_full[s], 1); ++i) {}
        }
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

// ---------------------------------------------------------------------------
// The same for two tiles of 128 queries of one head per CTA (256 consecutive tokens of a request).
// Tensor memory holds one score buffer and one output per query tile (2 x 128 + 2 x head size columns);
// the alternation is between the tiles, not between two buffers of one tile: while the softmax warps of
// tile A exponentiate, the tensor pipe multiplies for tile B.  Keys and values are loaded once for both
// tiles, into one ring of slots (K0 V0 K1 V1 ...), each slot with its own full / empty barrier.
//   warps 0-3   softmax of tile A, one thread per query row
//   warps 4-7   softmax of tile B
//   warp 8      loader (as above)
//   warp 9      one lane issues the products of both tiles, tile A's then tile B's: per key tile j the tile's
//               P . V, then its scores for j + 1, which go over the tile's own P (the tensor pipe runs what
//               one thread issues in order, so the P . V has read it).  The serial issue is what staggers the
//               tiles by half a period; with an issuing warp for each tile the two softmaxes ran in
//               lockstep, fought for the exponential unit and left the pipe idle meanwhile (321 us against
//               232 us for 2,048 tokens after 6,144).  The warp meets the softmax warps at named barriers:
//               an mbarrier test cost the issuing thread some hundred cycles while the pipe reads shared
//               memory, and one stood between every softmax and its products (257 us).
//   warps 10-11 nothing: they fill the third warpgroup, which hands most of its registers to the softmax
//               warpgroups (setmaxnreg), whose threads keep a row of 128 scores each
// A tile's period is its chain softmax (about 2,000 cycles: 590 reading the row out of tensor memory, 1,400
// exponentials) -> 16 products (1,400) -> softmax; the pipe is busy three quarters of the time.  Tried without
// gain: exponentials taken against the old reference maximum while the row's chunks arrive (259 us), the
// probabilities handed over in two halves (240 us), a warp that waits for the loads in the issuing warp's place
// (233 us), the row read by one x128 load (233 us), a part of the exponentials as polynomials (slower).
// Tile B sees 128 more keys than tile A: A takes part in key tiles 0 .. nA - 1, B in all of the unit's.
#define AT2_THREADS 384
#define AT2_BAR_P 1         // named barriers 1, 2: the probabilities of tile A / B are in tensor memory

template <int HD> struct At2Smem {
    static constexpr int HV = HD / 64;
    static constexpr int tile = HV * AT_HALF_BYTES;
    static constexpr int NS = HD >= 128 ? 5 : 8;      // slots of the key / value ring
    // [alignment slack | 1 KB: barriers | Q of tile A | Q of tile B | NS slots]
    static constexpr int q_off = 1024, kv_off = q_off + 2 * tile, end = kv_off + NS * tile;
    static constexpr int bytes = 1024 + end;
};

template <int HD>
__global__ void __launch_bounds__(AT2_THREADS, 1)
paged_prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                             const int* __restrict__ units, int n_units, const int* __restrict__ q_start,
                             const int* __restrict__ q_len, const int* __restrict__ ctx_len,
                             const int* __restrict__ block_table, int bt_width, int num_pages, int P, int H, int K,
                             float scale, unsigned* err) {
    extern __shared__ unsigned char at_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>(((size_t)at_raw + 1023) & ~(size_t)1023);
    constexpr int NS = At2Smem<HD>::NS;
    unsigned long long* q_full = reinterpret_cast<unsigned long long*>(sm);
    unsigned long long* full = q_full + 1;         // [NS] the slot's keys or values have landed
    unsigned long long* empty = full + NS;         // [NS] the products have read the slot
    unsigned long long* s_full = empty + NS;       // [2] scores of tile A / B
    unsigned long long* o_done = s_full + 2;       // [2] the last P . V of tile A / B landed
    unsigned long long* v_fixed = o_done + 2;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(v_fixed + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    constexpr int HV = HD / 64;
    constexpr int TILE = At2Smem<HD>::tile;
    constexpr int GROUP = HV * 1024;
    unsigned char* q_s = sm + At2Smem<HD>::q_off;      // tile t at + t * TILE
    unsigned char* kv_s = sm + At2Smem<HD>::kv_off;    // slot s at + s * TILE

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit_i = n_units - 1 - (int)blockIdx.y;      // later units hold more keys: start them first
    const int r = units[2 * unit_i], q_off = units[2 * unit_i + 1];
    const int h = blockIdx.x, kvh = h / (H / K);
    const int t0 = q_start[r] + q_off;
    const int rows_all = min(2 * AT_M, q_len[r] - q_off);
    const int rows_a = min(AT_M, rows_all), rows_b = rows_all - rows_a;
    const int p0 = ctx_len[r] + q_off;                 // position of the unit's first query
    const int p_last = p0 + rows_all - 1;              // and of its last valid one
    const int n_kt = p_last / AT_N + 1;                // key tiles 0 .. n_kt - 1
    const int n_a = (p0 + rows_a - 1) / AT_N + 1;      // of these, tile A reads the first n_a,
    const int n_b = rows_b > 0 ? n_kt : 0;             // tile B all (none when the unit has no tile B)
    const int ppt = AT_N / P;

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&o_done[t], 1);
        }
        mbar_init(v_fixed, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 9) {    // tensor memory: scores (and P) of tile t at columns [128 t, 128 t + 128), outputs at
                        // [256 + t * head size, ...)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    // registers: the launch allots 168 to each of the 384 threads; the third warpgroup keeps 88 and the softmax
    // warpgroups take 208 each.  88 + 2 x 208 = 3 x 168: an increase waits, without a limit, for registers that a
    // decrease has released, so the three must never sum to more than the launch allotted.
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n");
    if (warp == 8) {
        if (lane == 0) {
            // queries: rows t0 .. t0 + 255 of q [T, H * head size], columns of head h (rows past T read as zeros)
            mbar_expect_tx(q_full, 2 * TILE);
            for (int t = 0; t < 2; ++t)
                for (int hv = 0; hv < HV; ++hv)
                    tma_load_2d(q_s + t * TILE + hv * AT_HALF_BYTES, &map_q, q_full, h * HD + hv * 64, t0 + t * AT_M);
        }
        const int* bt = block_table + (size_t)r * bt_width;
        const int lp = 31 - __clz(P);
        auto page_of = [&](int jj) {
            const int pidx = jj * ppt + lane;
            return (lane < ppt && (pidx << lp) <= p_last && pidx < bt_width) ? bt[pidx] : -1;
        };
        int page = page_of(0);
        bool ok = true;
        int slot = 0, ph = 0;           // ring position of the next item (K0 V0 K1 V1 ...)
        for (int j = 0; j < n_kt && ok; ++j) {
            const int page_next = j + 1 < n_kt ? page_of(j + 1) : -1;
            const int n_pages = min(ppt, ((p_last - j * AT_N) >> lp) + 1);
            const bool have = lane < n_pages;
            const bool valid = have && page >= 0 && page < num_pages;
            if (have && !valid) atomicOr(err, AIE_DEV_PAGE_OOB);
            const int group0 = (((valid ? page : 0) * K + kvh) << lp) >> 3;
#pragma unroll
            for (int item = 0; item < 2; ++item) {
                if (lane == 0) {
                    ok = mbar_wait(&empty[slot], (unsigned)(ph ^ 1), abort_flag, err);
                    if (ok) mbar_expect_tx(&full[slot], (unsigned)n_pages * (unsigned)P * (unsigned)(HD * 2));
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (have)
                    tma_load_4d(kv_s + slot * TILE + lane * P * (HD * 2), item == 0 ? &map_k : &map_v, &full[slot], 0, 0, 0,
                                group0);
                __syncwarp();
                if (++slot == NS) {
                    slot = 0;
                    ph ^= 1;
                }
            }
            page = page_next;
        }
        __syncwarp();
        // the last tile: zero the value rows of keys past the sequence's end (whole warp)
        {
            const int item = 2 * (n_kt - 1) + 1, st = item % NS;
            const int first_bad = p_last + 1 - (n_kt - 1) * AT_N;
            bool ok2 = ok;
            if (ok2 && first_bad < AT_N) {
                if (lane == 0) ok2 = mbar_wait(&full[st], (unsigned)((item / NS) & 1), abort_flag, err);
                ok2 = __shfl_sync(0xffffffffu, ok2 ? 1 : 0, 0) != 0;
                if (ok2) {
                    unsigned char* vd = kv_s + st * TILE;
                    const int n_bad = AT_N - first_bad;
                    for (int i = lane; i < n_bad * HV * 8; i += 32) {
                        const int row = first_bad + i / (HV * 8), c = i % (HV * 8);
                        *reinterpret_cast<uint4*>(vd + (row >> 3) * GROUP + (c >> 3) * 1024 + (row & 7) * 128 + (c & 7) * 16) =
                            make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(v_fixed);
        }
    } else if (warp == 9) {
        // The whole warp walks the tiles (it meets the softmax warps at a named barrier); lane 0 issues.
        const unsigned idesc_s = umma_idesc(AT_N), idesc_o = umma_idesc(HD, true);
        const unsigned long long dq0 = umma_desc(q_s), dk0 = umma_desc(kv_s, GROUP), dv0 = umma_desc_mn(kv_s, 1024, GROUP);
        // S_t = Q_t . K^T with the keys of ring slot `slot`
        auto issue_scores = [&](int t, int slot) {
            const unsigned long long dq = dq0 + (unsigned long long)((t * TILE) >> 4);
            const unsigned long long dk = dk0 + (unsigned long long)((slot * TILE) >> 4);
            const unsigned ts = tmem_base + (unsigned)(t * AT_N);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                umma(ts, dq + (unsigned long long)((((ks >> 2) * AT_HALF_BYTES) >> 4) + 2 * (ks & 3)),
                     dk + (unsigned long long)((((ks >> 2) * 1024) >> 4) + 2 * (ks & 3)), idesc_s, ks > 0 ? 1u : 0u);
        };
        // O_t += P_t . V with the values of ring slot `slot`
        auto issue_pv = [&](int t, int slot, bool first) {
            const unsigned long long dv = dv0 + (unsigned long long)((slot * TILE) >> 4);
            const unsigned tp = tmem_base + (unsigned)(t * AT_N), to = tmem_base + 256u + (unsigned)(t * HD);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_a_tmem(to, tp + (unsigned)(ks * 8), dv + (unsigned long long)((ks * 2 * GROUP) >> 4), idesc_o,
                            (!first || ks > 0) ? 1u : 0u);
        };
        auto advance = [&](int& s_, int& p_) {
            if (++s_ == NS) {
                s_ = 0;
                p_ ^= 1;
            }
        };
        int sv = 0, pv = 0;             // ring position of K(0), then of V(j)
        bool ok = true;                 // lane 0's; once false, the warp only keeps its appointments at the barriers
        if (lane == 0) {
            ok = mbar_wait(q_full, 0, abort_flag, err);
            if (ok) ok = mbar_wait(&full[sv], 0, abort_flag, err);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                issue_scores(0, sv);
                umma_commit(&s_full[0]);
                if (n_b > 0) {
                    issue_scores(1, sv);
                    umma_commit(&s_full[1]);
                }
                umma_commit(&empty[sv]);
            }
        }
        advance(sv, pv);
        for (int j = 0; j < n_kt; ++j) {
            int sk1 = sv, pk1 = pv;     // ring position of K(j + 1)
            advance(sk1, pk1);
            const bool in_b = j < n_b, next_b = j + 1 < n_b;
            // operands first: the values of this tile and the keys of the next landed long ago as a rule, and
            // nothing but the probabilities then stands between the end of a softmax and its products
            if (lane == 0 && ok) {
                ok = mbar_wait(&full[sv], (unsigned)pv, abort_flag, err);
                if (ok && j == n_kt - 1) ok = mbar_wait(v_fixed, 0, abort_flag, err);
                if (ok && j + 1 < n_kt) ok = mbar_wait(&full[sk1], (unsigned)pk1, abort_flag, err);
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int n_t = t == 0 ? n_a : n_b;
                if (j >= n_t) continue;
                // the tile's probabilities are written: its 128 softmax threads arrive, this warp waits.  A
                // hardware barrier: an mbarrier test costs the issuing thread some hundred cycles while the
                // tensor pipe reads shared memory, and stood between every softmax and its products.
                asm volatile("bar.sync %0, %1;\n" ::"r"(AT2_BAR_P + t), "r"(AT_M + 32) : "memory");
                if (lane != 0 || !ok) continue;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // P . V, then at once the next scores over the same columns (which the P . V has read: the
                // pipe runs what one thread issues in order); the commits follow both
                issue_pv(t, sv, j == 0);
                if (j + 1 < n_t) {
                    issue_scores(t, sk1);
                    umma_commit(&s_full[t]);        // covers the P . V too: the softmax may rescale O once it sees it
                } else {
                    umma_commit(&o_done[t]);        // the tile's last product
                }
                if (t == 1 || !in_b) umma_commit(&empty[sv]);                          // last reader of the values
                if (j + 1 < n_t && (t == 1 || !next_b)) umma_commit(&empty[sk1]);     // and of the next keys
            }
            sv = sk1;
            pv = pk1;
            advance(sv, pv);
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;\n");
        // softmax of tile t = warp / 4: one thread per query row (warp w reads lanes 32 * (w % 4) .. + 31)
        const int t = warp >> 2;
        const int n_t = t == 0 ? n_a : n_b;
        const int rows_valid = t == 0 ? rows_a : rows_b;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int p0_t = p0 + t * AT_M;
        const int qpos = p0_t + row;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned tmem_s = tmem_base + (unsigned)(t * AT_N);
        const unsigned tmem_o = tmem_base + 256u + (unsigned)(t * HD);
        const float sl2 = scale * 1.4426950408889634f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_t; ++j) {
            // (a warp that gave up still arrives at the barrier for every tile: the issuing warp waits there
            // without a limit)
            if (ok) {
                if (lane == 0) ok = mbar_wait(&s_full[t], (unsigned)(j & 1), abort_flag, err);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (!ok) {
                asm volatile("bar.arrive %0, %1;\n" ::"r"(AT2_BAR_P + t), "r"(AT_M + 32) : "memory");
                continue;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int kbase = j * AT_N;
            const bool edge = kbase + AT_N - 1 > p0_t;
            unsigned sv[128];
            AT_LD32((sv + 0), tmem_s + lane_addr + 0);
            AT_LD32((sv + 32), tmem_s + lane_addr + 32);
            AT_LD32((sv + 64), tmem_s + lane_addr + 64);
            AT_LD32((sv + 96), tmem_s + lane_addr + 96);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (edge) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (kbase + i > qpos) sv[i] = 0xff800000u;
            }
            float tmax = -INFINITY, tmax2 = -INFINITY, tmax3 = -INFINITY, tmax4 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
                tmax = at_max3(tmax, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
                tmax2 = at_max3(tmax2, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
                tmax3 = at_max3(tmax3, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
                tmax4 = at_max3(tmax4, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
            }
            tmax = fmaxf(at_max3(tmax, tmax2, tmax3), tmax4) * sl2;
            float m_new = m_run, corr = 1.0f;
            if (tmax > m_run + AT_RESCALE_STEP) {
                m_new = tmax;
                corr = (m_run == -INFINITY) ? 0.f : exp2f(m_run - tmax);
            }
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            m_run = m_new;
            // (the previous P . V has landed: the commit that announced these scores was issued after it)
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    unsigned ov[32];
                    AT_LD32(ov, tmem_o + lane_addr + c0);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    AT_ST32(ov, tmem_o + lane_addr + c0);
                }
            }
            const unsigned long long sl2_2 = at_pack2(sl2, sl2), negm_2 = at_pack2(-m_use, -m_use);
            unsigned long long psum2 = 0ull, psum2b = 0ull;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                unsigned pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    unsigned long long x2;
                    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(x2) : "l"(at_pack2(__uint_as_float(sv[32 * c + i]), __uint_as_float(sv[32 * c + i + 1]))), "l"(sl2_2), "l"(negm_2));
                    float e0, e1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(at_lo(x2)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(at_hi(x2)));
                    if (i & 2) asm("add.rn.f32x2 %0, %1, %2;" : "=l"(psum2b) : "l"(psum2b), "l"(at_pack2(e0, e1)));
                    else asm("add.rn.f32x2 %0, %1, %2;" : "=l"(psum2) : "l"(psum2), "l"(at_pack2(e0, e1)));
                    __nv_bfloat162 bb = __floats2bfloat162_rn(e0, e1);
                    pk[i >> 1] = *reinterpret_cast<unsigned*>(&bb);
                }
                AT_ST16(pk, tmem_s + lane_addr + (unsigned)(16 * c));
            }
            asm("add.rn.f32x2 %0, %1, %2;" : "=l"(psum2) : "l"(psum2), "l"(psum2b));
            l_run = l_run * corr + (at_lo(psum2) + at_hi(psum2));
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            asm volatile("bar.arrive %0, %1;\n" ::"r"(AT2_BAR_P + t), "r"(AT_M + 32) : "memory");
        }
        if (ok && n_t > 0) {
            if (lane == 0) ok = mbar_wait(&o_done[t], 0, abort_flag, err);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (ok && n_t > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            bf16* dst = out + ((size_t)(t0 + t * AT_M + row) * H + h) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                unsigned ov[32];
                AT_LD32(ov, tmem_o + lane_addr + c0);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (row < rows_valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        unsigned pk[4];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(ov[i + e]) * inv,
                                                                     __uint_as_float(ov[i + e + 1]) * inv);
                            pk[e >> 1] = *reinterpret_cast<unsigned*>(&b);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {      // give copies in flight a bounded time to land
        for (int s = 0; s < NS; ++s) {
            for (unsigned i = 0; i < (1u << 16) && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i) {}
        }
    }
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

template <int HD>
static int launch_prefill_tc_pair(const void* q, const void* k_pages, const void* v_pages, void* out, const int* units,
                                  int n_units, const int* q_start, const int* q_len, const int* ctx_len,
                                  const int* block_table, int bt_width, int num_pages, int P, int T, int H, int K,
                                  float scale, unsigned* err, cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    int rc = tc_make_map_2d(&mq, q, (unsigned long long)T, (unsigned long long)H * HD, (unsigned long long)H * HD * 2, AT_M, 64);
    if (rc) return rc;
    const unsigned long long rows = (unsigned long long)num_pages * K * P;
    rc = tc_make_map_rows8(&mk, k_pages, rows, HD / 64, P / 8);
    if (rc) return rc;
    rc = tc_make_map_rows8(&mv, v_pages, rows, HD / 64, P / 8);
    if (rc) return rc;
    cudaFuncSetAttribute(paged_prefill_tc_pair_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, At2Smem<HD>::bytes);
    paged_prefill_tc_pair_kernel<HD><<<dim3(H, n_units), AT2_THREADS, At2Smem<HD>::bytes, stream>>>(
        mq, mk, mv, (bf16*)out, units, n_units, q_start, q_len, ctx_len, block_table, bt_width, num_pages, P, H, K,
        scale, err);
    AIE_LAUNCH_CHECK();
}

template <int HD>
static int launch_prefill_tc(const void* q, const void* k_pages, const void* v_pages, void* out, const int* tiles,
                             int n_tiles, const int* q_start, const int* q_len, const int* ctx_len,
                             const int* block_table, int bt_width, int num_pages, int P, int T, int H, int K,
                             float scale, unsigned* err, cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    int rc = tc_make_map_2d(&mq, q, (unsigned long long)T, (unsigned long long)H * HD, (unsigned long long)H * HD * 2, AT_M, 64);
    if (rc) return rc;
    const unsigned long long rows = (unsigned long long)num_pages * K * P;
    rc = tc_make_map_rows8(&mk, k_pages, rows, HD / 64, P / 8);
    if (rc) return rc;
    rc = tc_make_map_rows8(&mv, v_pages, rows, HD / 64, P / 8);
    if (rc) return rc;
    cudaFuncSetAttribute(paged_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, AtSmem<HD>::bytes);
    paged_prefill_tc_kernel<HD><<<dim3(H, n_tiles), AT_THREADS, AtSmem<HD>::bytes, stream>>>(
        mq, mk, mv, (bf16*)out, tiles, n_tiles, q_start, q_len, ctx_len, block_table, bt_width, num_pages, P, H, K,
        scale, err);
    AIE_LAUNCH_CHECK();
}

// q, out: [T, H, d] bf16; k_pages, v_pages: [num_pages, K, P, d] bf16 of one layer;
// tiles: [n_tiles][2] = (request row, offset of the 128-token tile within the request's tokens).
// Takes head sizes 64 and 128, pages of 8 .. 128 keys that divide 128 and layers without a window; refuses the
// rest (AIE_UNSUPPORTED): they take the mma.sync kernel.
extern "C" int aie_paged_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                              const int* tiles, int n_tiles, const int* q_start, const int* q_len,
                                              const int* ctx_len, const int* block_table, int bt_width,
                                              int num_pages, int P, int T, int H, int K, int d, int window,
                                              float scale, unsigned* err, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (K <= 0 || H % K) return AIE_BAD_ARG;
    if ((d != 64 && d != 128) || P < 8 || P > 128 || 128 % P || n_tiles > 65535 || window > 0) return AIE_UNSUPPORTED;
    if (((size_t)q & 15) || ((size_t)k_pages & 15) || ((size_t)v_pages & 15)) return AIE_UNSUPPORTED;
#define ARGS q, k_pages, v_pages, out, tiles, n_tiles, q_start, q_len, ctx_len, block_table, bt_width, num_pages, P, T, H, K, \
             scale, err, stream
    return d == 128 ? launch_prefill_tc<128>(ARGS) : launch_prefill_tc<64>(ARGS);
#undef ARGS
}

// The same with two query tiles per CTA.  units: [n_units][2] = (request row, offset of the 256-token unit
// within the request's tokens; a unit's last tile may be short or missing).  Same sizes as above.
extern "C" int aie_paged_attention_prefill_tc_pair(const void* q, const void* k_pages, const void* v_pages, void* out,
                                                   const int* units, int n_units, const int* q_start,
                                                   const int* q_len, const int* ctx_len, const int* block_table,
                                                   int bt_width, int num_pages, int P, int T, int H, int K, int d,
                                                   int window, float scale, unsigned* err, cudaStream_t stream) {
    if (n_units <= 0) return 0;
    if (K <= 0 || H % K) return AIE_BAD_ARG;
    if ((d != 64 && d != 128) || P < 8 || P > 128 || 128 % P || n_units > 65535 || window > 0) return AIE_UNSUPPORTED;
    if (((size_t)q & 15) || ((size_t)k_pages & 15) || ((size_t)v_pages & 15)) return AIE_UNSUPPORTED;
#define ARGS q, k_pages, v_pages, out, units, n_units, q_start, q_len, ctx_len, block_table, bt_width, num_pages, P, T, H, K, \
             scale, err, stream
    return d == 128 ? launch_prefill_tc_pair<128>(ARGS) : launch_prefill_tc_pair<64>(ARGS);
#undef ARGS
}
