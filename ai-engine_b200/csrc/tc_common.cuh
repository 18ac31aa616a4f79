// Helpers shared by the tcgen05 kernels: mbarriers with bounded waits, TMA tile loads, shared-memory
// and instruction descriptors of tcgen05.mma, commit.
#pragma once
#include <cuda.h>

#include "common.cuh"

#define TC_WAIT_LIMIT (1u << 24)

__device__ __forceinline__ unsigned tc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_plain(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(tc_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(tc_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up or when another role has aborted.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                          unsigned* err) {
    if (mbar_test_wait(bar, parity)) return true;       // the phase is often over already: no blocking wait then
    for (unsigned i = 0; i < TC_WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(err, AIE_DEV_WAIT_TIMEOUT);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(tc_smem(dst)), "l"(map), "r"(tc_smem(bar)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, unsigned long long* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
                 ::"r"(tc_smem(dst)), "l"(map), "r"(tc_smem(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle, groups of
// 8 rows 1024 bytes apart (what the TMA load with SWIZZLE_128B writes).
__device__ __forceinline__ unsigned long long umma_desc(const void* tile, unsigned group_stride_bytes = 1024) {
    unsigned long long d = 0;
    d |= (unsigned long long)((tc_smem(tile) >> 4) & 0x3FFFu);   // start address / 16
    d |= (unsigned long long)1 << 16;                             // leading byte offset / 16 (unused under swizzle)
    d |= (unsigned long long)(group_stride_bytes >> 4) << 32;     // stride byte offset / 16: next group of 8 rows
    d |= (unsigned long long)1 << 46;                             // descriptor version of sm_100
    d |= (unsigned long long)2 << 61;                             // SWIZZLE_128B
    return d;
}
// bf16 x bf16 -> f32, M = 128, N = n; both operands K-major unless b_mn_major
__device__ __forceinline__ unsigned umma_idesc(int n, bool b_mn_major = false) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                     unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
                 : "memory");
}
// the same with the A operand in tensor memory: 128 lanes = rows, 16-bit elements packed two to a
// 32-bit column along K (a step of K = 16 is 8 columns)
__device__ __forceinline__ void umma_a_tmem(unsigned tmem_d, unsigned tmem_a, unsigned long long b, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}


// ---------------------------------------------------------------------------
// host: tensor maps (the driver entry point is looked up once; libcuda is not linked)
typedef CUresult (*TcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline TcEncodeTiledFn tc_encode_fn() {
    static TcEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (TcEncodeTiledFn)p;
    }
    return fn;
}

// bf16 matrix [rows, 64 * halves] (contiguous rows, rows a multiple of 8) seen as [groups of 8 rows][halves of
// 64 columns][8 rows][64]: a box of `box_groups` groups lands in shared memory as, per group, the 8 rows of
// the first 64 columns (1 KB, 128-byte swizzled), then the 8 rows of the next 64 columns, and so on
static inline int tc_make_map_rows8(CUtensorMap* map, const void* ptr, unsigned long long rows, int halves,
                                    int box_groups) {
    TcEncodeTiledFn fn = tc_encode_fn();
    if (!fn) return AIE_UNSUPPORTED;
    cuuint64_t dims[4] = {64, 8, (cuuint64_t)halves, (cuuint64_t)(rows / 8)};
    cuuint64_t strides[3] = {(cuuint64_t)halves * 128, 128, (cuuint64_t)halves * 1024};
    cuuint32_t box[4] = {64, 8, (cuuint32_t)halves, (cuuint32_t)box_groups};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : AIE_UNSUPPORTED;
}

// bf16 matrix [rows, cols] with rows `row_stride_bytes` apart, tiles of [box_rows, box_cols]
// (box_cols * 2 bytes = 128: one swizzle row), 128-byte swizzle, zeros outside the matrix
static inline int tc_make_map_2d(CUtensorMap* map, const void* ptr, unsigned long long rows, unsigned long long cols,
                                 unsigned long long row_stride_bytes, int box_rows, int box_cols) {
    TcEncodeTiledFn fn = tc_encode_fn();
    if (!fn) return AIE_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : AIE_BAD_ARG;
}
