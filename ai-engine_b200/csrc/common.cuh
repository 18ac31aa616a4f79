// Shared device helpers for the sm_100a kernels: dtype conversion, block
// reductions with a fixed order (so a row's result does not depend on what
// else is in the batch), and the device error word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

// dtype codes of the extern "C" launchers
#define AIE_F32 0
#define AIE_BF16 1

// launcher return codes (>0 are cudaError_t values)
#define AIE_BAD_ARG (-1)
#define AIE_UNSUPPORTED (-2)

// bits of the device error word that kernels set instead of trapping
#define AIE_DEV_TOKEN_OOB 1u    // token id outside the vocabulary
#define AIE_DEV_PAGE_OOB 2u     // block table entry outside the pool
#define AIE_DEV_WAIT_TIMEOUT 4u // a bounded wait ran out
#define AIE_DEV_SLOT_OOB 8u     // request row / slot outside its table

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// four consecutive elements (the address is 4-element aligned)
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
    return make_float4(__bfloat162float(e[0]), __bfloat162float(e[1]), __bfloat162float(e[2]), __bfloat162float(e[3]));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) {
    *reinterpret_cast<float4*>(p) = v;
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max; every thread gets the result.  `red` is >= 32 floats of
// shared memory.  The order of additions is fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Programmatic dependent launch: a kernel launched with launch_pdl may become resident
// while the kernel before it in the stream is still running.  It must call pdl_wait()
// before it reads anything an earlier kernel wrote and before it writes anything an
// earlier kernel may still read; pdl_launch_dependents() lets the kernel after it start
// becoming resident.  Work placed before pdl_wait() (setting up barriers, fetching
// weights) overlaps the tail of the previous kernel.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// AI_ENGINE_B200_NO_PDL=1 launches every kernel fully serialised (for measurement).
static inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("AI_ENGINE_B200_NO_PDL");
        on = (e && e[0] == '1') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// What the launchers size their grids by, asked from the current device once: the number of SMs and
// the shared memory of one SM (148 and 228 KB on a B200).
static inline int aie_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 1;
        n = v;
    }
    return n;
}
static inline int aie_smem_per_sm() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess || v <= 0)
            v = 48 * 1024;
        n = v;
    }
    return n;
}

#define AIE_LAUNCH_CHECK()                                   \
    do {                                                     \
        cudaError_t e__ = cudaGetLastError();                \
        return (int)e__;                                     \
    } while (0)
