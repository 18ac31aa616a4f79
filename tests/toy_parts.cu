// Kernel of a toy mixer that the tests define outside the package: an exponential moving average over a
// request's tokens, s <- decay * s + h[t] * w, out[t] = s, with s kept in the request's state slot.
// One block per request of the step; its tokens run in order.  A row that only rounds the batch up
// (live[r] == 0) computes its output and leaves the state alone.
#include "common.cuh"

template <typename T>
__global__ void toy_ema_kernel(const T* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                               T* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ q_len,
                               const int* __restrict__ slots, const int* __restrict__ live, int D, int max_slots,
                               float decay, unsigned* err) {
    pdl_wait();
    const int r = blockIdx.x;
    const int slot = slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIE_DEV_SLOT_OOB);
        return;
    }
    const int a = q_start[r], n = q_len[r];
    const bool keep = live[r] != 0;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float s = state[(size_t)slot * D + c];
        const float wc = w[c];
        for (int t = a; t < a + n; ++t) {
            s = decay * s + to_f32(h[(size_t)t * D + c]) * wc;
            out[(size_t)t * D + c] = from_f32<T>(s);
        }
        if (keep) state[(size_t)slot * D + c] = s;
    }
}

extern "C" int toy_ema_scan(const void* h, int dtype, const float* w, float* state, void* out, const int* q_start,
                            const int* q_len, const int* slots, const int* live, int R, int D, int max_slots,
                            float decay, unsigned* err, cudaStream_t st) {
    if (R <= 0 || D <= 0) return AIE_BAD_ARG;
    if (dtype == AIE_F32)
        launch_pdl(toy_ema_kernel<float>, dim3(R), dim3(128), 0, st, (const float*)h, w, state, (float*)out, q_start,
                   q_len, slots, live, D, max_slots, decay, err);
    else if (dtype == AIE_BF16)
        launch_pdl(toy_ema_kernel<bf16>, dim3(R), dim3(128), 0, st, (const bf16*)h, w, state, (bf16*)out, q_start,
                   q_len, slots, live, D, max_slots, decay, err);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
