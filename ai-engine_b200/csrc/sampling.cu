// Sampling on the device, one block per row of logits
// (crates/ai-engine-runtime/src/sample.rs:12-55):
//   temperature == 0  -> argmax, the first maximum wins (strict '>', :51-55);
//   otherwise x = logit / T; order by x descending (ties: lower index first);
//   top-k keeps the first k; softmax with the maximum subtracted; top-p keeps the
//   shortest prefix whose mass reaches p; a uniform draw r walks the cumulative
//   sum in that order until r <= acc.
// Nothing is sorted.  "The first element of the descending order at which the
// cumulative weight reaches a target" is found by a radix search over the
// order-preserving bits of x, 8 bits a pass, with per-bin weights summed in
// shared memory; weights are counts (top-k) or exp(x - max) in 2^-40 fixed point
// (top-p and the draw), so sums are integers: exact, and the same on every run.
// The reference seeds a new generator on every call, so each step of a request
// draws the same r (:41); here r comes from the caller, one per request and step.
#include "common.cuh"

#define SAMPLE_THREADS 512
typedef unsigned long long u64;

__device__ __forceinline__ unsigned order_key(float x) {
    const unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Cut {  // elements at or before (key, idx) in the descending order are eligible
    unsigned key;
    int idx;
};
__device__ __forceinline__ bool eligible(unsigned key, int i, const Cut& c) {
    return key > c.key || (key == c.key && i <= c.idx);
}
__device__ __forceinline__ u64 fixed_mass(float x, float m) {
    return (u64)((double)expf(x - m) * 1099511627776.0);  // 2^40
}

struct SelectShared {
    u64 hist[256];
    u64 before;
    unsigned prefix;
    int found_idx;
    int warp_tot[SAMPLE_THREADS / 32];
    int n_ties;
    int min_idx;
    int done;
};

// First position of the descending order (restricted to `cut`) whose inclusive
// cumulative weight is >= target.  Returns its key and index and that weight.
__device__ void select_prefix(const float* __restrict__ row, int V, float T, float m, Cut cut,
                              bool by_mass, u64 target, SelectShared* s, unsigned* key_out,
                              int* idx_out, u64* acc_incl) {
    const int tid = threadIdx.x;
    if (tid == 0) { s->before = 0; s->prefix = 0; }
    unsigned mask = 0;
    for (int pass = 3; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int b = tid; b < 256; b += SAMPLE_THREADS) s->hist[b] = 0;
        __syncthreads();
        const unsigned prefix = s->prefix;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float x = row[i] / T;
            const unsigned key = order_key(x);
            if ((key & mask) != prefix || !eligible(key, i, cut)) continue;
            const u64 w = by_mass ? fixed_mass(x, m) : 1ull;
            if (w) atomicAdd(&s->hist[(key >> shift) & 255u], w);
        }
        __syncthreads();
        if (tid == 0) {
            u64 cum = s->before;
            int found = -1, last = -1;
            for (int b = 255; b >= 0; --b) {
                const u64 h = s->hist[b];
                if (!h) continue;
                last = b;
                if (cum + h >= target) { found = b; break; }
                cum += h;
            }
            if (found < 0) {          // target beyond the total (rounding): the last element
                found = last < 0 ? 0 : last;
                if (last >= 0) cum -= s->hist[last];
            }
            s->before = cum;
            s->prefix = prefix | ((unsigned)found << shift);
        }
        __syncthreads();
        mask |= 0xffu << shift;
    }
    const unsigned key = s->prefix;
    // ties: equal x, equal weight, ordered by index
    int cnt = 0, mn = 0x7fffffff;
    float xt = 0.f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = row[i] / T;
        if (order_key(x) == key && eligible(key, i, cut)) { ++cnt; mn = min(mn, i); xt = x; }
    }
    if (tid == 0) { s->n_ties = 0; s->min_idx = 0x7fffffff; s->found_idx = -1; s->done = 0; }
    __syncthreads();
    if (cnt) { atomicAdd(&s->n_ties, cnt); atomicMin(&s->min_idx, mn); }
    __syncthreads();
    const int n_ties = s->n_ties;
    const u64 before = s->before;
    // every thread derives the same rank j (1-based) among the ties
    u64 w = 1;
    if (by_mass) {
        // the tie weight: threads that saw a tie know x; share through hist[0]
        if (cnt && mn == s->min_idx) s->hist[0] = fixed_mass(xt, m);
        __syncthreads();
        w = s->hist[0];
    }
    long long j = 1;
    if (n_ties > 1 && w > 0 && target > before) {
        const u64 need = target - before;
        j = (long long)((need + w - 1) / w);
        if (j < 1) j = 1;
        if (j > n_ties) j = n_ties;
    }
    int idx = s->min_idx;
    if (j > 1) {
        int running = 0;
        const int lane = tid & 31, warp = tid >> 5;
        for (int base = 0; base < V; base += SAMPLE_THREADS) {
            const int i = base + tid;
            bool f = false;
            if (i < V) {
                const float x = row[i] / T;
                f = order_key(x) == key && eligible(key, i, cut);
            }
            const unsigned bal = __ballot_sync(0xffffffffu, f);
            if (lane == 0) s->warp_tot[warp] = __popc(bal);
            __syncthreads();
            int off = running, tot = 0;
            for (int wv = 0; wv < SAMPLE_THREADS / 32; ++wv) {
                const int c = s->warp_tot[wv];
                if (wv < warp) off += c;
                tot += c;
            }
            const int incl = off + __popc(bal & ((2u << lane) - 1u));
            if (f && incl == (int)j) { s->found_idx = i; s->done = 1; }
            running += tot;
            __syncthreads();
            if (s->done) break;
        }
        idx = s->found_idx;
    }
    __syncthreads();
    *key_out = key;
    *idx_out = idx;
    *acc_incl = before + (u64)j * w;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, int ld,
                   const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, const float* __restrict__ uniform,
                   int* __restrict__ out) {
    __shared__ SelectShared sel;
    __shared__ float red[32];
    __shared__ float best_v[SAMPLE_THREADS / 32];
    __shared__ int best_i[SAMPLE_THREADS / 32];
    __shared__ u64 zsum;
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature[r];

    if (T == 0.0f || V <= 1) {   // greedy: the first maximum
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float v = row[i];
            if (v > bv) { bv = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31) == 0) { best_v[tid >> 5] = bv; best_i[tid >> 5] = bi; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
                if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
            out[r] = (bi == 0x7fffffff) ? 0 : bi;
        }
        return;
    }

    float mx = -INFINITY;
    for (int i = tid; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, row[i] / T);
    const float m = block_max(mx, red);

    Cut cut{0u, 0x7fffffff};
    unsigned key;
    int idx;
    u64 acc;
    const int k = top_k[r];
    if (k > 0 && k < V) {
        select_prefix(row, V, T, m, cut, false, (u64)k, &sel, &key, &idx, &acc);
        cut.key = key;
        cut.idx = idx;
    }
    if (tid == 0) zsum = 0;
    __syncthreads();
    u64 zl = 0;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = row[i] / T;
        if (eligible(order_key(x), i, cut)) zl += fixed_mass(x, m);
    }
    if (zl) atomicAdd(&zsum, zl);
    __syncthreads();
    u64 Z = zsum;
    const float p = top_p[r];
    if (p > 0.f && p < 1.f) {
        u64 target = (u64)ceil((double)p * (double)Z);
        if (target < 1) target = 1;
        select_prefix(row, V, T, m, cut, true, target, &sel, &key, &idx, &acc);
        cut.key = key;
        cut.idx = idx;
        Z = acc;
    }
    u64 target = (u64)ceil((double)uniform[r] * (double)Z);
    if (target < 1) target = 1;
    if (target > Z) target = Z;
    select_prefix(row, V, T, m, cut, true, target, &sel, &key, &idx, &acc);
    if (tid == 0) out[r] = idx < 0 || idx >= V ? 0 : idx;
}

// Greedy alone, a row spread over `gridDim.y` blocks: each block packs its best (value, first index) as
// (order bits << 32 | ~index), so that an atomic maximum keeps the largest value and, among equals, the
// lowest index; the block that finishes last for a row writes the id and leaves the scratch zeroed.
// One block per row reads 513 KB of logits through one SM: 16 us at a vocabulary of 128K.
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const float* __restrict__ logits, int V, int ld, u64* __restrict__ best,
                   int* __restrict__ tickets, int* __restrict__ out) {
    __shared__ u64 wbest[8];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int per = (V + gridDim.y - 1) / gridDim.y;
    const int lo = blockIdx.y * per, hi = min(V, lo + per);
    u64 b = 0;
    for (int i = lo + tid; i < hi; i += 256) {
        const float v = row[i];
        if (v == v) {       // a NaN is never the maximum
            const u64 k = ((u64)order_key(v) << 32) | (u64)(0xFFFFFFFFu - (unsigned)i);
            b = k > b ? k : b;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const u64 ob = __shfl_xor_sync(0xffffffffu, b, o);
        b = ob > b ? ob : b;
    }
    if ((tid & 31) == 0) wbest[tid >> 5] = b;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; ++w) b = wbest[w] > b ? wbest[w] : b;
        if (b) atomicMax(&best[r], b);
        __threadfence();
        if (atomicAdd(&tickets[r], 1) == (int)gridDim.y - 1) {
            __threadfence();
            const u64 w = atomicExch(&best[r], 0ull);
            out[r] = w ? (int)(0xFFFFFFFFu - (unsigned)(w & 0xFFFFFFFFull)) : 0;
            tickets[r] = 0;
        }
    }
}

// out[r] = index of the first maximum of row r.  best [N] (64-bit) and tickets [N] must be zero on entry and
// are zero again on return.
extern "C" int aie_argmax_rows(const float* logits, int N, int V, int ld, void* best, int* tickets, int* out,
                               cudaStream_t stream) {
    if (N <= 0) return 0;
    if (V <= 0) return AIE_BAD_ARG;
    int chunks = (V + 8191) / 8192;         // at least 8K logits a block
    if (chunks > 32) chunks = 32;
    argmax_rows_kernel<<<dim3(N, chunks), 256, 0, stream>>>(logits, V, ld, (u64*)best, tickets, out);
    AIE_LAUNCH_CHECK();
}

extern "C" int aie_sample_rows(const float* logits, int N, int V, int ld, const float* temperature,
                               const int* top_k, const float* top_p, const float* uniform, int* out,
                               cudaStream_t stream) {
    if (N <= 0) return 0;
    if (V <= 0) return AIE_BAD_ARG;
    sample_rows_kernel<<<N, SAMPLE_THREADS, 0, stream>>>(logits, V, ld, temperature, top_k, top_p,
                                                         uniform, out);
    AIE_LAUNCH_CHECK();
}
