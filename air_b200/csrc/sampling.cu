// Choosing the next token on the device: the lowest index of the maximum (greedy), or an
// index drawn from softmax(logits / temperature), optionally cut to the k largest logits and then
// to the shortest prefix of the descending order whose weights reach the share p (AIR's sampler,
// src/runtime/sampling.cpp:9-62: top-k after a stable descending sort, then top-p, at least one kept),
// with a uniform number that the host supplies for the row.  One block per row of logits [R, V]
// (float32).  Nothing is sorted: the k-th largest logit and the logit at which the share is reached
// are found by bisection over the logits' bit patterns (32 counting passes over the row, which lies
// in L2), ties at such a value are kept in index order as a stable sort would; the draw then walks
// the kept indices in index order, which gives AIR's distribution but, for the same uniform number,
// not the token that AIR's walk in descending order gives (the host sampler does that).
#include "common.cuh"

namespace air {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// temperature == nullptr or temperature[r] <= 0: greedy.  Otherwise the drawn index is the
// first i (in index order) with sum_{j<=i} w_j >= u * sum_j w_j, w_j = exp((x_j - max) / T).
// With slots and last_token the chosen index is also stored at last_token[slots[r]], where the
// embedding kernel of the next step finds it.
// A row whose maximum is not finite sets *status (AIR flags non-finite logits on the device,
// src/cuda/cuda_backend.cu:621-624).
// A float's bits as an unsigned number of the same order.
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_total(float v, float* scratch32) {     // every thread gets the sum
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch32[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < SAMPLE_THREADS / 32; ++i) t += scratch32[i];
    return t;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, const int* __restrict__ top_k, const float* __restrict__ top_p,
              int* __restrict__ out, const int* __restrict__ slots, int* __restrict__ last_token, int V,
              int* status) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float partial[SAMPLE_THREADS];
    __shared__ float s_max;
    __shared__ int s_arg;
    pdl_enter(TR_SAMPLE);
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * V;

    float v = -INFINITY;
    int idx = 0x7fffffff;
    bool bad = false;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float xi = x[i];
        if (!(fabsf(xi) <= 3.4e38f)) bad = true;
        argmax_combine(v, idx, xi, i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(v, idx, ov, oi);
    }
    if (__syncthreads_or(bad) && tid == 0 && status) atomicExch(status, 3);
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w) argmax_combine(v, idx, sv[w], si[w]);
        s_max = v;
        s_arg = idx == 0x7fffffff ? 0 : idx;
    }
    __syncthreads();
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) {
            out[r] = s_arg;
            if (slots && last_token) last_token[slots[r]] = s_arg;
        }
        return;
    }
    // contiguous chunk per thread, so that ties and the walk are in index order
    const float inv_t = 1.f / temp;
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(V, tid * chunk), end = min(V, begin + chunk);
    __shared__ int tie_before[SAMPLE_THREADS];      // ties at the cut's value in the chunks before this thread's
    __shared__ float s_w32[32];

    // The kept set is {key > cut} and the first `ties` indices with key == cut.  Without a cut: everything.
    uint32_t cut = 0;
    int ties = 0x7fffffff;

    // Which threshold keeps exactly what a stable descending sort cut at `need` would keep, where `need` is a
    // count (WEIGHTED = false: the k largest) or a mass of weights (WEIGHTED = true: the share p), among
    // the indices that the cut so far keeps.
    auto kept = [&](uint32_t key, int tie_rank) { return key > cut || (key == cut && tie_rank < ties); };
    const int k = top_k ? top_k[r] : 0;
    const float share = top_p ? top_p[r] : 1.f;
    for (int pass = 0; pass < 2; ++pass) {
        const bool weighted = pass == 1;
        if (!weighted && !(k > 0 && k < V)) continue;
        if (weighted && !(share < 1.f)) continue;
        // what is kept so far, as a count or a mass
        float need;
        {
            int rank = 0;
            // (tie ranks of the cut so far: recount this thread's start)
            int mine = 0;
            for (int i = begin; i < end; ++i) mine += order_key(x[i]) == cut ? 1 : 0;
            tie_before[tid] = mine;
            __syncthreads();
            if (tid == 0) {
                int run = 0;
                for (int i = 0; i < SAMPLE_THREADS; ++i) { const int c = tie_before[i]; tie_before[i] = run; run += c; }
            }
            __syncthreads();
            rank = tie_before[tid];
            float acc = 0.f;
            for (int i = begin; i < end; ++i) {
                const uint32_t key = order_key(x[i]);
                const bool in = kept(key, rank);
                if (key == cut) ++rank;
                if (in) acc += weighted ? expf((x[i] - s_max) * inv_t) : 1.f;
            }
            const float total = block_total(acc, s_w32);
            need = weighted ? share * total : (float)k;
            if (!weighted && total <= need) continue;         // fewer than k are there at all
        }
        // the largest key K with measure{kept so far, key >= K} >= need
        uint32_t lo = 0, hi = 0xffffffffu;
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2 + 1;
            int rank = tie_before[tid];
            float acc = 0.f;
            for (int i = begin; i < end; ++i) {
                const uint32_t key = order_key(x[i]);
                const bool in = kept(key, rank);
                if (key == cut) ++rank;
                if (in && key >= mid) acc += weighted ? expf((x[i] - s_max) * inv_t) : 1.f;
            }
            if (block_total(acc, s_w32) >= need) lo = mid; else hi = mid - 1;
        }
        // how many of the ties at that key are kept: as many as it takes to reach `need` (at least one)
        int rank = tie_before[tid];
        float above = 0.f;
        for (int i = begin; i < end; ++i) {
            const uint32_t key = order_key(x[i]);
            const bool in = kept(key, rank);
            if (key == cut) ++rank;
            if (in && key > lo) above += weighted ? expf((x[i] - s_max) * inv_t) : 1.f;
        }
        above = block_total(above, s_w32);
        // weight of one tie = weight of the key `lo` itself (some kept index has exactly this key)
        float one = 1.f;
        if (weighted) {
            const uint32_t b = (lo & 0x80000000u) ? (lo & 0x7fffffffu) : ~lo;
            one = expf((__uint_as_float(b) - s_max) * inv_t);
        }
        int new_ties = (int)ceilf((need - above) / one - 1e-6f);
        new_ties = max(1, new_ties);
        if (lo == cut && ties != 0x7fffffff) new_ties = min(new_ties, ties);
        cut = lo;
        ties = new_ties;
        __syncthreads();
    }

    // tie ranks of the final cut, then the walk over the kept indices in index order
    {
        int mine = 0;
        for (int i = begin; i < end; ++i) mine += order_key(x[i]) == cut ? 1 : 0;
        tie_before[tid] = mine;
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int i = 0; i < SAMPLE_THREADS; ++i) { const int c = tie_before[i]; tie_before[i] = run; run += c; }
        }
        __syncthreads();
    }
    float sum = 0.f;
    {
        int rank = tie_before[tid];
        for (int i = begin; i < end; ++i) {
            const uint32_t key = order_key(x[i]);
            const bool in = kept(key, rank);
            if (key == cut) ++rank;
            if (in) sum += expf((x[i] - s_max) * inv_t);
        }
    }
    partial[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) total += partial[i];
        const float target = uniform[r] * total;
        float cum = 0.f;
        int owner = SAMPLE_THREADS - 1;
        for (int i = 0; i < SAMPLE_THREADS; ++i) {
            if (cum + partial[i] >= target && partial[i] > 0.f) { owner = i; break; }
            cum += partial[i];
        }
        const int b = min(V, owner * chunk), e = min(V, b + chunk);
        int chosen = s_arg;
        int rank = tie_before[owner];
        for (int i = b; i < e; ++i) {
            const uint32_t key = order_key(x[i]);
            const bool in = kept(key, rank);
            if (key == cut) ++rank;
            if (!in) continue;
            cum += expf((x[i] - s_max) * inv_t);
            chosen = i;
            if (cum >= target) break;
        }
        out[r] = chosen;
        if (slots && last_token) last_token[slots[r]] = chosen;
    }
}

}  // namespace air

// top_k [R] int (0: off) and top_p [R] float (1: off) may be null.
AIR_API int air_sample(const float* logits, const float* temperature, const float* uniform, const int* top_k,
                       const float* top_p, int* out, const int* slots, int* last_token, int R, int V, int* status,
                       cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::sample_kernel, R, air::SAMPLE_THREADS, 0, stream, logits, temperature, uniform, top_k,
                       top_p, out, slots, last_token, V, status);
}

AIR_API int air_trace_set_sampling(unsigned long long* buffer) { return air::set_trace_here(buffer); }
