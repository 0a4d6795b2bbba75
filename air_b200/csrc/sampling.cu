// Choosing the next token on the device: the lowest index of the maximum (greedy), or an
// index drawn from softmax(logits / temperature) with a uniform number that the host
// supplies for the row.  One block per row of logits [R, V] (float32).
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
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out, const int* __restrict__ slots,
              int* __restrict__ last_token, int V, int* status) {
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
    // contiguous chunk per thread, so that the walk is in index order
    const float inv_t = 1.f / temp;
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(V, tid * chunk), end = min(V, begin + chunk);
    float sum = 0.f;
    for (int i = begin; i < end; ++i) sum += expf((x[i] - s_max) * inv_t);
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
        for (int i = b; i < e; ++i) {
            cum += expf((x[i] - s_max) * inv_t);
            chosen = i;
            if (cum >= target) break;
        }
        out[r] = chosen;
        if (slots && last_token) last_token[slots[r]] = chosen;
    }
}

}  // namespace air

AIR_API int air_sample(const float* logits, const float* temperature, const float* uniform, int* out,
                       const int* slots, int* last_token, int R, int V, int* status, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::sample_kernel, R, air::SAMPLE_THREADS, 0, stream, logits, temperature, uniform, out,
                       slots, last_token, V, status);
}

AIR_API int air_trace_set_sampling(unsigned long long* buffer) { return air::set_trace_here(buffer); }
