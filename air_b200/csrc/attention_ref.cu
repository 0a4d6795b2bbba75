// Paged attention with 32-bit arithmetic for any batch: portions of prompts and single
// decoded tokens alike.  It is the kernel of the float32 path and the fallback of the
// bfloat16 path for head sizes that the tensor-core kernels do not take.
//
// One block per (token, query head), four warps.  Keys are visited in blocks of 32 aligned
// to their absolute position; warp w takes the blocks whose index is w modulo 4, keeps a
// running maximum, sum and weighted value (online softmax), and the four partial results
// are merged in a fixed order.  What a query computes therefore depends only on its
// position and on the cache's contents, not on how the tokens were cut into steps or on
// what else is in the batch.
//
// q, out: [T, H, d].  cache: [page, 2, K, P, d] (keys then values).  block_table: [slots, max_blocks],
// row token_seq[t] for token t (negative: padding, skipped).
// A query at position p sees keys max(0, p - window + 1) .. p (window 0: all keys).
#include "common.cuh"

namespace air {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_ref_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                           const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ token_seq, const int* __restrict__ positions,
                           T* __restrict__ out, int H, int K, int d, int P, int window, float scale) {
    __shared__ float sq[ATT_MAX_D];
    __shared__ float sm[ATT_WARPS], sl[ATT_WARPS];
    __shared__ float sacc[ATT_WARPS][ATT_MAX_D];
    pdl_enter(TR_ATT_REF);
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (token_seq[t] < 0) return;  // padding
    const int pos = positions[t];
    const int kvh = (int)(((long long)h * K) / H);
    const int* bt = block_table + (size_t)token_seq[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    for (int i = threadIdx.x; i < d; i += blockDim.x) sq[i] = to_float(q[((size_t)t * H + h) * d + i]);
    __syncthreads();

    const int chunks = (d + 31) / 32;
    float acc[ATT_MAX_D / 32];
#pragma unroll
    for (int c = 0; c < ATT_MAX_D / 32; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    const size_t page_stride = (size_t)2 * K * P * d;
    const size_t v_offset = (size_t)K * P * d;
    for (int b = (lo / 32 / ATT_WARPS) * ATT_WARPS + warp; b * 32 <= pos; b += ATT_WARPS) {
        const int key = b * 32 + lane;
        const bool valid = key >= lo && key <= pos;
        size_t base = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[key / P];
            base = (size_t)page * page_stride + ((size_t)kvh * P + (size_t)(key % P)) * d;
            const T* kp = cache + base;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot = fmaf(sq[i], to_float(kp[i]), dot);
            s = dot * scale;
        }
        const float bm = warp_max(s);
        if (bm == -INFINITY) continue;  // the whole block is outside the window
        const float m_new = fmaxf(m, bm);
        const float corr = expf(m - m_new);  // 0 when m was -inf
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < ATT_MAX_D / 32; ++c) acc[c] *= corr;
        m = m_new;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
            if (pj == 0.f) continue;  // same for the whole warp
            const T* vp = cache + bj + v_offset;
#pragma unroll
            for (int c = 0; c < ATT_MAX_D / 32; ++c) {
                const int i = c * 32 + lane;
                if (c < chunks && i < d) acc[c] = fmaf(pj, to_float(vp[i]), acc[c]);
            }
        }
    }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int c = 0; c < ATT_MAX_D / 32; ++c) {
        const int i = c * 32 + lane;
        if (c < chunks && i < d) sacc[warp][i] = acc[c];
    }
    __syncthreads();
    float mm = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm[w]);
    float total = 0.f;
    float weight[ATT_WARPS];
    for (int w = 0; w < ATT_WARPS; ++w) {
        weight[w] = sm[w] == -INFINITY ? 0.f : expf(sm[w] - mm);
        total += sl[w] * weight[w];
    }
    const float inv = 1.f / total;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) o += sacc[w][i] * weight[w];
        out[((size_t)t * H + h) * d + i] = from_float<T>(o * inv);
    }
}

}  // namespace air

AIR_API int air_paged_attention_ref(const void* q, const void* cache, int dtype, const int* block_table,
                                    int max_blocks, const int* token_seq, const int* positions, void* out,
                                    int T, int H, int K, int d, int P, int window, float scale,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > air::ATT_MAX_D || H <= 0 || K <= 0 || H > 65535) return AIR_ERR_BAD_ARGUMENT;
    dim3 grid(T, H);
    AIR_DISPATCH(dtype, TT, {
        return air::launch(air::paged_attention_ref_kernel<TT>, grid, air::ATT_WARPS * 32, 0, stream, (const TT*)q,
                           (const TT*)cache, block_table, max_blocks, token_seq, positions, (TT*)out, H, K, d, P,
                           window, scale);
    });
    return 0;
}

AIR_API int air_trace_set_attention_ref(unsigned long long* buffer) { return air::set_trace_here(buffer); }
