// True 32-bit matrix product on the CUDA cores: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
// No tensor cores and no reduced-precision mode.  Every element of C is accumulated over k
// in ascending order by one thread with fused multiply-adds, so a row of C does not depend
// on which other rows are in the batch: the 32-bit path gives the same bits for a token
// whether it is computed alone, in a portion of a prompt or in a mixed batch.
#include "common.cuh"

namespace air {

constexpr int GB = 64;   // tile of C is GB x GB
constexpr int GK = 16;   // k-step

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                       const float* __restrict__ bias, float* __restrict__ C,
                                                       int M, int N, int K) {
    __shared__ float sa[GK][GB + 4];
    __shared__ float sw[GK][GB + 4];
    pdl_enter(TR_GEMM_F32);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
    float acc[4][4] = {};
    const int lr = tid >> 2;            // 0..63: row of the tile this thread loads
    const int lk = (tid & 3) * 4;       // 0,4,8,12: first k of its four elements
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int am = m0 + lr, wn = n0 + lr;
            sa[lk + j][lr] = (am < M && k < K) ? A[(size_t)am * K + k] : 0.f;
            sw[lk + j][lr] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sa[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = sw[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * N + n] = acc[i][j] + (bias ? bias[n] : 0.f);
        }
    }
}

}  // namespace air

AIR_API int air_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                         cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return AIR_ERR_BAD_ARGUMENT;
    dim3 grid((N + air::GB - 1) / air::GB, (M + air::GB - 1) / air::GB);
    if (grid.y > 65535) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::gemm_f32_kernel, grid, 256, 0, stream, A, W, bias, C, M, N, K);
}

AIR_API int air_trace_set_gemm_f32(unsigned long long* buffer) { return air::set_trace_here(buffer); }
