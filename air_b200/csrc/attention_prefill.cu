// Causal attention over the paged cache for prompt portions in bfloat16 (any batch: several
// requests, portions of any length, decoded tokens among them).
//
// The batch's tokens are cut on the host into tiles of up to 16 consecutive tokens of one
// request.  A block takes one tile and one kv head; each of its warps takes one query head of
// the group and computes the 16 x keys score matrix of that head with the tensor cores
// (mma.sync m16n8k16, bf16 in, fp32 out), 16 keys at a time, with the online softmax in 32-bit.
// Keys and values come straight from the pages into registers, with the same mapping of MMA
// slots to the head dimension as the decode kernel (attention_decode.cu): a thread's operands
// are 16-byte pieces of rows of K and V.  The warps of a block walk the same keys at the same
// time, so the group's heads share the loaded lines in L1: the cache is read once per group.
//
// tiles [n, 4] int32: (slot, index of the tile's first token in the batch, its position, rows).
// q, out: [T, H, D] bf16.  cache: [page, 2, K, P, D] bf16.  block_table [slots, max_blocks].
// The query at position p sees keys max(0, p - window + 1) .. p (window 0: all keys).
#include "common.cuh"
#include "mma.cuh"

namespace air {

constexpr int PRE_MAX_WARPS = 8;

template <int D>
__global__ void __launch_bounds__(PRE_MAX_WARPS * 32)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tiles,
                         __nv_bfloat16* __restrict__ out, int H, int K, int P, int window, float scale_log2) {
    constexpr int KC = D / 32, NT = D / 8, NG = D / 64;
    extern __shared__ float smem[];   // [warps][16][D + 4]: the output tile of each warp
    pdl_enter(TR_ATT_PREFILL);
    const int G = H / K;
    const int head_blocks = (G + PRE_MAX_WARPS - 1) / PRE_MAX_WARPS;
    const int kvh = blockIdx.y / head_blocks, hb = blockIdx.y % head_blocks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hg = hb * PRE_MAX_WARPS + warp;        // head within the group
    if (hg >= G) return;
    const int h = kvh * G + hg;
    const int g = lane >> 2, tq = lane & 3;
    const int* tile = tiles + 4 * blockIdx.x;
    const int slot = tile[0], tok0 = tile[1], pos0 = tile[2], rows = tile[3];
    const int* bt = block_table + (size_t)slot * max_blocks;
    const int last = pos0 + rows - 1;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int p0 = pos0 + g, p1 = pos0 + g + 8;     // positions of this thread's two rows

    uint4 qa[KC], qb[KC];
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        qa[c] = g < rows ? ldg16(q + ((size_t)(tok0 + g) * H + h) * D + 32 * c + 8 * tq) : make_uint4(0, 0, 0, 0);
        qb[c] = g + 8 < rows ? ldg16(q + ((size_t)(tok0 + g + 8) * H + h) * D + 32 * c + 8 * tq)
                             : make_uint4(0, 0, 0, 0);
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const size_t page_stride = (size_t)2 * K * P * D;
    const size_t v_offset = (size_t)K * P * D;
    for (int kt = lo / 16; kt * 16 <= last; ++kt) {
        const int kbase = kt * 16;
        const int page = bt[kbase / P];
        const __nv_bfloat16* kp = cache + (size_t)page * page_stride + ((size_t)kvh * P + (kbase % P)) * D;
        const __nv_bfloat16* vp = kp + v_offset;
        uint4 kf[2][KC];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < KC; ++c) kf[j][c] = ldg16(kp + (size_t)(8 * j + g) * D + 32 * c + 8 * tq);
        uint4 vf[4][NG];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int n = 0; n < NG; ++n)
                vf[i][n] = ldg16(vp + (size_t)(2 * tq + (i & 1) + 8 * (i >> 1)) * D + 64 * n + 8 * g);

        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                mma_bf16_16816(s[j], qa[c].x, qb[c].x, qa[c].y, qb[c].y, kf[j][c].x, kf[j][c].y);
                mma_bf16_16816(s[j], qa[c].z, qb[c].z, qa[c].w, qb[c].w, kf[j][c].z, kf[j][c].w);
            }
        }
        const bool inner = kbase + 15 <= pos0 && (window <= 0 || kbase > last - window);  // no mask needed
        float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kbase + 8 * j + 2 * tq + e;
                const bool ok0 = inner || (key <= p0 && (window <= 0 || key > p0 - window));
                const bool ok1 = inner || (key <= p1 && (window <= 0 || key > p1 - window));
                s[j][e] = ok0 ? s[j][e] * scale_log2 : -INFINITY;
                s[j][2 + e] = ok1 ? s[j][2 + e] * scale_log2 : -INFINITY;
                tm0 = fmaxf(tm0, s[j][e]);
                tm1 = fmaxf(tm1, s[j][2 + e]);
            }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float n0 = fmaxf(m0, tm0), n1 = fmaxf(m1, tm1);
        // a row that has seen no key yet keeps maximum -inf: subtract 0 instead, all its p are 0
        const float b0 = n0 == -INFINITY ? 0.f : n0, b1 = n1 == -INFINITY ? 0.f : n1;
        const float c0 = exp2f(m0 - b0), c1 = exp2f(m1 - b1);
        m0 = n0;
        m1 = n1;
        float p[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            p[j][0] = exp2f(s[j][0] - b0);
            p[j][1] = exp2f(s[j][1] - b0);
            p[j][2] = exp2f(s[j][2] - b1);
            p[j][3] = exp2f(s[j][3] - b1);
        }
        l0 = l0 * c0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
        l1 = l1 * c1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
        const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]), pa1 = pack_bf16(p[0][2], p[0][3]);
        const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]), pa3 = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o[n][0] *= c0;
            o[n][1] *= c0;
            o[n][2] *= c1;
            o[n][3] *= c1;
        }
#pragma unroll
        for (int n = 0; n < NG; ++n) {
            const uint32_t a[4] = {vf[0][n].x, vf[0][n].y, vf[0][n].z, vf[0][n].w};
            const uint32_t b[4] = {vf[1][n].x, vf[1][n].y, vf[1][n].z, vf[1][n].w};
            const uint32_t c[4] = {vf[2][n].x, vf[2][n].y, vf[2][n].z, vf[2][n].w};
            const uint32_t d[4] = {vf[3][n].x, vf[3][n].y, vf[3][n].z, vf[3][n].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                mma_bf16_16816(o[8 * n + 2 * w], pa0, pa1, pa2, pa3, __byte_perm(a[w], b[w], 0x5410),
                               __byte_perm(c[w], d[w], 0x5410));
                mma_bf16_16816(o[8 * n + 2 * w + 1], pa0, pa1, pa2, pa3, __byte_perm(a[w], b[w], 0x7632),
                               __byte_perm(c[w], d[w], 0x7632));
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;

    // through shared memory, so that rows are written in whole 16-byte pieces
    float* so = smem + (size_t)warp * 16 * (D + 4);
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = (n / 8) * 64 + 8 * (2 * tq + (e & 1)) + (n % 8);
            so[(g + 8 * (e >> 1)) * (D + 4) + col] = o[n][e] * ((e >> 1) ? i1 : i0);
        }
    __syncwarp();
    for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
        const int r = idx / (D / 8), c8 = (idx % (D / 8)) * 8;
        if (r >= rows) continue;
        const float* src = so + r * (D + 4) + c8;
        uint4 v;
        v.x = pack_bf16(src[0], src[1]);
        v.y = pack_bf16(src[2], src[3]);
        v.z = pack_bf16(src[4], src[5]);
        v.w = pack_bf16(src[6], src[7]);
        *reinterpret_cast<uint4*>(out + ((size_t)(tok0 + r) * H + h) * D + c8) = v;
    }
}

template <int D>
int launch_prefill(const void* q, const void* cache, const int* block_table, int max_blocks, const int* tiles,
                   int n_tiles, void* out, int H, int K, int P, int window, float scale, cudaStream_t stream) {
    const int G = H / K;
    const int warps = G < PRE_MAX_WARPS ? G : PRE_MAX_WARPS;
    const int head_blocks = (G + PRE_MAX_WARPS - 1) / PRE_MAX_WARPS;
    const size_t smem = (size_t)warps * 16 * (D + 4) * sizeof(float);
    auto kernel = prefill_attention_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_tiles, K * head_blocks);
    return launch(kernel, grid, warps * 32, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache,
                  block_table, max_blocks, tiles, (__nv_bfloat16*)out, H, K, P, window, scale * 1.4426950408889634f);
}

}  // namespace air

AIR_API int air_prefill_attention(const void* q, const void* cache, const int* block_table, int max_blocks,
                                  const int* tiles, int n_tiles, void* out, int H, int K, int D, int P, int window,
                                  float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (H <= 0 || K <= 0 || H % K || P % 16 || K * ((H / K + 7) / 8) > 65535) return AIR_ERR_BAD_ARGUMENT;
    switch (D) {
        case 64:
            return air::launch_prefill<64>(q, cache, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window,
                                           scale, stream);
        case 128:
            return air::launch_prefill<128>(q, cache, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window,
                                            scale, stream);
        case 256:
            return air::launch_prefill<256>(q, cache, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window,
                                            scale, stream);
        default:
            return AIR_ERR_BAD_ARGUMENT;
    }
}

AIR_API int air_trace_set_attention_prefill(unsigned long long* buffer) { return air::set_trace_here(buffer); }
