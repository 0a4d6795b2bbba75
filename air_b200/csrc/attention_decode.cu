// Decode attention over the paged cache for bfloat16: one query token per request, grouped
// query heads, keys split over several blocks (split-KV) and merged by a second kernel.
//
// Decoding reads every key and value of the request once and does little arithmetic on them,
// so the kernel is built around the memory system: each warp streams its own 16-key tiles
// straight from global memory into registers with 16-byte loads and feeds them to the tensor
// cores (mma.sync m16n8k16, bf16 in, fp32 out) with the query heads of the group as the M
// dimension, so the G query heads that share a kv head share every byte that is loaded.
// Nothing is transposed by ldmatrix and no tile is shared between threads through shared memory:
//
//  * S = Q K^T: the k index of the MMA is the head dimension.  A dot product does not care in
//    which order its terms are added, so the k slots of an MMA are mapped to the head dimension
//    such that a thread's slots are 8 consecutive elements of a row of K (one 16-byte load)
//    and the same 8 elements of a row of Q.
//  * O = P V: the MMA's B operand wants, per register, the same column of two consecutive keys.
//    A thread loads 8 consecutive columns of the four keys it is responsible for and builds
//    those registers with one byte-permute each; the n index of the MMA is mapped to the head
//    dimension accordingly and mapped back when O is written.
//
// grid = (splits, kv_heads * head_blocks, tokens), 4 warps.  Block (s, ., t) takes the s-th share
// of the token's 16-key tiles; its warps take tiles round-robin, each with its own running
// maximum, sum and output (online softmax in 32-bit), merged through shared memory.  With one
// split the block writes the output; otherwise it writes (max, sum, unnormalised output) to
// scratch memory and `decode_combine_kernel` merges the splits.
//
// q, out: [T, H, D] bf16.  cache: [page, 2, K, P, D] bf16.  block_table [slots, max_blocks].
// token_seq[t]: slot (negative: padding, skipped).  A query at position p sees keys
// max(0, p - window + 1) .. p (window 0: all).
#include "common.cuh"
#include "mma.cuh"

namespace air {

constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = 3;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
                 : "memory");
}

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ token_seq, const int* __restrict__ positions,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int H, int K, int P, int window, float scale_log2) {
    constexpr int KC = D / 32;   // 32-element chunks of the head dimension (QK^T)
    constexpr int NT = D / 8;    // 8-column tiles of the output (PV)
    constexpr int NG = D / 64;   // 64-column groups
    extern __shared__ float smem[];
    float* sm_o = smem;                          // [warps][16][D]
    float* sm_m = smem + DEC_WARPS * 16 * D;     // [warps][16]
    float* sm_l = sm_m + DEC_WARPS * 16;         // [warps][16]

    pdl_enter(TR_ATT_DECODE);
    const int t = blockIdx.z;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int G = H / K;
    const int head_blocks = (G + 15) / 16;
    const int kvh = blockIdx.y / head_blocks, hb = blockIdx.y % head_blocks;
    const int split = blockIdx.x, splits = gridDim.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)slot * max_blocks;

    // this block's tiles
    const int tile0 = lo / 16, tile1 = pos / 16 + 1;
    const int per = (tile1 - tile0 + splits - 1) / splits;
    const int begin = tile0 + split * per, end = min(tile1, begin + per);

    // query fragments: rows g and g + 8 of the block of 16 heads
    const int r0 = hb * 16 + g, r1 = r0 + 8;
    uint4 qa[KC], qb[KC];
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        qa[c] = r0 < G ? ldg16(q + ((size_t)t * H + kvh * G + r0) * D + 32 * c + 8 * tq) : make_uint4(0, 0, 0, 0);
        qb[c] = r1 < G ? ldg16(q + ((size_t)t * H + kvh * G + r1) * D + 32 * c + 8 * tq) : make_uint4(0, 0, 0, 0);
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // Keys and values are fetched two tiles ahead with cp.async into a ring in shared memory in which
    // every thread has places of its own: it copies exactly the 16-byte pieces that it will later
    // load into its own registers, so the ring needs no barrier; it only extends the registers.
    constexpr int PIECES = 2 * KC + 4 * NG;
    uint4* ring = reinterpret_cast<uint4*>(smem);
    const size_t page_stride = (size_t)2 * K * P * D;
    const size_t v_offset = (size_t)K * P * D;
    const int my_tiles = begin + warp < end ? (end - begin - warp + DEC_WARPS - 1) / DEC_WARPS : 0;
    auto issue = [&](int i) {
        if (i < my_tiles) {
            const int kbase = (begin + warp + i * DEC_WARPS) * 16;
            const int page = bt[kbase / P];
            const __nv_bfloat16* kp = cache + (size_t)page * page_stride + ((size_t)kvh * P + (kbase % P)) * D;
            const __nv_bfloat16* vp = kp + v_offset;
            uint4* dst = ring + (size_t)(i % DEC_STAGES) * PIECES * (DEC_WARPS * 32) + threadIdx.x;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < KC; ++c)
                    cp_async16(dst + (j * KC + c) * (DEC_WARPS * 32), kp + (size_t)(8 * j + g) * D + 32 * c + 8 * tq);
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4)
#pragma unroll
                for (int n = 0; n < NG; ++n)
                    cp_async16(dst + (2 * KC + i4 * NG + n) * (DEC_WARPS * 32),
                               vp + (size_t)(2 * tq + (i4 & 1) + 8 * (i4 >> 1)) * D + 64 * n + 8 * g);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int i = 0; i < DEC_STAGES - 1; ++i) issue(i);
    for (int it = 0; it < my_tiles; ++it) {
        const int kbase = (begin + warp + it * DEC_WARPS) * 16;
        issue(it + DEC_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(DEC_STAGES - 1) : "memory");
        const uint4* src = ring + (size_t)(it % DEC_STAGES) * PIECES * (DEC_WARPS * 32) + threadIdx.x;
        // K: rows g and 8 + g of the tile; V: rows 2tq, 2tq+1, 8+2tq, 9+2tq
        uint4 kf[2][KC];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < KC; ++c) kf[j][c] = src[(j * KC + c) * (DEC_WARPS * 32)];
        uint4 vf[4][NG];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int n = 0; n < NG; ++n) vf[i][n] = src[(2 * KC + i * NG + n) * (DEC_WARPS * 32)];

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
        // mask and scale (scores in units of log2 e)
        float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kbase + 8 * j + 2 * tq + e;
                const bool ok = key >= lo && key <= pos;
                s[j][e] = ok ? s[j][e] * scale_log2 : -INFINITY;
                s[j][2 + e] = ok ? s[j][2 + e] * scale_log2 : -INFINITY;
                tm0 = fmaxf(tm0, s[j][e]);
                tm1 = fmaxf(tm1, s[j][2 + e]);
            }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float n0 = fmaxf(m0, tm0), n1 = fmaxf(m1, tm1);
        if (n0 == -INFINITY) continue;   // no visible key yet (same for both rows and all lanes)
        const float c0 = exp2f(m0 - n0), c1 = exp2f(m1 - n1);
        m0 = n0;
        m1 = n1;
        float p[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            p[j][0] = exp2f(s[j][0] - n0);
            p[j][1] = exp2f(s[j][1] - n0);
            p[j][2] = exp2f(s[j][2] - n1);
            p[j][3] = exp2f(s[j][3] - n1);
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
            const uint32_t a[4] = {vf[0][n].x, vf[0][n].y, vf[0][n].z, vf[0][n].w};   // key 2tq
            const uint32_t b[4] = {vf[1][n].x, vf[1][n].y, vf[1][n].z, vf[1][n].w};   // key 2tq + 1
            const uint32_t c[4] = {vf[2][n].x, vf[2][n].y, vf[2][n].z, vf[2][n].w};   // key 8 + 2tq
            const uint32_t d[4] = {vf[3][n].x, vf[3][n].y, vf[3][n].z, vf[3][n].w};   // key 9 + 2tq
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                mma_bf16_16816(o[8 * n + 2 * w], pa0, pa1, pa2, pa3, __byte_perm(a[w], b[w], 0x5410),
                               __byte_perm(c[w], d[w], 0x5410));
                mma_bf16_16816(o[8 * n + 2 * w + 1], pa0, pa1, pa2, pa3, __byte_perm(a[w], b[w], 0x7632),
                               __byte_perm(c[w], d[w], 0x7632));
            }
        }
    }
    // sums over the four threads of a row
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // merge the warps (the ring is done with: its memory is used again).
    // Output tile n, accumulator e holds column (n/8)*64 + 8*(2tq + (e&1)) + n%8.
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (tq == 0) {
        sm_m[warp * 16 + g] = m0;
        sm_m[warp * 16 + g + 8] = m1;
        sm_l[warp * 16 + g] = l0;
        sm_l[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = (n / 8) * 64 + 8 * (2 * tq + (e & 1)) + (n % 8);
            sm_o[(warp * 16 + g + 8 * (e >> 1)) * D + col] = o[n][e];
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * D; idx += blockDim.x) {
        const int r = idx / D, col = idx % D;
        if (hb * 16 + r >= G) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_m[w * 16 + r]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float wgt = sm_m[w * 16 + r] == -INFINITY ? 0.f : exp2f(sm_m[w * 16 + r] - mm);
            acc += sm_o[(w * 16 + r) * D + col] * wgt;
            ll += sm_l[w * 16 + r] * wgt;
        }
        const int h = kvh * G + hb * 16 + r;
        if (splits == 1) {
            out[((size_t)t * H + h) * D + col] = __float2bfloat16_rn(acc / ll);
        } else {
            const size_t pi = ((size_t)t * H + h) * splits + split;
            part_o[pi * D + col] = acc;
            if (col == 0) {
                part_ml[pi * 2] = mm;
                part_ml[pi * 2 + 1] = ll;
            }
        }
    }
}

// Merges the splits of one (token, head): out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// The kernel is a chain of latencies, so a thread asks for CHUNK splits' values at once (all of them, up
// to 32; and for the token's slot beside them: a padding token has its place in the buffers too) and
// folds them into a running maximum, sum and value, in the order of the splits.
template <int D, int CHUNK>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      const int* __restrict__ token_seq, __nv_bfloat16* __restrict__ out, int H,
                                      int splits) {
    pdl_enter(TR_ATT_COMBINE);
    const int t = blockIdx.y, h = blockIdx.x;
    const size_t base = ((size_t)t * H + h) * splits;
    const int slot = token_seq[t];
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
        float mm = -INFINITY, ll = 0.f, acc = 0.f;
        for (int s0 = 0; s0 < splits; s0 += CHUNK) {
            float m[CHUNK], l[CHUNK], o[CHUNK];
#pragma unroll
            for (int i = 0; i < CHUNK; ++i) {
                const bool in = s0 + i < splits;
                const float2 ml = in ? *reinterpret_cast<const float2*>(part_ml + (base + s0 + i) * 2)
                                     : make_float2(-INFINITY, 0.f);
                m[i] = ml.x;
                l[i] = ml.y;
                o[i] = in ? part_o[(base + s0 + i) * D + col] : 0.f;
            }
            float top = mm;
#pragma unroll
            for (int i = 0; i < CHUNK; ++i) top = fmaxf(top, m[i]);
            if (top == -INFINITY) continue;            // nothing seen yet
            const float keep = exp2f(mm - top);         // 0 while mm is -inf
            ll *= keep;
            acc *= keep;
#pragma unroll
            for (int i = 0; i < CHUNK; ++i) {
                if (m[i] == -INFINITY) continue;        // (its values are not looked at: they may be anything)
                const float w = exp2f(m[i] - top);
                ll += l[i] * w;
                acc += o[i] * w;
            }
            mm = top;
        }
        if (slot >= 0) out[((size_t)t * H + h) * D + col] = __float2bfloat16_rn(acc / ll);
    }
}

// The merge kernel with all of a thread's loads in one round where the splits are up to 32.
template <int D>
int launch_combine(const float* part_o, const float* part_ml, const int* token_seq, __nv_bfloat16* out, int T, int H,
                   int splits, cudaStream_t stream) {
    const int threads = D >= 128 ? 128 : 64;
    if (splits <= 8)
        return launch(decode_combine_kernel<D, 8>, dim3(H, T), threads, 0, stream, part_o, part_ml, token_seq, out, H,
                      splits);
    if (splits <= 16)
        return launch(decode_combine_kernel<D, 16>, dim3(H, T), threads, 0, stream, part_o, part_ml, token_seq, out, H,
                      splits);
    return launch(decode_combine_kernel<D, 32>, dim3(H, T), threads, 0, stream, part_o, part_ml, token_seq, out, H,
                  splits);
}

template <int D>
int launch_decode(const void* q, const void* cache, const int* block_table, int max_blocks, const int* token_seq,
                  const int* positions, void* out, float* part_o, float* part_ml, int T, int H, int K, int P,
                  int window, float scale, int splits, cudaStream_t stream) {
    const int G = H / K;
    const int head_blocks = (G + 15) / 16;
    const size_t merge = (size_t)(DEC_WARPS * 16 * D + 2 * DEC_WARPS * 16) * sizeof(float);
    const size_t ring = (size_t)DEC_STAGES * (2 * (D / 32) + 4 * (D / 64)) * DEC_WARPS * 32 * 16;
    const size_t smem = merge > ring ? merge : ring;
    auto kernel = decode_attention_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(splits, K * head_blocks, T);
    int rc = launch(kernel, grid, DEC_WARPS * 32, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache,
                    block_table, max_blocks, token_seq, positions, (__nv_bfloat16*)out, part_o, part_ml, H, K, P,
                    window, scale * 1.4426950408889634f);
    if (rc == 0 && splits > 1)
        rc = launch_combine<D>(part_o, part_ml, token_seq, (__nv_bfloat16*)out, T, H, splits, stream);
    return rc;
}

}  // namespace air

// Scratch: part_o needs T*H*splits*D floats and part_ml T*H*splits*2 floats when splits > 1.
AIR_API int air_decode_attention(const void* q, const void* cache, const int* block_table, int max_blocks,
                                 const int* token_seq, const int* positions, void* out, float* part_o,
                                 float* part_ml, int T, int H, int K, int D, int P, int window, float scale,
                                 int splits, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || H % K || P % 16 || splits < 1 || T > 65535 || (splits > 1 && (!part_o || !part_ml)))
        return AIR_ERR_BAD_ARGUMENT;
    switch (D) {
        case 64:
            return air::launch_decode<64>(q, cache, block_table, max_blocks, token_seq, positions, out, part_o, part_ml,
                                          T, H, K, P, window, scale, splits, stream);
        case 128:
            return air::launch_decode<128>(q, cache, block_table, max_blocks, token_seq, positions, out, part_o,
                                           part_ml, T, H, K, P, window, scale, splits, stream);
        case 256:
            return air::launch_decode<256>(q, cache, block_table, max_blocks, token_seq, positions, out, part_o,
                                           part_ml, T, H, K, P, window, scale, splits, stream);
        default:
            return AIR_ERR_BAD_ARGUMENT;
    }
}

// The merge of the splits alone (used by the kernels that produce the partial results elsewhere).
AIR_API int air_decode_combine(const float* part_o, const float* part_ml, const int* token_seq, void* out, int T,
                               int H, int D, int splits, cudaStream_t stream) {
    using namespace air;
    switch (D) {
        case 64: return launch_combine<64>(part_o, part_ml, token_seq, (__nv_bfloat16*)out, T, H, splits, stream);
        case 128: return launch_combine<128>(part_o, part_ml, token_seq, (__nv_bfloat16*)out, T, H, splits, stream);
        case 256: return launch_combine<256>(part_o, part_ml, token_seq, (__nv_bfloat16*)out, T, H, splits, stream);
        default: return AIR_ERR_BAD_ARGUMENT;
    }
}

// ---------------------------------------------------------------------------------------------
// air_decode_attention_static: the same attention for callers that must not allocate.
// Declared and described in no_alloc.h.
#include <mutex>

#include "no_alloc.h"

// The split-KV partial results live here instead of in memory that the caller allocates.  Every
// GPU that loads this library holds these AIR_STATIC_SCRATCH_FLOATS * 4 bytes until the process
// exits.  In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) float g_static_scratch[AIR_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// The device address of g_static_scratch on the current device, looked up once per device.
int static_scratch(float** address) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) return AIR_ERR_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_address[device] = static_cast<float*>(p);
    }
    *address = g_scratch_address[device];
    return 0;
}
}  // namespace

AIR_API long long air_decode_attention_static_capacity(void) { return AIR_STATIC_SCRATCH_FLOATS; }

AIR_API long long air_decode_attention_static_need(int T, int H, int D, int splits) {
    if (splits <= 1) return 0;
    return (long long)T * H * splits * (D + 2);
}

AIR_API const char* air_decode_attention_static_error(int code) {
    switch (code) {
        case 0: return "ok";
        case AIR_ERR_BAD_ARGUMENT: return "a size that the decode attention kernel does not take";
        case AIR_ERR_STATIC_SCRATCH: return "tokens * heads * splits * (head_dim + 2) exceeds the built-in scratch "
                                            "(air_decode_attention_static_capacity floats): use fewer splits or "
                                            "fewer tokens per call";
        default: return "a CUDA error (the code is a cudaError_t)";
    }
}

AIR_API int air_decode_attention_static(const void* q, const void* cache, const int* block_table, int max_blocks,
                                        const int* token_seq, const int* positions, void* out, int T, int H, int K,
                                        int D, int P, int window, float scale, int splits, cudaStream_t stream) {
    if (T <= 0) return 0;
    // sizes that the kernel does not take are a bad argument, whatever their scratch would be
    if (splits < 1 || H <= 0 || K <= 0 || H % K || P <= 0 || P % 16 || T > 65535 || (D != 64 && D != 128 && D != 256))
        return AIR_ERR_BAD_ARGUMENT;
    const long long need = air_decode_attention_static_need(T, H, D, splits);
    if (need > AIR_STATIC_SCRATCH_FLOATS) return AIR_ERR_STATIC_SCRATCH;
    float* scratch = nullptr;
    if (splits > 1) {
        const int rc = static_scratch(&scratch);
        if (rc != 0) return rc;
    }
    // Layout in the scratch: outputs [T*H*splits*D], then (max, sum) pairs [T*H*splits*2].  Nothing
    // has to be cleared: for every token that is not padding, the entries that the merge uses are written
    // by this call's first kernel (a padding token's entries are whatever an earlier call left; the merge
    // loads them and stores nothing).
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)T * H * splits * D : nullptr;
    return air_decode_attention(q, cache, block_table, max_blocks, token_seq, positions, out, part_o, part_ml, T, H,
                                K, D, P, window, scale, splits, stream);
}

AIR_API int air_trace_set_attention_decode(unsigned long long* buffer) { return air::set_trace_here(buffer); }
