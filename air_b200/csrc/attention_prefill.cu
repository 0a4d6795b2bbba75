// Causal attention over the paged cache for prompt portions in bfloat16 (any batch: several
// requests, portions of any length, decoded tokens among them).
//
// The host cuts the batch's tokens into tiles of up to 16 consecutive tokens of one request, in
// groups of 8 tiles that never straddle two requests (a group is filled up with empty tiles).  A
// block takes TT consecutive tiles of a group and Gh query heads of one kv head, TT * Gh <= 8: one
// warp per (tile, head), so that all its warps want the same keys.  A producer warp brings 64-key
// tiles of K and V from the pages into a ring of shared-memory stages with TMA (128-byte swizzle);
// the other warps wait on the stage's mbarrier, take their MMA operands from it with ldmatrix and
// compute 16 x 64 scores at a time with mma.sync m16n8k16 (bf16 in, fp32 out), softmax online in
// 32-bit.  A tile of keys is thus fetched once for up to 128 query rows.
//
// tiles [8n, 4] int32: (slot, index of the tile's first token in the batch, its position, rows);
// rows = 0 marks an empty tile.  q, out: [T, H, D] bf16.  cache: [page, 2, K, P, D] bf16.
// block_table [slots, max_blocks].  The query at position p sees keys max(0, p - window + 1) .. p.
// Every wait on an mbarrier is bounded (tma.cuh); on giving up the block flags *status = 6.
#include "common.cuh"
#include "mma.cuh"
#include "tma.cuh"

namespace air {

constexpr int PF_MAX_CONSUMERS = 8;
constexpr int PF_TILE = 64;      // keys per stage
constexpr int PF_STAGES = 3;
constexpr int PF_GROUP = 8;      // tiles of 16 tokens per group in the host's list

template <int D>
__global__ void __launch_bounds__((PF_MAX_CONSUMERS + 1) * 32)
prefill_attention_kernel(const __grid_constant__ CUtensorMap map_cache, const __nv_bfloat16* __restrict__ q,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tiles,
                         __nv_bfloat16* __restrict__ out, int H, int K, int P, int window, float scale_log2, int Gh,
                         int TT, int* status) {
    constexpr int SUB = D / 64;
    constexpr int SUB_BYTES = PF_TILE * 128;
    constexpr int STAGE_BYTES = 2 * SUB * SUB_BYTES;
    constexpr int KS = D / 16, NT = D / 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + PF_STAGES * STAGE_BYTES);
    uint64_t* empty = full + PF_STAGES;
    volatile int* abort_flag = (volatile int*)(empty + PF_STAGES);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int consumers = TT * Gh;
    if (threadIdx.x == 0) {
        for (int i = 0; i < PF_STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], consumers);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (P < PF_TILE || window > 0) {   // see attention_decode_tma.cu: rows that no copy fills must not hold NaN bits
        for (int i = threadIdx.x; i < PF_STAGES * STAGE_BYTES / 16; i += blockDim.x)
            reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();
    trace_point(TR_ATT_PREFILL);

    // the block's tiles: heavy ones (late in their request) first
    const int first_entry = (gridDim.x - 1 - blockIdx.x) * TT;
    int slot = -1, pos_first = 0, pos_last = -1;
    for (int i = 0; i < TT; ++i) {
        const int* e = tiles + 4 * (first_entry + i);
        if (e[3] > 0) {
            if (slot < 0) { slot = e[0]; pos_first = e[2]; }
            pos_last = e[2] + e[3] - 1;
        }
    }
    if (slot < 0) return;     // only empty tiles
    const int G = H / K;
    const int head_blocks = (G + Gh - 1) / Gh;
    const int kvh = blockIdx.y / head_blocks, hb = blockIdx.y % head_blocks;
    const int* bt = block_table + (size_t)slot * max_blocks;
    const int lo_block = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int tile0 = lo_block / PF_TILE, n_tiles = pos_last / PF_TILE + 1 - tile0;

    if (warp == consumers) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            const int box_rows = P < PF_TILE ? P : PF_TILE;
            const int boxes = PF_TILE / box_rows;
            for (int it = 0; it < n_tiles; ++it) {
                const int stage = it % PF_STAGES;
                if (it >= PF_STAGES && !mbar_wait(&empty[stage], ((it / PF_STAGES) - 1) & 1, abort_flag)) break;
                const int kbase = (tile0 + it) * PF_TILE;
                int valid = 0;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    valid += (first <= pos_last && first + box_rows - 1 >= lo_block) ? 1 : 0;
                }
                mbar_expect_tx(&full[stage], (uint32_t)(valid * box_rows * 128 * SUB * 2));
                uint8_t* dst = smem + stage * STAGE_BYTES;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    if (!(first <= pos_last && first + box_rows - 1 >= lo_block)) continue;
                    const int page = bt[first / P];
                    const int row_k = ((page * 2) * K + kvh) * P + first % P;
                    const int row_v = row_k + K * P;
#pragma unroll
                    for (int s = 0; s < SUB; ++s) {
                        tma_load_2d(dst + s * SUB_BYTES + b * box_rows * 128, &map_cache, 64 * s, row_k, &full[stage]);
                        tma_load_2d(dst + (SUB + s) * SUB_BYTES + b * box_rows * 128, &map_cache, 64 * s, row_v,
                                    &full[stage]);
                    }
                }
            }
        }
    } else if (warp < consumers) {
        // ------------------------------------------------------------ consumers: one (tile, head) each
        const int* e = tiles + 4 * (first_entry + warp / Gh);
        const int tok0 = e[1], pos0 = e[2], rows = e[3];
        const int hg = hb * Gh + warp % Gh;
        const bool active = rows > 0 && hg < G;
        const int h = kvh * G + hg;
        const int g = lane >> 2, tq = lane & 3;
        const int mat = lane >> 3, mrow = lane & 7;
        const int last = pos0 + rows - 1;
        const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
        const int p0 = pos0 + g, p1 = pos0 + g + 8;
        uint32_t qa[KS][4];
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            const __nv_bfloat16* q0 = q + ((size_t)(tok0 + g) * H + h) * D + 16 * kk + 2 * tq;
            const __nv_bfloat16* q1 = q + ((size_t)(tok0 + g + 8) * H + h) * D + 16 * kk + 2 * tq;
            const bool a0 = active && g < rows, a1 = active && g + 8 < rows;
            qa[kk][0] = a0 ? __ldg(reinterpret_cast<const uint32_t*>(q0)) : 0u;
            qa[kk][1] = a1 ? __ldg(reinterpret_cast<const uint32_t*>(q1)) : 0u;
            qa[kk][2] = a0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + 8)) : 0u;
            qa[kk][3] = a1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + 8)) : 0u;
        }
        float o[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        for (int it = 0; it < n_tiles; ++it) {
            const int stage = it % PF_STAGES;
            if (!mbar_wait(&full[stage], (it / PF_STAGES) & 1, abort_flag)) break;
            const int kbase = (tile0 + it) * PF_TILE;
            if (active && kbase <= last && kbase + PF_TILE - 1 >= lo) {
                const uint32_t kt = smem_u32(smem + stage * STAGE_BYTES);
                const uint32_t vt = kt + SUB * SUB_BYTES;
                float s[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        uint32_t b[4];
                        ldmatrix_x4(b, swizzled(kt + (kk / 4) * SUB_BYTES, 16 * np + (mat >> 1) * 8 + mrow,
                                                2 * (kk % 4) + (mat & 1)));
                        mma_bf16_16816(s[2 * np], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b[0], b[1]);
                        mma_bf16_16816(s[2 * np + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b[2], b[3]);
                    }
                }
                const bool inner = kbase + PF_TILE - 1 <= pos0 && (window <= 0 || kbase > last - window);
                float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int ee = 0; ee < 2; ++ee) {
                        const int key = kbase + 8 * j + 2 * tq + ee;
                        const bool ok0 = inner || (key <= p0 && (window <= 0 || key > p0 - window));
                        const bool ok1 = inner || (key <= p1 && (window <= 0 || key > p1 - window));
                        s[j][ee] = ok0 ? s[j][ee] * scale_log2 : -INFINITY;
                        s[j][2 + ee] = ok1 ? s[j][2 + ee] * scale_log2 : -INFINITY;
                        tm0 = fmaxf(tm0, s[j][ee]);
                        tm1 = fmaxf(tm1, s[j][2 + ee]);
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
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    s[j][0] = exp2f(s[j][0] - b0);
                    s[j][1] = exp2f(s[j][1] - b0);
                    s[j][2] = exp2f(s[j][2] - b1);
                    s[j][3] = exp2f(s[j][3] - b1);
                    sum0 += s[j][0] + s[j][1];
                    sum1 += s[j][2] + s[j][3];
                }
                l0 = l0 * c0 + sum0;
                l1 = l1 * c1 + sum1;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    o[n][0] *= c0;
                    o[n][1] *= c0;
                    o[n][2] *= c1;
                    o[n][3] *= c1;
                }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint32_t pa0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]), pa1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
                    const uint32_t pa2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
                    const uint32_t pa3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
                    for (int n = 0; n < NT; n += 2) {
                        uint32_t b[4];
                        const int chunk = n + (mat >> 1);
                        ldmatrix_x4_trans(b, swizzled(vt + (chunk / 8) * SUB_BYTES, 16 * ks + (mat & 1) * 8 + mrow,
                                                      chunk % 8));
                        mma_bf16_16816(o[n], pa0, pa1, pa2, pa3, b[0], b[1]);
                        mma_bf16_16816(o[n + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
        }
        if (active && !*abort_flag) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
            __nv_bfloat16* d0 = out + ((size_t)(tok0 + g) * H + h) * D + 2 * tq;
            __nv_bfloat16* d1 = out + ((size_t)(tok0 + g + 8) * H + h) * D + 2 * tq;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                if (g < rows) *reinterpret_cast<uint32_t*>(d0 + 8 * n) = pack_bf16(o[n][0] * i0, o[n][1] * i0);
                if (g + 8 < rows) *reinterpret_cast<uint32_t*>(d1 + 8 * n) = pack_bf16(o[n][2] * i1, o[n][3] * i1);
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 32; ++i) __nanosleep(2000);
        if (threadIdx.x == 0 && status) atomicExch(status, 6);
    }
}

template <int D>
int launch_prefill(const CUtensorMap& map, const void* q, const int* block_table, int max_blocks, const int* tiles,
                   int n_tiles, void* out, int H, int K, int P, int window, float scale, int* status,
                   cudaStream_t stream) {
    const int G = H / K;
    const int Gh = G < PF_MAX_CONSUMERS ? G : PF_MAX_CONSUMERS;
    int TT = PF_MAX_CONSUMERS / Gh;                      // tiles per block: 1, 2, 4 or 8
    TT = TT >= 8 ? 8 : (TT >= 4 ? 4 : (TT >= 2 ? 2 : 1));
    const int head_blocks = (G + Gh - 1) / Gh;
    const size_t smem = 1024 + (size_t)PF_STAGES * 2 * (D / 64) * PF_TILE * 128 + 128;
    auto kernel = prefill_attention_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch(kernel, dim3(n_tiles / TT, K * head_blocks), (TT * Gh + 1) * 32, smem, stream, map,
                  (const __nv_bfloat16*)q, block_table, max_blocks, tiles, (__nv_bfloat16*)out, H, K, P, window,
                  scale * 1.4426950408889634f, Gh, TT, status);
}

}  // namespace air

// tiles: n_tiles entries, a multiple of 8, in groups of 8 that each belong to one request.
AIR_API int air_prefill_attention(const void* q, const void* cache, long long pages, const int* block_table,
                                  int max_blocks, const int* tiles, int n_tiles, void* out, int H, int K, int D, int P,
                                  int window, float scale, int* status, cudaStream_t stream) {
    using namespace air;
    if (n_tiles <= 0) return 0;
    if (H <= 0 || K <= 0 || H % K || P % 16 || (P < 64 ? 64 % P : P % 64) || n_tiles % PF_GROUP || ((uintptr_t)cache & 15) ||
        K * ((H / K + 7) / 8) > 65535)
        return AIR_ERR_BAD_ARGUMENT;
    CUtensorMap map;
    const int map_rc = tensor_map_2d(&map, cache, pages * 2 * K * P, D, P < PF_TILE ? P : PF_TILE);
    if (map_rc) return map_rc;
    switch (D) {
        case 64:
            return launch_prefill<64>(map, q, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window, scale,
                                      status, stream);
        case 128:
            return launch_prefill<128>(map, q, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window, scale,
                                       status, stream);
        case 256:
            return launch_prefill<256>(map, q, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window, scale,
                                       status, stream);
        default:
            return AIR_ERR_BAD_ARGUMENT;
    }
}

AIR_API int air_trace_set_attention_prefill(unsigned long long* buffer) { return air::set_trace_here(buffer); }
