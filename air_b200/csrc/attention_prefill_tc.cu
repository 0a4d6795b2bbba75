// Causal attention over the paged cache for prompt portions in bfloat16 on the fifth-generation
// tensor cores: both products of attention are tcgen05.mma with operands in shared memory and
// accumulators in tensor memory.
//
// A block takes one group of the host's tile list (up to 128 consecutive tokens of one request,
// see attention_prefill.cu) and one query head; its 128 query rows are the M dimension.
//   warp 0    TMA: the Q tile once, then 64-key tiles of K and V from the pages into a ring;
//   warp 1    issues S = Q K^T (M 128, N 64, k = head dim) into one of two S accumulators and,
//             one tile behind, O += P V (M 128, N = head dim, k = 64 keys; V is the MN-major operand,
//             read as it lies in the page);
//   warps 2-5 softmax: thread r owns query row r.  It reads its row of S from tensor memory, masks,
//             keeps a reference maximum and the sum (32-bit), rescales its row of O in tensor memory
//             when the maximum has moved far, and writes its row of P as bfloat16 into shared memory in
//             the swizzled K-major layout that the second product reads.  No value crosses threads.
// S(j+1) is multiplied while softmax works on S(j); P V (j) follows as soon as P(j) is written.
//
// tiles, q, out, cache, block_table, window as in attention_prefill.cu.  Head size 64 or 128.
// Every wait on an mbarrier is bounded (tma.cuh); on giving up the block flags *status = 7.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace air {

constexpr int AT_BM = 128;      // query rows per block
constexpr int AT_BN = 64;       // keys per step
constexpr int AT_STAGES = 3;
constexpr int AT_THREADS = 192;
constexpr int AT_GROUP = 8;     // 16-token tiles per group of the host's list

// 2^x by the special-function unit in one instruction (2^-inf = 0; relative error about 2^-22,
// far below what rounding the probabilities to bfloat16 adds).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_cache,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tiles,
                            __nv_bfloat16* __restrict__ out, int H, int K, int P, int window, float scale_log2,
                            int* status) {
    constexpr int SUB = D / 64;
    constexpr int Q_BYTES = SUB * AT_BM * 128;
    constexpr int KV_SUB = AT_BN * 128;                    // 8 KB: one 64-column sub-tile of 64 keys
    constexpr int STAGE_BYTES = 2 * SUB * KV_SUB;
    constexpr int P_BYTES = AT_BM * 128;                   // [128 rows][64 keys] bf16
    constexpr uint32_t TMEM_COLS = 256;                    // S0 | S1 | O
    constexpr uint32_t O_COL = 2 * AT_BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sq = smem;
    uint8_t* skv = sq + Q_BYTES;
    uint8_t* sp = skv + AT_STAGES * STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(sp + 2 * P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;
    uint64_t* kv_empty = kv_full + AT_STAGES;
    uint64_t* s_full = kv_empty + AT_STAGES;     // [2]
    uint64_t* s_free = s_full + 2;               // [2]
    uint64_t* p_ready = s_free + 2;              // [2]
    uint64_t* pv_done = p_ready + 2;             // [2]: tile j completes pv_done[j & 1]
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < AT_STAGES; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_free[i], 4);
            mbar_init(&p_ready[i], 4);
        }
        mbar_init(&pv_done[0], 1);
        mbar_init(&pv_done[1], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    if (P < AT_BN || window > 0) {   // rows that no copy fills must not hold NaN bits (see attention_decode_tma.cu)
        for (int i = threadIdx.x; i < AT_STAGES * STAGE_BYTES / 16; i += AT_THREADS)
            reinterpret_cast<uint4*>(skv)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();
    trace_point(TR_ATT_PREFILL);

    // the block's group of tiles (heavy groups first) and head
    const int* grp = tiles + 4 * AT_GROUP * (gridDim.x - 1 - blockIdx.x);
    int count = 0;
    for (int i = 0; i < AT_GROUP; ++i) count += grp[4 * i + 3];
    const int slot = grp[0], tok0 = grp[1], pos0 = grp[2];
    const int h = blockIdx.y;
    const int kvh = (int)(((long long)h * K) / H);
    const int* bt = block_table + (size_t)slot * max_blocks;
    const int pos_last = pos0 + count - 1;
    const int lo_block = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int tile0 = lo_block / AT_BN;
    const int n_tiles = count > 0 ? pos_last / AT_BN + 1 - tile0 : 0;

    if (warp == 0) {
        if (lane == 0 && n_tiles > 0) {
            // ------------------------------------------------ producer
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int s = 0; s < SUB; ++s) tma_load_2d(sq + s * AT_BM * 128, &map_q, h * D + 64 * s, tok0, q_full);
            const int box_rows = P < AT_BN ? P : AT_BN;
            const int boxes = AT_BN / box_rows;
            for (int it = 0; it < n_tiles; ++it) {
                const int stage = it % AT_STAGES;
                if (it >= AT_STAGES && !mbar_wait(&kv_empty[stage], ((it / AT_STAGES) - 1) & 1, abort_flag)) break;
                const int kbase = (tile0 + it) * AT_BN;
                int valid = 0;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    valid += (first <= pos_last && first + box_rows - 1 >= lo_block) ? 1 : 0;
                }
                mbar_expect_tx(&kv_full[stage], (uint32_t)(valid * box_rows * 128 * SUB * 2));
                uint8_t* dst = skv + stage * STAGE_BYTES;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    if (!(first <= pos_last && first + box_rows - 1 >= lo_block)) continue;
                    const int page = bt[first / P];
                    const int row_k = ((page * 2) * K + kvh) * P + first % P;
                    const int row_v = row_k + K * P;
#pragma unroll
                    for (int s = 0; s < SUB; ++s) {
                        tma_load_2d(dst + s * KV_SUB + b * box_rows * 128, &map_cache, 64 * s, row_k, &kv_full[stage]);
                        tma_load_2d(dst + (SUB + s) * KV_SUB + b * box_rows * 128, &map_cache, 64 * s, row_v,
                                    &kv_full[stage]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_tiles > 0) {
            // ------------------------------------------------ MMA issuer
            constexpr uint32_t idesc_qk = umma_idesc(AT_BM, AT_BN);
            constexpr uint32_t idesc_pv = umma_idesc(AT_BM, D, true);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            tc_fence_after();
            for (int it = 0; it <= n_tiles && ok; ++it) {
                if (it < n_tiles) {
                    // S(it) = Q K(it)^T into S[it & 1]
                    const int stage = it % AT_STAGES, b = it & 1;
                    ok = mbar_wait(&kv_full[stage], (it / AT_STAGES) & 1, abort_flag);
                    if (ok && it >= 2) ok = mbar_wait(&s_free[b], ((it >> 1) - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t kaddr = smem_u32(skv + stage * STAGE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk)
                        umma_bf16(tmem_base + b * AT_BN, umma_desc(smem_u32(sq) + (kk / 4) * AT_BM * 128) + 2 * (kk % 4),
                                  umma_desc(kaddr + (kk / 4) * KV_SUB) + 2 * (kk % 4), idesc_qk, kk > 0 ? 1u : 0u);
                    umma_commit(&s_full[b]);
                }
                if (it >= 1) {
                    // O += P(it-1) V(it-1)
                    const int j = it - 1, stage = j % AT_STAGES, b = j & 1;
                    ok = mbar_wait(&p_ready[b], (j >> 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t vaddr = smem_u32(skv + stage * STAGE_BYTES + SUB * KV_SUB);
                    const uint32_t paddr = smem_u32(sp + b * P_BYTES);
#pragma unroll
                    for (int ks = 0; ks < AT_BN / 16; ++ks)
                        umma_bf16(tmem_base + O_COL, umma_desc(paddr) + 2 * ks, umma_desc_mn(vaddr + ks * 16 * 128, KV_SUB),
                                  idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&kv_empty[stage]);
                    umma_commit(&pv_done[b]);
                }
            }
        }
    } else if (n_tiles > 0) {
        // ---------------------------------------------------- softmax: one thread per query row
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int pos = pos0 + r;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_tiles && ok; ++it) {
            const int b = it & 1;
            ok = mbar_wait(&s_full[b], (it >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[2][32];
            tmem_ld32(tmem_base + lane_addr + b * AT_BN, sv[0]);
            tmem_ld32(tmem_base + lane_addr + b * AT_BN + 32, sv[1]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[b]);
            const int kbase = (tile0 + it) * AT_BN;
            // Scores stay as the product left them; the scale goes into the exponent's multiply-add.
            // Only tiles on the diagonal or at a window's edge need the mask (the same for the warp).
            const int warp_first = pos0 + quarter * 32;
            const bool full_tile = kbase + AT_BN - 1 <= warp_first && (window <= 0 || kbase > warp_first + 31 - window);
            float mx = -INFINITY;
            if (full_tile) {
#pragma unroll
                for (int c = 0; c < AT_BN; ++c) mx = fmaxf(mx, __uint_as_float(sv[c >> 5][c & 31]));
            } else {
#pragma unroll
                for (int c = 0; c < AT_BN; ++c) {
                    const int key = kbase + c;
                    const bool vis = key <= pos && (window <= 0 || key > pos - window);
                    const float x = vis ? __uint_as_float(sv[c >> 5][c & 31]) : -INFINITY;
                    sv[c >> 5][c & 31] = __float_as_uint(x);
                    mx = fmaxf(mx, x);
                }
            }
            mx *= scale_log2;    // the scale is positive: the maximum of the scaled scores
            // The reference maximum m of the row moves only when the tile's maximum exceeds it by more
            // than 2^8 (or the row had seen no key): probabilities up to 256 are harmless in bfloat16 and
            // in the 32-bit sums, and a row of O that is not rescaled does not have to wait for the
            // product that is still writing it.
            const bool move = mx > m + 8.f;
            const float m_new = move ? mx : m;
            const float base = m_new == -INFINITY ? 0.f : m_new;   // a row that sees no key yet
            const float corr = move ? fast_exp2(m - base) : 1.f;
            m = m_new;
            float sum = 0.f;
            uint32_t pk[AT_BN / 2];
#pragma unroll
            for (int c = 0; c < AT_BN; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), scale_log2, -base));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sv[(c + 1) >> 5][(c + 1) & 31]), scale_log2, -base));
                sum += p0 + p1;
                const __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&v);
            }
            l = l * corr + sum;
            // P[b] was read by the product of tile it-2: that one must have completed.  (Two barriers
            // take turns, so that the one waited for is always the latest that can have completed:
            // a wait by parity cannot tell a phase from the one two later.)
            if (it >= 2) {
                ok = mbar_wait(&pv_done[b], ((it >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
            }
            if (it >= 1 && __any_sync(0xffffffffu, move)) {
                // O must be rescaled: every product issued so far (up to tile it-1) has to be complete
                ok = mbar_wait(&pv_done[b ^ 1], ((it - 1) >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_base + lane_addr + O_COL + c, ov);
#pragma unroll
                    for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * corr);
                    tmem_st32(tmem_base + lane_addr + O_COL + c, ov);
                }
            }
            // P(it): this row's 64 probabilities, 8 chunks of 16 bytes at their swizzled places
            uint8_t* prow = sp + b * P_BYTES + r * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) =
                    make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        if (ok && n_tiles >= 2) ok = mbar_wait(&pv_done[n_tiles & 1], ((n_tiles - 2) >> 1) & 1, abort_flag);
        if (ok) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag);
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + ((size_t)(tok0 + r) * H + h) * D;
#pragma unroll
            for (int c = 0; c < D; c += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_base + lane_addr + O_COL + c, ov);
                if (r < count) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        float y[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) y[k] = __uint_as_float(ov[e + k]) * inv;
                        store4(dst + c + e, *(const float(*)[4])&y[0]);
                        store4(dst + c + e + 4, *(const float(*)[4])&y[4]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 32; ++i) __nanosleep(2000);
        if (threadIdx.x == 0 && status) atomicExch(status, 7);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

static int make_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiled enc = encode_tiled();
    if (!enc) return AIR_ERR_BAD_ARGUMENT;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 200000 + (int)r;
}

template <int D>
int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mc, const int* block_table, int max_blocks,
                      const int* tiles, int n_tiles, void* out, int H, int K, int P, int window, float scale, int* status,
                      cudaStream_t stream) {
    const size_t smem = 1024 + (size_t)(D / 64) * AT_BM * 128 + (size_t)AT_STAGES * 2 * (D / 64) * AT_BN * 128 +
                        2 * AT_BM * 128 + 256;
    auto kernel = prefill_attention_tc_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch(kernel, dim3(n_tiles / AT_GROUP, H), AT_THREADS, smem, stream, mq, mc, block_table, max_blocks, tiles,
                  (__nv_bfloat16*)out, H, K, P, window, scale * 1.4426950408889634f, status);
}

}  // namespace air

// q [T, H, D] bf16.  tiles: n_tiles entries in groups of 8 per request.  Head size 64 or 128.
AIR_API int air_prefill_attention_tc(const void* q, int T, const void* cache, long long pages, const int* block_table,
                                     int max_blocks, const int* tiles, int n_tiles, void* out, int H, int K, int D,
                                     int P, int window, float scale, int* status, cudaStream_t stream) {
    using namespace air;
    if (n_tiles <= 0) return 0;
    if (H <= 0 || K <= 0 || H % K || P % 16 || (P < 64 && 64 % P) || n_tiles % AT_GROUP || H > 65535 ||
        ((uintptr_t)cache & 15) || ((uintptr_t)q & 15) || (D != 64 && D != 128))
        return AIR_ERR_BAD_ARGUMENT;
    CUtensorMap mq, mc;
    int rc = make_map_2d(&mq, q, T, (long long)H * D, AT_BM);
    if (rc) return rc;
    rc = make_map_2d(&mc, cache, pages * 2 * K * P, D, P < AT_BN ? P : AT_BN);
    if (rc) return rc;
    if (D == 64)
        return launch_prefill_tc<64>(mq, mc, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window, scale, status,
                                     stream);
    return launch_prefill_tc<128>(mq, mc, block_table, max_blocks, tiles, n_tiles, out, H, K, P, window, scale, status,
                                  stream);
}

AIR_API int air_trace_set_attention_prefill_tc(unsigned long long* buffer) { return air::set_trace_here(buffer); }
