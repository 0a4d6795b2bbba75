// Causal attention over the paged cache for prompt portions in bfloat16 on the fifth-generation
// tensor cores: both products of attention are tcgen05.mma with accumulators in tensor memory.
//
// A block takes two consecutive groups of the host's tile list (two row tiles of up to 128
// consecutive tokens of one request, see attention_prefill.cu) and one query head.  The two row
// tiles share one stream of 64-key tiles of K and V, so a key tile is fetched once for 256 queries.
//   warp 0      TMA: the Q tiles once, then the key tiles from the pages into a ring;
//   warps 1, 2  one issuer per row tile: S = Q K^T (M 128, N 64, k = head dim) into one of the row
//               tile's two S accumulators and, one key tile behind, O += P V (M 128, N = head dim,
//               k = 64 keys; P is the A operand in tensor memory, V the MN-major B operand, read as
//               it lies in the page).  tcgen05.mma is all but synchronous for its issuer (a second
//               instruction waits until the first has started), so whatever an issuer does between
//               two products leaves the tensor cores idle: with two issuers one's waits are the
//               other's work.
//   warps 4-7, 8-11  softmax of the two row tiles: thread r owns query row r.  It reads its row of S
//               from tensor memory, masks, keeps a reference maximum and the sum (32-bit), rescales
//               its row of O in tensor memory when the maximum has moved far, and writes its row of P
//               as bfloat16 pairs over the scores it came from.  No value crosses threads.  A warp's
//               ex2 takes eight cycles on the special-function unit, so part of the exponentials are
//               computed on the multiply-add pipe instead (exp2_fma).
// S(j+1) is multiplied while softmax works on S(j); P V (j) follows as soon as P(j) is written.
// Under the causal mask the second row tile takes two more key tiles than the first; with a
// window it also starts later.  A row tile's issuer hands back the stages it does not take.
//
// The grid is (heads, pairs) with the last pair of the list first: blocks are handed out in the order of
// blockIdx.x, then blockIdx.y, so all heads of the heaviest pair of a prompt start first.
//
// With a list of segments the grid is that list instead: block i takes segments[i] = (pair, head, first key tile
// of the pair's stream, key tiles, slot).  The host cuts long streams so when whole (pair, head) items would leave
// SMs idle (a short portion on top of thousands of tokens: few items, each over the whole context).  A segment
// with slot >= 0 writes, instead of the output rows, its unnormalised sums part_o[slot][256 rows][D], and per row
// its reference maximum (in powers of two) and its sum of probabilities part_ml[slot][256] (0 where the row saw no
// key); prefill_combine_kernel then merges an item's slots, in their order, into the output rows.
//
// tiles, q, out, cache, block_table, window as in attention_prefill.cu; the list pads every request
// to whole pairs of groups.  Head size 64 or 128; pages of a divisor or a multiple of 64 tokens.
// Every wait on an mbarrier is bounded (tma.cuh); on giving up the block flags *status = 7.  A list
// whose second group does not go on where the first ends flags *status = 8 (that group is skipped).
#include <limits.h>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace air {

constexpr int AT_BM = 128;      // query rows per block
constexpr int AT_BN = 64;       // keys per step
constexpr int AT_ROW_TILES = 2; // row tiles of 128 queries per block, on one stream of keys
constexpr int AT_STAGES = 4;
constexpr int AT_THREADS = 384; // warp 0 copies, warps 1 and 2 issue, warps 4-7 and 8-11 are the two softmax groups
constexpr int AT_GROUP = 8;     // 16-token tiles per group of the host's list (one row tile)

// 2^x by the special-function unit in one instruction (2^-inf = 0; relative error about 2^-22,
// far below what rounding the probabilities to bfloat16 adds).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two non-negative floats to a pair of bfloat16 (round half up) with integer adds and one byte
// permute.  The conversion instruction shares the special-function pipe with ex2, which is what
// this kernel waits for most (79 % busy before this change); the integer pipe is nearly idle.
__device__ __forceinline__ uint32_t pack_bf16_alu(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for a pair, on the multiply-add pipe instead of the special-function unit (which takes eight
// cycles for a warp's ex2 and is what a row-per-thread softmax waits for).  x is clamped to -126,
// rounded to the nearest integer n by adding 1.5 * 2^23, 2^(x - n) is a cubic on [-0.5, 0.5] (minimax
// in relative error, 7.5e-5: far below the bfloat16 rounding of the probabilities), and n goes into the
// exponent field by an integer shift and add.
__device__ __forceinline__ float2 exp2_fma(float2 x) {
    const float magic = 12582912.f;
    x.x = fmaxf(x.x, -126.f);
    x.y = fmaxf(x.y, -126.f);
    const float2 t = __fadd2_rn(x, make_float2(magic, magic));
    const float2 f = __fadd2_rn(x, __fadd2_rn(make_float2(magic, magic), make_float2(-t.x, -t.y)));
    float2 q = __ffma2_rn(f, make_float2(0.0551716685f, 0.0551716685f), make_float2(0.242611125f, 0.242611125f));
    q = __ffma2_rn(q, f, make_float2(0.693260968f, 0.693260968f));
    q = __ffma2_rn(q, f, make_float2(0.999928057f, 0.999928057f));
    return make_float2(__uint_as_float(__float_as_uint(q.x) + (__float_as_uint(t.x) << 23)),
                       __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(t.y) << 23)));
}
// Which of every eight pairs of a row take exp2_fma (the rest take ex2): balances the two pipes.
constexpr uint32_t EXP_FMA_PAIRS = 0x52;

// One row tile's softmax (see the file's head).  X picks the tile's accumulators and barriers.
struct RowTile {
    int count;       // query rows of the tile that exist
    int pos0;        // position of its first row
    int tok0;        // flat index of its first row
    int first;       // index in the block's key stream of the first key tile it takes
    int n;           // key tiles it takes
};

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_cache,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tiles,
                            int n_pairs, const int* __restrict__ segments, int n_slots, float* __restrict__ part_o,
                            float2* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int H, int K, int P,
                            int window, float scale_log2, int* __restrict__ status) {
    constexpr int SUB = D / 64;                            // 64-column (128-byte) sub-tiles per row
    constexpr int Q_BYTES = SUB * AT_BM * 128;             // one row tile of Q
    constexpr int KV_SUB = AT_BN * 128;                    // one sub-tile of K or V
    constexpr int STAGE_BYTES = 2 * SUB * KV_SUB;          // K then V
    constexpr uint32_t TMEM_COLS = 512;                    // S_A0 S_A1 | S_B0 S_B1 | O_A | O_B
    constexpr uint32_t O_COL = 2 * AT_ROW_TILES * AT_BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sq = smem;
    uint8_t* skv = sq + AT_ROW_TILES * Q_BYTES;
    uint64_t* bars = (uint64_t*)(skv + AT_STAGES * STAGE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;
    uint64_t* kv_empty = kv_full + AT_STAGES;
    uint64_t* s_full = kv_empty + AT_STAGES;     // [row tile][2]
    uint64_t* p_ready = s_full + 4;              // [row tile][2]
    uint64_t* pv_done = p_ready + 4;             // [row tile][2]: key tile j of a row tile completes [j & 1]
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < AT_STAGES; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], AT_ROW_TILES);   // one arrival per issuer
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_ready[i], 4);
            mbar_init(&pv_done[i], 1);
        }
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

    // The block's two groups of the list (heavy ones first) and its head.  The second group has to go
    // on where the first, a full one, ends; the host's list pads every request to whole pairs.
    // (blocks are handed out in the order of blockIdx.x, then blockIdx.y: all heads of the heaviest pair
    // first, then all heads of the next, so that the light pairs fill in behind the heavy ones)
    int pair = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
    int seg_first = 0, seg_count = INT_MAX, slot_out = -1;
    if (segments) {
        const int* sg = segments + 5 * blockIdx.x;
        pair = sg[0], h = sg[1], seg_first = sg[2], seg_count = sg[3], slot_out = sg[4];
    }
    const bool bad_segment = pair < 0 || pair >= n_pairs || h < 0 || h >= H || seg_first < 0 || seg_count < 0 ||
                             slot_out >= n_slots;
    if (bad_segment) pair = 0;
    const int* grp = tiles + 4 * AT_GROUP * AT_ROW_TILES * pair;
    int count_a = 0, count_b = 0;
    for (int i = 0; i < AT_GROUP && !bad_segment; ++i) {
        count_a += grp[4 * i + 3];
        count_b += grp[4 * (AT_GROUP + i) + 3];
    }
    if (bad_segment && threadIdx.x == 0 && status) atomicExch(status, 8);
    const int slot = grp[0], tok0 = grp[1], pos0 = grp[2];
    if (count_b > 0 && (count_a != AT_BM || grp[4 * AT_GROUP] != slot || grp[4 * AT_GROUP + 1] != tok0 + AT_BM ||
                        grp[4 * AT_GROUP + 2] != pos0 + AT_BM)) {
        if (threadIdx.x == 0 && status) atomicExch(status, 8);
        count_b = 0;
    }
    const int kvh = (int)(((long long)h * K) / H);
    const int* bt = block_table + (size_t)slot * max_blocks;
    const bool has_b = count_b > 0;
    const int pos_last_a = pos0 + count_a - 1;
    const int pos_last = has_b ? pos0 + AT_BM + count_b - 1 : pos_last_a;
    const int lo_a = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int lo_b = window > 0 ? max(0, pos0 + AT_BM - window + 1) : 0;
    // The pair's whole stream of key tiles, then the part of it that is this block's, and what of that part each
    // row tile takes.
    const int tile0_all = lo_a / AT_BN;                                           // the stream's first key tile
    const int n_all = count_a > 0 ? pos_last / AT_BN + 1 - tile0_all : 0;
    const int s0 = min(seg_first, n_all);
    const int s1 = (int)min((long long)n_all, (long long)s0 + seg_count);
    const int tile0 = tile0_all + s0;                                             // the block's first key tile
    const int n_stream = s1 - s0;                                                 // key tiles the block fetches
    auto clipped = [&](int count, int pos, int tok, int first, int n) {
        const int a = max(first, s0), b = min(first + n, s1);
        return b > a ? RowTile{count, pos, tok, a - s0, b - a} : RowTile{count, pos, tok, 0, 0};
    };
    RowTile rt[AT_ROW_TILES];
    rt[0] = clipped(count_a, pos0, tok0, 0, count_a > 0 ? pos_last_a / AT_BN + 1 - tile0_all : 0);
    const int first_b = has_b ? lo_b / AT_BN - tile0_all : 0;
    rt[1] = clipped(count_b, pos0 + AT_BM, tok0 + AT_BM, first_b, has_b ? n_all - first_b : 0);

    if (warp == 0) {
        if (lane == 0 && n_stream > 0) {
            // ------------------------------------------------ producer
            // (the lanes holding 32 entries of the block table at a time, instead of one load in front of every
            // tile's copies, was measured: no change, the ring hides that load)
            mbar_expect_tx(q_full, (uint32_t)(Q_BYTES * (has_b ? 2 : 1)));
            for (int x = 0; x < (has_b ? 2 : 1); ++x)
#pragma unroll
                for (int s = 0; s < SUB; ++s)
                    tma_load_2d(sq + x * Q_BYTES + s * AT_BM * 128, &map_q, h * D + 64 * s, tok0 + x * AT_BM, q_full);
            const int box_rows = P < AT_BN ? P : AT_BN;
            const int boxes = AT_BN / box_rows;
            for (int it = 0; it < n_stream; ++it) {
                const int stage = it % AT_STAGES;
                if (it >= AT_STAGES && !mbar_wait(&kv_empty[stage], ((it / AT_STAGES) - 1) & 1, abort_flag)) break;
                const int kbase = (tile0 + it) * AT_BN;
                int valid = 0;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    valid += (first <= pos_last && first + box_rows - 1 >= lo_a) ? 1 : 0;
                }
                mbar_expect_tx(&kv_full[stage], (uint32_t)(valid * box_rows * 128 * SUB * 2));
                uint8_t* dst = skv + stage * STAGE_BYTES;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    if (!(first <= pos_last && first + box_rows - 1 >= lo_a)) continue;
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
    } else if (warp == 1 || warp == 2) {
        if (n_stream > 0) {
            // ------------------------------------------------ MMA issuers, one warp per row tile: while one
            // waits for its softmax, the other's products keep the tensor cores busy.  The warp runs
            // together and an elected lane issues (the operands then stay in uniform registers).
            // A row tile takes the key tiles [first, first + n) of the stream; for the others its
            // issuer only hands the stage back (after it was filled, so that it cannot run ahead).
            const int x = warp - 1;
            const RowTile me = x ? rt[1] : rt[0];
            constexpr uint32_t idesc_qk = umma_idesc(AT_BM, AT_BN);
            constexpr uint32_t idesc_pv = umma_idesc(AT_BM, D, true);
            const uint32_t qaddr = smem_u32(sq + x * Q_BYTES);
            const uint32_t s_cols = tmem_base + 2 * x * AT_BN;
            const uint32_t o_cols = tmem_base + O_COL + x * D;
            uint64_t* my_s_full = s_full + 2 * x;
            uint64_t* my_p_ready = p_ready + 2 * x;
            uint64_t* my_pv_done = pv_done + 2 * x;
            bool ok = true;
            auto pass = [&](int from, int to) {   // key tiles that this row tile does not take
                for (int t = from; t < to && ok; ++t) {
                    const int stage = t % AT_STAGES;
                    ok = __all_sync(0xffffffffu, mbar_wait(&kv_full[stage], (t / AT_STAGES) & 1, abort_flag));
                    if (ok && elect_one()) mbar_arrive(&kv_empty[stage]);
                    __syncwarp();
                }
            };
            pass(0, me.first);
            if (me.n > 0) {
                ok = ok && __all_sync(0xffffffffu, mbar_wait(q_full, 0, abort_flag));
                tc_fence_after();
            }
            for (int j = 0; j <= me.n && ok && me.n > 0; ++j) {
                if (j < me.n) {
                    // S(j) = Q K(j)^T into S[j & 1] (which held P(j-2): the product that read it was
                    // issued before this one)
                    const int t = me.first + j, stage = t % AT_STAGES;
                    if (!mbar_try_wait(&kv_full[stage], (t / AT_STAGES) & 1))      // (mostly there already: one try)
                        ok = __all_sync(0xffffffffu, mbar_wait(&kv_full[stage], (t / AT_STAGES) & 1, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t kaddr = smem_u32(skv + stage * STAGE_BYTES);
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk)
                            umma_bf16(s_cols + (j & 1) * AT_BN, umma_desc(qaddr + (kk / 4) * AT_BM * 128) + 2 * (kk % 4),
                                      umma_desc(kaddr + (kk / 4) * KV_SUB) + 2 * (kk % 4), idesc_qk, kk > 0 ? 1u : 0u);
                        umma_commit(&my_s_full[j & 1]);
                    }
                    __syncwarp();
                }
                if (j >= 1) {
                    // O += P(j-1) V(j-1), P from tensor memory (where S(j-1) was)
                    const int u = j - 1, t = me.first + u, stage = t % AT_STAGES;
                    ok = __all_sync(0xffffffffu, mbar_wait(&my_p_ready[u & 1], (u >> 1) & 1, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t vaddr = smem_u32(skv + stage * STAGE_BYTES + SUB * KV_SUB);
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < AT_BN / 16; ++ks)
                            umma_bf16_ts(o_cols, s_cols + (u & 1) * AT_BN + 8 * ks, umma_desc_mn(vaddr + ks * 16 * 128, KV_SUB),
                                         idesc_pv, (u > 0 || ks > 0) ? 1u : 0u);
                        umma_commit(&my_pv_done[u & 1]);
                        umma_commit(&kv_empty[stage]);
                    }
                    __syncwarp();
                }
            }
            pass(me.first + me.n, n_stream);
        }
    } else if (warp >= 4 && (warp >= 8 ? rt[1].n : rt[0].n) == 0) {
        // a row tile that has no key in this segment: its rows of the slot say so
        const int x = (warp - 4) >> 2, r = (warp & 3) * 32 + lane;
        if (slot_out >= 0 && r < (x ? rt[1].count : rt[0].count))
            part_ml[(size_t)slot_out * (AT_ROW_TILES * AT_BM) + x * AT_BM + r] = make_float2(-INFINITY, 0.f);
    } else if (warp >= 4) {
        // ---------------------------------------------------- softmax: one thread per query row
        const int x = (warp - 4) >> 2;
        const RowTile me = x ? rt[1] : rt[0];
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int pos = me.pos0 + r;
        uint64_t* my_s_full = s_full + 2 * x;
        uint64_t* my_p_ready = p_ready + 2 * x;
        uint64_t* my_pv_done = pv_done + 2 * x;
        const uint32_t my_s = tmem_base + lane_addr + 2 * x * AT_BN;
        const uint32_t my_o = tmem_base + lane_addr + O_COL + x * D;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < me.n && ok; ++it) {
            const int b = it & 1;
            ok = mbar_wait(&my_s_full[b], (it >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[AT_BN];
            tmem_ld64(my_s + b * AT_BN, sv);
            const int kbase = (tile0 + me.first + it) * AT_BN;
            // Scores stay as the product left them; the scale goes into the exponent's multiply-add.
            // Only tiles on the diagonal or at a window's edge need the mask (the same for the warp).
            const int warp_first = me.pos0 + quarter * 32;
            const bool full_tile = kbase + AT_BN - 1 <= warp_first && (window <= 0 || kbase > warp_first + 31 - window);
            // (four running maxima and, below, two pairs of running sums: independent chains)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (full_tile) {
#pragma unroll
                for (int c = 0; c < AT_BN; c += 2)
                    mx4[(c >> 1) & 3] = max3(mx4[(c >> 1) & 3], __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
            } else {
#pragma unroll
                for (int c = 0; c < AT_BN; ++c) {
                    const int key = kbase + c;
                    const bool vis = key <= pos && (window <= 0 || key > pos - window);
                    const float v = vis ? __uint_as_float(sv[c]) : -INFINITY;
                    sv[c] = __float_as_uint(v);
                    mx4[c & 3] = fmaxf(mx4[c & 3], v);
                }
            }
            // the scale is positive: the maximum of the scaled scores
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // The reference maximum m of the row moves only when the tile's maximum exceeds it by more
            // than 2^8 (or the row had seen no key): probabilities up to 256 are harmless in bfloat16 and
            // in the 32-bit sums, and a row of O that is not rescaled does not have to wait for the
            // product that is still writing it.
            const bool move = mx > m + 8.f;
            const float m_new = move ? mx : m;
            const float base = m_new == -INFINITY ? 0.f : m_new;   // a row that sees no key yet
            const float corr = move ? fast_exp2(m - base) : 1.f;
            m = m_new;
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            uint32_t pk[AT_BN / 2];
            const float2 scale2 = make_float2(scale_log2, scale_log2), nbase2 = make_float2(-base, -base);
            if (full_tile) {
#pragma unroll
                for (int c = 0; c < AT_BN; c += 2) {
                    const float2 v =
                        __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, nbase2);
                    float2 pr;
                    if ((EXP_FMA_PAIRS >> ((c >> 1) & 7)) & 1) {
                        pr = exp2_fma(v);
                    } else {
                        pr.x = fast_exp2(v.x);
                        pr.y = fast_exp2(v.y);
                    }
                    sum2[(c >> 1) & 1] = __fadd2_rn(sum2[(c >> 1) & 1], pr);
                    pk[c >> 1] = pack_bf16_alu(pr.x, pr.y);
                }
            } else {   // (a masked key's -inf stays with ex2)
#pragma unroll
                for (int c = 0; c < AT_BN; c += 2) {
                    const float2 v =
                        __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, nbase2);
                    const float2 pr = make_float2(fast_exp2(v.x), fast_exp2(v.y));
                    sum2[(c >> 1) & 1] = __fadd2_rn(sum2[(c >> 1) & 1], pr);
                    pk[c >> 1] = pack_bf16_alu(pr.x, pr.y);
                }
            }
            l = l * corr + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
            // The product of tile it-2 has completed (S(it) was written after it, in the order of
            // issue).  Looking at its barrier all the same, every time, keeps the parity that a wait
            // sees at most one phase behind: a wait by parity cannot tell a phase from the one two later.
            if (it >= 2) {
                ok = mbar_wait(&my_pv_done[b], ((it >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
            }
            if (it >= 1 && __any_sync(0xffffffffu, move)) {
                // O must be rescaled: every product issued so far (up to tile it-1) has to be complete
                ok = mbar_wait(&my_pv_done[b ^ 1], ((it - 1) >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(my_o + c, ov);
#pragma unroll
                    for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * corr);
                    tmem_st32(my_o + c, ov);
                }
            }
            // P(it): this row's 64 probabilities as 32 columns of pairs, over the scores they came from;
            // the second product reads its A operand there: no shared memory and no proxy fence on the way
            tmem_st32(my_s + b * AT_BN, pk);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&my_p_ready[b]);
        }
        if (ok && me.n >= 2) ok = mbar_wait(&my_pv_done[me.n & 1], ((me.n - 2) >> 1) & 1, abort_flag);
        if (ok) ok = mbar_wait(&my_pv_done[(me.n - 1) & 1], ((me.n - 1) >> 1) & 1, abort_flag);
        if (ok) {
            // The rows leave through the row tile's own Q tile in shared memory, which no product reads any more:
            // thread r puts its row there in 16-byte chunks (chunk c at place c ^ r of the row: no two lanes of a
            // quarter-warp on one bank), then the warp copies its 32 rows out, a whole row per instruction.  (A
            // thread that stores its own row to global memory writes 8 of every 32-byte sector per instruction:
            // 6-7 us for the tile, measured, against about 1 us so.)
            tc_fence_after();
            constexpr int ROWB = D * 2, CHUNKS = ROWB / 16, LANEB = ROWB / 32;
            uint8_t* stage = sq + x * Q_BYTES;
            auto put = [&](int chunk, uint4 v) {
                *reinterpret_cast<uint4*>(stage + r * ROWB + ((chunk ^ (r & (CHUNKS - 1))) << 4)) = v;
            };
            auto copy_out = [&](uint8_t* row0, size_t row_bytes) {
                __syncwarp();
                const int byte = lane * LANEB;
                for (int i = 0; i < 32; ++i) {
                    const int row = quarter * 32 + i;
                    if (row >= me.count) break;
                    const uint8_t* src = stage + row * ROWB + (((byte >> 4) ^ (row & (CHUNKS - 1))) << 4) + (byte & 15);
                    uint8_t* dst = row0 + row * row_bytes + byte;
                    if constexpr (LANEB == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
                    else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
                }
                __syncwarp();
            };
            if (slot_out >= 0) {
                // the segment's sums as they are (float32, half the columns at a time), and what the merge needs
                // to weigh them
                const size_t row = (size_t)slot_out * (AT_ROW_TILES * AT_BM) + x * AT_BM;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int c = 0; c < D / 2; c += 32) {
                        uint32_t ov[32];
                        tmem_ld32(my_o + half * (D / 2) + c, ov);
#pragma unroll
                        for (int e = 0; e < 32; e += 4) put((c + e) >> 2, make_uint4(ov[e], ov[e + 1], ov[e + 2], ov[e + 3]));
                    }
                    copy_out(reinterpret_cast<uint8_t*>(part_o + row * D + half * (D / 2)), (size_t)D * 4);
                }
                if (r < me.count) part_ml[row + r] = make_float2(m, l);
            } else {
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(my_o + c, ov);
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint32_t pk[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(ov[e + 2 * k]) * inv,
                                                                             __uint_as_float(ov[e + 2 * k + 1]) * inv);
                            pk[k] = *reinterpret_cast<const uint32_t*>(&two);
                        }
                        put((c + e) >> 3, make_uint4(pk[0], pk[1], pk[2], pk[3]));
                    }
                }
                copy_out(reinterpret_cast<uint8_t*>(out + ((size_t)me.tok0 * H + h) * D), (size_t)H * D * 2);
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

// Merges the slots of the cut items: out row = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s with M the largest
// m_s, the slots in their order.  items [m, 4] = (pair, head, first slot, slots).  Grid (items, 32): a block takes 8
// of the pair's 256 rows, a warp one row, a lane D / 32 columns.  Lane s first weighs slot s (all slots' maxima and
// sums are loaded at once), then the warp adds the slots' rows, four loads in flight.
template <int D>
__global__ void __launch_bounds__(256)
prefill_combine_kernel(const int* __restrict__ tiles, int n_pairs, const int* __restrict__ items, int n_slots,
                       const float* __restrict__ part_o, const float2* __restrict__ part_ml,
                       __nv_bfloat16* __restrict__ out, int H, int* __restrict__ status) {
    constexpr int CP = D / 32;
    constexpr int ROWS = AT_ROW_TILES * AT_BM;
    pdl_enter(TR_ATT_COMBINE);
    const int* item = items + 4 * blockIdx.x;
    const int pair = item[0], h = item[1], slot0 = item[2], n = item[3];
    if (pair < 0 || pair >= n_pairs || h < 0 || h >= H || slot0 < 0 || n < 1 || slot0 + n > n_slots) {
        if (threadIdx.x == 0 && status) atomicExch(status, 8);
        return;
    }
    const int* grp = tiles + 4 * AT_GROUP * AT_ROW_TILES * pair;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.y * 8 + warp;
    // rows of the pair that exist: the counts of the 16 entries (lanes 0-15 hold one each)
    const int mine = lane < AT_GROUP * AT_ROW_TILES ? grp[4 * lane + 3] : 0;
    const int before = __reduce_add_sync(0xffffffffu, lane < AT_GROUP ? mine : 0);
    const int after = __reduce_add_sync(0xffffffffu, lane < AT_GROUP ? 0 : mine);
    if (!(r < AT_BM ? r < before : r - AT_BM < after)) return;
    const int tok0 = grp[1];
    float top = -INFINITY, weight = 0.f, acc[CP];
#pragma unroll
    for (int c = 0; c < CP; ++c) acc[c] = 0.f;
    // (more than 32 slots: in rounds; the running sums are rescaled when a round raises the maximum)
    for (int s0 = 0; s0 < n; s0 += 32) {
        const int s = s0 + lane;
        const float2 ml = s < n ? part_ml[(size_t)(slot0 + s) * ROWS + r] : make_float2(-INFINITY, 0.f);
        const bool live = ml.y > 0.f;
        const float round_top = warp_max(live ? ml.x : -INFINITY);
        if (round_top == -INFINITY) continue;
        const float new_top = fmaxf(top, round_top);
        const float keep = top == -INFINITY ? 0.f : exp2f(top - new_top);
        top = new_top;
        const float w = live ? exp2f(ml.x - top) : 0.f;
        weight = weight * keep + warp_sum(w * ml.y);
#pragma unroll
        for (int c = 0; c < CP; ++c) acc[c] *= keep;
        const int round = min(32, n - s0);
        const float* src = part_o + ((size_t)(slot0 + s0) * ROWS + r) * D + lane * CP;
#pragma unroll 4
        for (int j = 0; j < round; ++j) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (wj > 0.f) {
                float v[CP];
                if constexpr (CP == 4) {
                    const float4 t = *reinterpret_cast<const float4*>(src + (size_t)j * ROWS * D);
                    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
                } else {
                    const float2 t = *reinterpret_cast<const float2*>(src + (size_t)j * ROWS * D);
                    v[0] = t.x, v[1] = t.y;
                }
#pragma unroll
                for (int c = 0; c < CP; ++c) acc[c] += wj * v[c];
            }
        }
    }
    const float inv = weight > 0.f ? 1.f / weight : 0.f;
    __nv_bfloat16* dst = out + ((size_t)(tok0 + r) * H + h) * D + lane * CP;
#pragma unroll
    for (int c = 0; c < CP; c += 2)
        *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(acc[c] * inv, acc[c + 1] * inv);
}

static int make_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    return tensor_map_2d(map, base, rows, cols, box_rows);
}

template <int D>
int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mc, const int* block_table, int max_blocks,
                      const int* tiles, int n_tiles, const int* segments, int n_segments, const int* items, int n_items,
                      int n_slots, float* part_o, float* part_ml, void* out, int H, int K, int P, int window, float scale,
                      int* status, cudaStream_t stream) {
    // (more than half of an SM's shared memory, so that two blocks never share its tensor memory)
    size_t smem = 1024 + (size_t)AT_ROW_TILES * (D / 64) * AT_BM * 128 +
                  (size_t)AT_STAGES * 2 * (D / 64) * AT_BN * 128 + 256;
    if (smem < 120 * 1024) smem = 120 * 1024;
    auto kernel = prefill_attention_tc_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int n_pairs = n_tiles / (AT_GROUP * AT_ROW_TILES);
    const dim3 grid = segments ? dim3(n_segments) : dim3(H, n_pairs);
    int rc = launch(kernel, grid, AT_THREADS, smem, stream, mq, mc, block_table, max_blocks, tiles, n_pairs, segments,
                    n_slots, part_o, (float2*)part_ml, (__nv_bfloat16*)out, H, K, P, window,
                    scale * 1.4426950408889634f, status);
    if (rc || !segments || n_items <= 0) return rc;
    return launch(prefill_combine_kernel<D>, dim3(n_items, AT_ROW_TILES * AT_BM / 8), 256, 0, stream, tiles, n_pairs,
                  items, n_slots, (const float*)part_o, (const float2*)part_ml, (__nv_bfloat16*)out, H, status);
}

}  // namespace air

// q [T, H, D] bf16.  tiles: n_tiles entries in groups of 16 per request.  Head size 64 or 128.
// segments (or null: one block per pair and head) [n_segments, 5], items [n_items, 4], part_o float32
// [n_slots, 256, D] and part_ml float32 [n_slots, 256, 2]: see the head of this file.
AIR_API int air_prefill_attention_tc(const void* q, int T, const void* cache, long long pages, const int* block_table,
                                     int max_blocks, const int* tiles, int n_tiles, const int* segments, int n_segments,
                                     const int* items, int n_items, int n_slots, float* part_o, float* part_ml,
                                     void* out, int H, int K, int D, int P, int window, float scale, int* status,
                                     cudaStream_t stream) {
    using namespace air;
    if (n_tiles <= 0) return 0;
    if (segments && (n_segments <= 0 || n_items < 0 || n_slots < 0 || (n_items > 0 && !items) ||
                     (n_slots > 0 && (!part_o || !part_ml || ((uintptr_t)part_o & 15) || ((uintptr_t)part_ml & 7)))))
        return AIR_ERR_BAD_ARGUMENT;
    if (!segments) n_items = n_slots = 0;
    if (H <= 0 || K <= 0 || H % K || P % 16 || (P < 64 ? 64 % P : P % 64) || n_tiles % (AT_GROUP * AT_ROW_TILES) || n_tiles / (AT_GROUP * AT_ROW_TILES) > 65535 ||
        ((uintptr_t)cache & 15) || ((uintptr_t)q & 15) || (D != 64 && D != 128))
        return AIR_ERR_BAD_ARGUMENT;
    CUtensorMap mq, mc;
    int rc = make_map_2d(&mq, q, T, (long long)H * D, AT_BM);
    if (rc) return rc;
    rc = make_map_2d(&mc, cache, pages * 2 * K * P, D, P < AT_BN ? P : AT_BN);
    if (rc) return rc;
    if (D == 64)
        return launch_prefill_tc<64>(mq, mc, block_table, max_blocks, tiles, n_tiles, segments, n_segments, items, n_items,
                                     n_slots, part_o, part_ml, out, H, K, P, window, scale, status, stream);
    return launch_prefill_tc<128>(mq, mc, block_table, max_blocks, tiles, n_tiles, segments, n_segments, items, n_items,
                                  n_slots, part_o, part_ml, out, H, K, P, window, scale, status, stream);
}

AIR_API int air_trace_set_attention_prefill_tc(unsigned long long* buffer) { return air::set_trace_here(buffer); }
