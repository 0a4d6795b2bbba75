// Decode attention over the paged cache for bfloat16, keys and values moved by the copy engine.
//
// The same split of the work as attention_decode.cu (one query token per request, the query heads
// of a group as the M dimension of mma.sync m16n8k16, the token's keys split over `splits` blocks,
// partial results merged by decode_combine), but the bytes take another road.  A producer warp
// issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of 64-key tiles of K and V from the
// pages into a ring of shared-memory stages; mbarriers tell the four consumer warps when a tile has
// landed and the producer when a stage is free again.  Each consumer warp takes 16 of the tile's 64
// keys and reads its MMA operands with ldmatrix (K as it lies, V transposed), which the swizzle makes
// free of bank conflicts.  The copy engine asks memory for whole rows at a time, which a warp's
// 16-byte loads do not, and the consumers issue no load instructions for the cache at all.
//
// The cache [page, 2, K, P, D] is addressed as a matrix of rows of D elements; a 64-key tile is
// 64 / min(P, 64) boxes of min(P, 64) rows, each found through the block table.
// Every wait on an mbarrier is bounded (tma.cuh); on giving up the block flags *status = 5.
//
// With `fresh.qkv` the kernel also does what qkv_rope_store does for its token (elementwise.cu): it adds up
// the partial sums of the q/k/v product and the bias, rotates q and k by the table's row of the token's
// position, keeps q in shared memory, and writes k and v to the page.  The blocks whose tiles hold the
// token's own position do not wait for that write to be visible to the copy engine: they put the two new
// rows into the tile in shared memory once it has landed.  A decode step is then one launch shorter per
// layer, and the keys start to stream as soon as the product has ended.
#include "common.cuh"
#include "mma.cuh"
#include "tma.cuh"

namespace air {

constexpr int DT_CONSUMERS = 4;
constexpr int DT_THREADS = (DT_CONSUMERS + 1) * 32;
constexpr int DT_TILE = 64;     // keys per stage
constexpr int DT_STAGES = 3;
constexpr int FRESH_PARTS = 4;  // partial sums of the q/k/v product that a thread asks for at once

// The token's new q, k and v as the product left them (see the head of the file); qkv == nullptr: q is read
// from `q`, and k and v are in the cache already.
struct FreshQkv {
    const float* qkv;        // [parts][T][(H + 2 K) D] partial sums
    int parts;
    size_t part_stride;
    const float* bias;       // [(H + 2 K) D] or nullptr
    const float* table;      // [positions][D]: cos | sin
    __nv_bfloat16* cache;    // where k and v are written (nullptr: another run has written them)
};

template <int D>
__global__ void __launch_bounds__(DT_THREADS)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_cache, const FreshQkv fresh,
                            const __nv_bfloat16* __restrict__ q,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_seq,
                            const int* __restrict__ positions, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ part_o, float* __restrict__ part_ml, int H, int K, int P, int window,
                            float scale_log2, int* status) {
    constexpr int SUB = D / 64;                 // 64-column sub-tiles of a row
    constexpr int SUB_BYTES = DT_TILE * 128;    // 8 KB
    constexpr int STAGE_BYTES = 2 * SUB * SUB_BYTES;
    constexpr int KS = D / 16;                  // k-steps of Q K^T
    constexpr int NT = D / 8;                   // 8-column tiles of the output
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + DT_STAGES * STAGE_BYTES);
    uint64_t* empty = full + DT_STAGES;
    volatile int* abort_flag = (volatile int*)(empty + DT_STAGES);
    __nv_bfloat16* sm_q = (__nv_bfloat16*)((uint8_t*)(empty + DT_STAGES) + 64);   // [16][D], with fresh.qkv
    __nv_bfloat16* sm_kv = sm_q + 16 * D;                                          // [2][D]: the new k and v rows
    float* sm_o = (float*)smem;                              // after the walk: [warps][16][D]
    float* sm_m = sm_o + DT_CONSUMERS * 16 * D;              // [warps][16]
    float* sm_l = sm_m + DT_CONSUMERS * 16;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < DT_STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], DT_CONSUMERS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Where a tile is not filled by one copy (pages smaller than a tile, pages that a window has given
    // back) the ring starts as zeros: rows that no copy fills then hold zeros or earlier keys, never
    // bits that could be NaN.
    if (P < DT_TILE || window > 0) {
        for (int i = threadIdx.x; i < DT_STAGES * STAGE_BYTES / 16; i += DT_THREADS)
            reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // keys and values pass through L2 once: evict-first, so that their stream leaves the weights that the
    // following products have asked for there
    uint64_t kv_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(kv_policy));
    // With fresh.qkv the predecessor is the q/k/v product, whose output only the consumer warps read: the
    // producer warp does not wait for it.  What it reads was written long before: the step's positions, slots
    // and block tables (copied or updated before the step's first kernel, which lets nothing start before that
    // is done, see embedding_kernel) and keys and values of earlier steps; the token's own key and value never
    // come from the copy (they are patched into the tile from shared memory).  So the first tiles of old keys
    // are on their way while the product's last blocks still run.  Without fresh.qkv the token's key and value
    // were written to the page by the predecessor itself, and everybody waits.
    if (!(warp == DT_CONSUMERS && fresh.qkv)) pdl_wait();
    trace_point(TR_ATT_DECODE);

    const int t = blockIdx.z;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int G = H / K;
    const int head_blocks = (G + 15) / 16;
    const int kvh = blockIdx.y / head_blocks, hb = blockIdx.y % head_blocks;
    const int split = blockIdx.x, splits = gridDim.x;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)slot * max_blocks;
    const int tile0 = lo / DT_TILE, tile1 = pos / DT_TILE + 1;
    const int per = (tile1 - tile0 + splits - 1) / splits;
    const int begin = tile0 + split * per, end = min(tile1, begin + per);
    const int n_tiles = max(0, end - begin);

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int g = lane >> 2, tq = lane & 3;

    if (warp == DT_CONSUMERS) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            const int box_rows = P < DT_TILE ? P : DT_TILE;
            const int boxes = DT_TILE / box_rows;
            for (int it = 0; it < n_tiles; ++it) {
                const int stage = it % DT_STAGES;
                if (it >= DT_STAGES && !mbar_wait(&empty[stage], ((it / DT_STAGES) - 1) & 1, abort_flag)) break;
                const int kbase = (begin + it) * DT_TILE;
                int valid = 0;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    valid += (first <= pos && first + box_rows - 1 >= lo) ? 1 : 0;
                }
                mbar_expect_tx(&full[stage], (uint32_t)(valid * box_rows * 128 * SUB * 2));
                uint8_t* dst = smem + stage * STAGE_BYTES;
                for (int b = 0; b < boxes; ++b) {
                    const int first = kbase + b * box_rows;
                    if (!(first <= pos && first + box_rows - 1 >= lo)) continue;
                    const int page = bt[first / P];
                    const int row_k = ((page * 2) * K + kvh) * P + first % P;
                    const int row_v = row_k + K * P;
#pragma unroll
                    for (int s = 0; s < SUB; ++s) {
                        tma_load_2d_hint(dst + s * SUB_BYTES + b * box_rows * 128, &map_cache, 64 * s, row_k, &full[stage],
                                         kv_policy);
                        tma_load_2d_hint(dst + (SUB + s) * SUB_BYTES + b * box_rows * 128, &map_cache, 64 * s, row_v,
                                         &full[stage], kv_policy);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ consumers: 16 keys of every tile each
        const int r0 = hb * 16 + g, r1 = r0 + 8;
        uint32_t qa[KS][4];
        const int own_tile = pos / DT_TILE;           // the tile that holds the token's own key
        const bool patch = fresh.qkv && fresh.cache && own_tile >= begin && own_tile < end;
        if (fresh.qkv) {
            // this block's query heads, and k and v where its tiles hold the new key: items of four pairs
            // (i, i + D/2), as in qkv_rope_store_vec4_kernel
            constexpr int HALF = D / 2, PER_HEAD = HALF / 4;
            const int width = (H + 2 * K) * D;
            const int nq = min(16, G - hb * 16);
            const int heads = nq + (patch ? 2 : 0);
            const float* in = fresh.qkv + (size_t)t * width;
            const float* cs = fresh.table + (size_t)pos * D;
            __nv_bfloat16* kdst = nullptr;
            if (patch && hb == 0) {
                const int page = bt[pos / P];
                if (page < 0) {
                    if (threadIdx.x == 0 && status) atomicExch(status, 2);
                } else {
                    kdst = fresh.cache + ((size_t)page * 2 * K * P + (size_t)kvh * P + (size_t)(pos % P)) * D;
                }
            }
            for (int idx = threadIdx.x; idx < heads * PER_HEAD; idx += DT_CONSUMERS * 32) {
                const int hh = idx / PER_HEAD, j = (idx % PER_HEAD) * 4;
                const int col = (hh < nq ? kvh * G + hb * 16 + hh : (hh == nq ? H + kvh : H + K + kvh)) * D;
                // all of the item's loads are asked for at once (up to FRESH_PARTS partial sums, the bias, the
                // table's row): with few tiles to stream this chain of latencies is what the block waits for
                float a[4], b[4], pa[FRESH_PARTS - 1][4], pb[FRESH_PARTS - 1][4];
                float ba[4] = {0.f, 0.f, 0.f, 0.f}, bb[4] = {0.f, 0.f, 0.f, 0.f}, c[4], sn[4];
                load4(in + col + j, a);
                load4(in + col + HALF + j, b);
#pragma unroll
                for (int part = 1; part < FRESH_PARTS; ++part)
                    if (part < fresh.parts) {
                        load4(in + part * fresh.part_stride + col + j, pa[part - 1]);
                        load4(in + part * fresh.part_stride + col + HALF + j, pb[part - 1]);
                    }
                if (fresh.bias) {
                    load4(fresh.bias + col + j, ba);
                    load4(fresh.bias + col + HALF + j, bb);
                }
                if (hh <= nq) {
                    load4(cs + j, c);
                    load4(cs + HALF + j, sn);
                }
#pragma unroll
                for (int part = 1; part < FRESH_PARTS; ++part)
                    if (part < fresh.parts) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) { a[e] += pa[part - 1][e]; b[e] += pb[part - 1][e]; }
                    }
                for (int part = FRESH_PARTS; part < fresh.parts; ++part) {
                    float x[4], y[4];
                    load4(in + part * fresh.part_stride + col + j, x);
                    load4(in + part * fresh.part_stride + col + HALF + j, y);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { a[e] += x[e]; b[e] += y[e]; }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) { a[e] += ba[e]; b[e] += bb[e]; }
                if (hh <= nq) {                       // q and k are rotated, v is not
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float ra = a[e] * c[e] - b[e] * sn[e], rb = a[e] * sn[e] + b[e] * c[e];
                        a[e] = ra;
                        b[e] = rb;
                    }
                }
                __nv_bfloat16* dst = hh < nq ? sm_q + hh * D : sm_kv + (hh - nq) * D;
                store4(dst + j, a);
                store4(dst + HALF + j, b);
                if (hh >= nq && kdst) {
                    __nv_bfloat16* gdst = kdst + (hh == nq ? (size_t)0 : (size_t)K * P * D);
                    store4(gdst + j, a);
                    store4(gdst + HALF + j, b);
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(DT_CONSUMERS * 32) : "memory");
        }
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            if (fresh.qkv) {
                const __nv_bfloat16* q0 = sm_q + g * D + 16 * kk + 2 * tq;
                const __nv_bfloat16* q1 = q0 + 8 * D;
                qa[kk][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0) : 0u;
                qa[kk][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1) : 0u;
                qa[kk][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + 8) : 0u;
                qa[kk][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + 8) : 0u;
            } else {
                const __nv_bfloat16* q0 = q + ((size_t)t * H + kvh * G + r0) * D + 16 * kk + 2 * tq;
                const __nv_bfloat16* q1 = q + ((size_t)t * H + kvh * G + r1) * D + 16 * kk + 2 * tq;
                qa[kk][0] = r0 < G ? __ldg(reinterpret_cast<const uint32_t*>(q0)) : 0u;
                qa[kk][1] = r1 < G ? __ldg(reinterpret_cast<const uint32_t*>(q1)) : 0u;
                qa[kk][2] = r0 < G ? __ldg(reinterpret_cast<const uint32_t*>(q0 + 8)) : 0u;
                qa[kk][3] = r1 < G ? __ldg(reinterpret_cast<const uint32_t*>(q1 + 8)) : 0u;
            }
        }
        const int mat = lane >> 3, mrow = lane & 7;   // ldmatrix: which 8x8 matrix this lane addresses, which row
        bool alive = true;
        for (int it = 0; it < n_tiles; ++it) {
            const int stage = it % DT_STAGES;
            // (a warp whose wait ran out goes on without work, so that it still meets the others at the barrier below)
            if (alive && !mbar_wait(&full[stage], (it / DT_STAGES) & 1, abort_flag)) alive = false;
            if (patch && begin + it == own_tile) {
                // the token's own k and v: into their row of the tile (what the copy brought there is older)
                const int row = pos - own_tile * DT_TILE;
                if (alive && threadIdx.x < 2 * (D / 8)) {
                    const int which = threadIdx.x / (D / 8), c = threadIdx.x % (D / 8);
                    const uint4 val = *reinterpret_cast<const uint4*>(sm_kv + which * D + c * 8);
                    const uint32_t at = swizzled(smem_u32(smem + stage * STAGE_BYTES) + (which * SUB + c / 8) * SUB_BYTES,
                                                 row, c % 8);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(val.x), "r"(val.y),
                                 "r"(val.z), "r"(val.w) : "memory");
                }
                asm volatile("bar.sync 1, %0;" ::"n"(DT_CONSUMERS * 32) : "memory");
            }
            if (!alive) continue;
            const int kbase = (begin + it) * DT_TILE + 16 * warp;     // this warp's 16 keys
            if (kbase <= pos && kbase + 15 >= lo) {
                const uint32_t kt = smem_u32(smem + stage * STAGE_BYTES);
                const uint32_t vt = kt + SUB * SUB_BYTES;
                float s[2][4] = {};
#pragma unroll
                for (int kk = 0; kk < KS; ++kk) {
                    // matrices: (keys 0-7, d 16kk..+7), (keys 0-7, d 16kk+8..), (keys 8-15, same two)
                    uint32_t b[4];
                    ldmatrix_x4(b, swizzled(kt + (kk / 4) * SUB_BYTES, 16 * warp + (mat >> 1) * 8 + mrow,
                                            2 * (kk % 4) + (mat & 1)));
                    mma_bf16_16816(s[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b[0], b[1]);
                    mma_bf16_16816(s[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b[2], b[3]);
                }
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
                const float n0 = fmaxf(m0, tm0), n1 = fmaxf(m1, tm1);   // finite: at least one key is visible
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
                for (int n = 0; n < NT; n += 2) {
                    // matrices: (keys 0-7, d 8n..+7), (keys 8-15, same), (keys 0-7, d 8(n+1)..), (keys 8-15, same)
                    uint32_t b[4];
                    const int chunk = n + (mat >> 1);
                    ldmatrix_x4_trans(b, swizzled(vt + (chunk / 8) * SUB_BYTES, 16 * warp + (mat & 1) * 8 + mrow,
                                                  chunk % 8));
                    mma_bf16_16816(o[n], pa0, pa1, pa2, pa3, b[0], b[1]);
                    mma_bf16_16816(o[n + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }

    // ---------------------------------------------------------------- merge the four warps
    __syncthreads();   // every tile has been consumed: the ring's memory is used again
    if (*abort_flag) {
        for (int i = 0; i < 32; ++i) __nanosleep(2000);   // copies on their way may still land
        if (threadIdx.x == 0 && status) atomicExch(status, 5);
        return;
    }
    if (warp < DT_CONSUMERS) {
        if (tq == 0) {
            sm_m[warp * 16 + g] = m0;
            sm_m[warp * 16 + g + 8] = m1;
            sm_l[warp * 16 + g] = l0;
            sm_l[warp * 16 + g + 8] = l1;
        }
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                sm_o[(warp * 16 + g + 8 * (e >> 1)) * D + 8 * n + 2 * tq + (e & 1)] = o[n][e];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * D; idx += DT_THREADS) {
        const int r = idx / D, col = idx % D;
        if (hb * 16 + r >= G) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DT_CONSUMERS; ++w) mm = fmaxf(mm, sm_m[w * 16 + r]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < DT_CONSUMERS; ++w) {
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

template <int D>
int launch_decode_tma(const CUtensorMap& map, const FreshQkv& fresh, const void* q, const int* block_table, int max_blocks,
                      const int* token_seq, const int* positions, void* out, float* part_o, float* part_ml, int T,
                      int H, int K, int P, int window, float scale, int splits, int* status, cudaStream_t stream) {
    const int head_blocks = (H / K + 15) / 16;
    const size_t ring = (size_t)DT_STAGES * 2 * (D / 64) * DT_TILE * 128;
    const size_t merge = (size_t)(DT_CONSUMERS * 16 * D + 2 * DT_CONSUMERS * 16) * sizeof(float);
    const size_t smem = 1024 + (ring > merge ? ring : merge) + 128 + (fresh.qkv ? (size_t)18 * D * 2 : 0);
    auto kernel = decode_attention_tma_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch(kernel, dim3(splits, K * head_blocks, T), DT_THREADS, smem, stream, map, fresh, (const __nv_bfloat16*)q,
                  block_table, max_blocks, token_seq, positions, (__nv_bfloat16*)out, part_o, part_ml, H, K, P, window,
                  scale * 1.4426950408889634f, status);
}

}  // namespace air

// The merge of the splits (attention_decode.cu).
extern "C" int air_decode_combine(const float* part_o, const float* part_ml, const int* token_seq, void* out, int T,
                                  int H, int D, int splits, cudaStream_t stream);

namespace air {

static int decode_attention_tma(const FreshQkv& fresh, const void* q, const void* cache, long long pages,
                                const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                void* out, float* part_o, float* part_ml, int T, int H, int K, int D, int P, int window,
                                float scale, int splits, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || H % K || P % 16 || (P < 64 ? 64 % P : P % 64) || splits < 1 || T > 65535 ||
        (splits > 1 && (!part_o || !part_ml)) || ((uintptr_t)cache & 15))
        return AIR_ERR_BAD_ARGUMENT;
    CUtensorMap map;
    const int map_rc = tensor_map_2d(&map, cache, pages * 2 * K * P, D, P < DT_TILE ? P : DT_TILE);
    if (map_rc) return map_rc;
    int rc;
    switch (D) {
        case 64:
            rc = launch_decode_tma<64>(map, fresh, q, block_table, max_blocks, token_seq, positions, out, part_o, part_ml,
                                       T, H, K, P, window, scale, splits, status, stream);
            break;
        case 128:
            rc = launch_decode_tma<128>(map, fresh, q, block_table, max_blocks, token_seq, positions, out, part_o,
                                        part_ml, T, H, K, P, window, scale, splits, status, stream);
            break;
        case 256:
            rc = launch_decode_tma<256>(map, fresh, q, block_table, max_blocks, token_seq, positions, out, part_o,
                                        part_ml, T, H, K, P, window, scale, splits, status, stream);
            break;
        default:
            return AIR_ERR_BAD_ARGUMENT;
    }
    if (rc == 0 && splits > 1) rc = air_decode_combine(part_o, part_ml, token_seq, out, T, H, D, splits, stream);
    return rc;
}

}  // namespace air

// Arguments as air_decode_attention (attention_decode.cu), plus the number of pages of the cache
// (its first dimension) and the status word.
AIR_API int air_decode_attention_tma(const void* q, const void* cache, long long pages, const int* block_table,
                                     int max_blocks, const int* token_seq, const int* positions, void* out,
                                     float* part_o, float* part_ml, int T, int H, int K, int D, int P, int window,
                                     float scale, int splits, int* status, cudaStream_t stream) {
    return air::decode_attention_tma(air::FreshQkv{nullptr, 0, 0, nullptr, nullptr, nullptr}, q, cache, pages,
                                     block_table, max_blocks, token_seq, positions, out, part_o, part_ml, T, H, K, D, P,
                                     window, scale, splits, status, stream);
}

// The same from the q/k/v product's output instead of q: qkv float32 [parts][T][(H + 2 K) D] (partial sums that
// are added in order), bias float32 or null, table float32 [positions][D] (cos | sin: all of a head is
// rotated); write_kv = 0 where another run's layer has written this step's keys and values already.
AIR_API int air_decode_attention_tma_fresh(const float* qkv, int parts, const float* bias, const float* table,
                                           int write_kv, void* cache, long long pages, const int* block_table,
                                           int max_blocks, const int* token_seq, const int* positions, void* out,
                                           float* part_o, float* part_ml, int T, int H, int K, int D, int P,
                                           int window, float scale, int splits, int* status, cudaStream_t stream) {
    if (!qkv || !table || parts < 1 || ((uintptr_t)qkv & 15) || ((uintptr_t)bias & 15) || ((uintptr_t)table & 15))
        return AIR_ERR_BAD_ARGUMENT;
    const air::FreshQkv fresh{qkv, parts, (size_t)T * (size_t)(H + 2 * K) * (size_t)D, bias, table,
                              write_kv ? (__nv_bfloat16*)cache : nullptr};
    return air::decode_attention_tma(fresh, nullptr, cache, pages, block_table, max_blocks, token_seq, positions, out,
                                     part_o, part_ml, T, H, K, D, P, window, scale, splits, status, stream);
}

AIR_API int air_trace_set_attention_decode_tma(unsigned long long* buffer) { return air::set_trace_here(buffer); }
