// bfloat16 matrix product on the fifth-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T with
// float32 accumulation in tensor memory and the TOKENS as the M side of the instruction, with the
// epilogues that the decoder wants fused in.  It serves any number of rows; for up to 64 tokens and
// tiles of 128 or 256 rows of W the engine takes gemm_tc_small.cu (the weights as the M side) instead.
//
// One persistent block per SM, 192 threads:
//   warp 0   one lane issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//            of an up to 128 x 64 tile of A and a BN x 64 tile of W per stage into a ring of stages;
//   warp 1   allocates tensor memory; an elected lane issues tcgen05.mma (M = 128, N = BN, K = 16, four
//            per stage) into one of two accumulators and commits the stage's "empty" barrier;
//   warps 2-5  read a finished accumulator with tcgen05.ld (each thread one row = one token, 32
//            columns at a time) and write the result, while the next tile is being multiplied.
// A thread of the epilogue holds a whole row of the tile, so what the decoder does per token and
// output column pair is done in registers:
//   EPI_F32 / EPI_BF16  store C
//   EPI_SILU            W holds, per tile, BN/2 rows of the gate projection followed by the BN/2 rows
//                       of the up projection for the same outputs: out = silu(gate) * up as bfloat16
//   EPI_PARTIAL         the k range is split over `splits` blocks; each writes its partial sums to
//                       C[split][M][N] (float32), which the consumer (norm or rotary kernel) adds up
//                       in a fixed order.  This keeps all 148 SMs streaming weights when M is small.
// With many tokens (AR = 256) a block's tile is 256 x 256: two products per k step share the tile of W,
// each with its own 128 rows of A and its own accumulator (all 512 columns of tensor memory, so the
// epilogue, by eight warps, is not overlapped with the next tile).  An SM takes 64 bytes a cycle from
// L2; a 128 x 256 tile needs 48 KB per 512 cycles of products and so waits for its operands a third of
// the time, a 256 x 256 tile needs 64 KB per 1024 cycles.
// Rows of A beyond M are not loaded (the box of A is only as tall as needed); the accumulator rows
// they would feed hold garbage that is never read.  Rows of W beyond N are zero-filled by TMA.
//
// Every wait on an mbarrier is bounded: when a wait gives up, the block sets a flag, every role
// leaves its loop, outstanding copies are given time to land, tensor memory is freed and *status
// is set to 4.  The host reads *status with the step's other error codes.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace air {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_THREADS = 192;       // 320 with AR = 256: eight epilogue warps

enum { EPI_F32 = 0, EPI_BF16 = 1, EPI_SILU = 2, EPI_PARTIAL = 3 };

struct TcArgs {
    void* out;          // EPI_F32/PARTIAL: float [splits][M][N]; EPI_BF16: bf16 [M][N]; EPI_SILU: bf16 [M][N/2]
    int M, N, K;
    int a_rows;         // height of A's TMA box: 16, 64, 128 or 256
    int splits;         // parts of the k range (1 unless EPI_PARTIAL)
    int prefetch;       // further k-tiles of W that a block asks into L2 before its predecessor has ended
    int* status;
};

// Stages of the ring for a tile width and a height of A's box: what fits in 196 KB, at most 24.
__host__ __device__ constexpr int tc_stages(int bn, int ar) {
    return 196 * 1024 / ((ar + bn) * TC_BK * 2) > 24 ? 24 : 196 * 1024 / ((ar + bn) * TC_BK * 2);
}

// BN: tile width.  AR: rows of A that are loaded (16, 64, 128, or 256 for two row halves): with few tokens a stage is small,
// so the ring is deep and most of a block's share of W is under way before the predecessor ends.
// The MMA always reads 128 rows from the stage's address; what lies beyond AR rows is other tiles'
// data, feeding accumulator rows that are never read.
template <int BN, int EPI, int AR>
__global__ void __launch_bounds__(AR == 256 ? 320 : TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const TcArgs args) {
    constexpr int STAGE_A = AR * TC_BK * 2;
    constexpr int STAGE_W = BN * TC_BK * 2;
    constexpr int STAGES = tc_stages(BN, AR);
    static_assert(STAGES >= 2 && STAGES * STAGE_W >= TC_BM * TC_BK * 2, "the MMA's 128-row read must stay inside");
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;       // two accumulators; a power of two
    constexpr int HALVES = AR == 256 ? 2 : 1;                  // row halves of a tile, one accumulator each
    constexpr int NACC = AR == 256 ? 1 : 2;                    // tiles whose accumulators fit at a time
    constexpr int TILE_M = HALVES * TC_BM;
    constexpr int EPI_WARPS = 4 * HALVES;
    static_assert(AR != 256 || BN == 256, "two row halves take all of tensor memory at BN = 256 only");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sa = smem;
    uint8_t* sw = smem + STAGES * STAGE_A;
    uint64_t* bars = (uint64_t*)(sw + STAGES * STAGE_W);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (args.M + TILE_M - 1) / TILE_M;
    const int n_tiles = (args.N + BN - 1) / BN;
    const int k_tiles = (args.K + TC_BK - 1) / TC_BK;
    const int k_per = (k_tiles + args.splits - 1) / args.splits;
    const int total = m_tiles * n_tiles * args.splits;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------ producer
            const uint32_t bytes = (uint32_t)(STAGE_A + STAGE_W);
            uint32_t stage = 0, phase = 0;
            bool first = true;
            trace_point(TR_GEMM_TC + 100);   // when this block became resident
            for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x) {
                const int split = tile % args.splits;
                const int mn = tile / args.splits;
                const int m0 = (mn % m_tiles) * TILE_M, n0 = (mn / m_tiles) * BN;
                const int k_begin = split * k_per, k_end = min(k_tiles, k_begin + k_per);
                int kt = k_begin;
                if (first) {
                    // The weights are written by no kernel: the first stages' tiles of W are fetched
                    // while the predecessor in the stream may still be running; the tiles of A (its
                    // output) follow once it has completed.
                    first = false;
                    const int pre = min(STAGES, k_end - k_begin);
                    for (int i = 0; i < pre; ++i) {
                        mbar_expect_tx(&full[i], bytes);
                        tma_load_2d(sw + i * STAGE_W, &map_w, (k_begin + i) * TC_BK, n0, &full[i]);
                    }
                    const int ahead = min(pre + args.prefetch, k_end - k_begin);
                    for (int i = pre; i < ahead; ++i) tma_prefetch_l2(&map_w, (k_begin + i) * TC_BK, n0);
                    pdl_wait();
                    trace_point(TR_GEMM_TC);
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d(sa + i * STAGE_A, &map_a, (k_begin + i) * TC_BK, m0, &full[i]);
                    kt = k_begin + pre;
                    if (pre == STAGES) phase = 1; else stage = pre;
                }
                for (; kt < k_end; ++kt) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;
                    mbar_expect_tx(&full[stage], bytes);
                    tma_load_2d(sa + stage * STAGE_A, &map_a, kt * TC_BK, m0, &full[stage]);
                    tma_load_2d(sw + stage * STAGE_W, &map_w, kt * TC_BK, n0, &full[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        {
            // ------------------------------------------------ MMA issuer.  The warp runs together and
            // an elected lane issues: the operands then stay in uniform registers.  tcgen05.mma is all
            // but synchronous for its issuer, so every instruction between two products is time in
            // which the tensor cores wait; this loop is kept as short as it can be.
            constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
            const uint64_t da0 = umma_desc(smem_u32(sa)), dw0 = umma_desc(smem_u32(sw));
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok && !*abort_flag; tile += gridDim.x, ++it) {
                const int split = tile % args.splits;
                const int k_begin = split * k_per, k_end = min(k_tiles, k_begin + k_per);
                const uint32_t acc = it % NACC, acc_phase = (it / NACC) & 1;
                // (a last row tile that holds at most 128 rows needs no second product per k step: 544 rows
                // are two tiles of 256 and one of 32, and that one costs half)
                const int halves_here =
                    (HALVES == 2 && ((tile / args.splits) % m_tiles) * TILE_M + TC_BM >= args.M) ? 1 : HALVES;
                ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + acc * BN;
                for (int kt = k_begin; kt < k_end; ++kt) {
                    // (a stage that is already there costs one try; the bounded loop only where the issuer has to wait)
                    if (!mbar_try_wait(&full[stage], phase)) ok = __all_sync(0xffffffffu, mbar_wait(&full[stage], phase, abort_flag));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // (the start address field counts 16 bytes)
                    const uint64_t da = da0 + (uint64_t)(stage * (STAGE_A >> 4));
                    const uint64_t dw = dw0 + (uint64_t)(stage * (STAGE_W >> 4));
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)
#pragma unroll
                            for (int hf = 0; hf < HALVES; ++hf)
                                if (hf < halves_here)
                                    umma_bf16(d + hf * BN, da + (uint64_t)(hf * (TC_BM * TC_BK * 2 >> 4)) + 2 * k, dw + 2 * k,
                                              idesc, (kt > k_begin || k > 0) ? 1u : 0u);
                        umma_commit(&empty[stage]);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok && elect_one()) umma_commit(&acc_full[acc]);
                __syncwarp();
            }
        }
    } else {
        // ---------------------------------------------------- epilogue: warps 2..5
        pdl_wait();   // nothing is written before the predecessor has completed
        const int quarter = warp & 3;                     // the 32 lanes of tensor memory this warp may read
        const int half = (warp - 2) >> 2;                 // which 128 rows of the tile (0 unless AR = 256)
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++it) {
            const int split = tile % args.splits;
            const int mn = tile / args.splits;
            const int m0 = (mn % m_tiles) * TILE_M + half * TC_BM, n0 = (mn / m_tiles) * BN;
            const uint32_t acc = it % NACC, acc_phase = (it / NACC) & 1;
            if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const bool warp_has_rows = m0 + quarter * 32 < args.M;
            if (warp_has_rows) {
                const uint32_t taddr = tmem_base + (acc + half) * BN + ((uint32_t)(quarter * 32) << 16);
                if (EPI == EPI_SILU) {
                    __nv_bfloat16* out = (__nv_bfloat16*)args.out + (size_t)row * (args.N / 2) + n0 / 2;
#pragma unroll 1
                    for (int c = 0; c < BN / 2; c += 32) {
                        uint32_t gate[32], up[32];
                        tmem_ld32(taddr + c, gate);
                        tmem_ld32(taddr + BN / 2 + c, up);
                        if (row < args.M) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                if (n0 / 2 + c + j >= args.N / 2) break;
                                float y[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const float g = __uint_as_float(gate[j + e]), u = __uint_as_float(up[j + e]);
                                    y[e] = g / (1.f + expf(-g)) * u;
                                }
                                store4(out + c + j, *(const float(*)[4])&y[0]);
                                store4(out + c + j + 4, *(const float(*)[4])&y[4]);
                            }
                        }
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < BN; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(taddr + c, v);
                        if (row < args.M) {
                            if (EPI == EPI_BF16) {
                                __nv_bfloat16* out = (__nv_bfloat16*)args.out + (size_t)row * args.N + n0 + c;
#pragma unroll
                                for (int j = 0; j < 32; j += 4) {
                                    if (n0 + c + j >= args.N) break;
                                    const float y[4] = {__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                        __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])};
                                    store4(out + j, y);
                                }
                            } else {
                                float* out = (float*)args.out + ((size_t)split * args.M + row) * args.N + n0 + c;
#pragma unroll
                                for (int j = 0; j < 32; j += 4) {
                                    if (n0 + c + j >= args.N) break;
                                    *reinterpret_cast<float4*>(out + j) =
                                        make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                    __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                                }
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
    }

    // ---------------------------------------------------------- leaving
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        // copies that were issued may still be on their way: give them time before the block ends
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 4);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------ host side
// A tensor map of a row-major bf16 matrix [rows, cols] with boxes of box_rows x 64 and 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    return tensor_map_2d(map, base, rows, cols, box_rows);
}

template <int BN, int EPI, int AR>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, const TcArgs& args, int blocks, cudaStream_t stream) {
    constexpr int STAGES = tc_stages(BN, AR);
    // always more than half of an SM's shared memory, so that two blocks never share an SM (and its
    // 512 columns of tensor memory)
    const size_t smem = 1024 + (size_t)STAGES * (AR + BN) * TC_BK * 2 + 16 * STAGES + 256;
    const size_t request = smem < 120 * 1024 ? 120 * 1024 : smem;
    auto kernel = gemm_tc_kernel<BN, EPI, AR>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)request);
    if (e != cudaSuccess) return (int)e;
    return launch(kernel, blocks, AR == 256 ? 320 : TC_THREADS, request, stream, ma, mw, args);
}

template <int BN, int AR>
static int dispatch_epi(int epi, const CUtensorMap& ma, const CUtensorMap& mw, const TcArgs& args, int blocks,
                        cudaStream_t stream) {
    switch (epi) {
        case EPI_F32: return launch_tc<BN, EPI_F32, AR>(ma, mw, args, blocks, stream);
        case EPI_BF16: return launch_tc<BN, EPI_BF16, AR>(ma, mw, args, blocks, stream);
        case EPI_SILU:
            if constexpr (BN >= 64) return launch_tc<BN, EPI_SILU, AR>(ma, mw, args, blocks, stream);
            return AIR_ERR_BAD_ARGUMENT;
        case EPI_PARTIAL: return launch_tc<BN, EPI_PARTIAL, AR>(ma, mw, args, blocks, stream);
        default: return AIR_ERR_BAD_ARGUMENT;
    }
}

template <int BN>
static int dispatch_rows(int a_rows, int epi, const CUtensorMap& ma, const CUtensorMap& mw, const TcArgs& args,
                         int blocks, cudaStream_t stream) {
    switch (a_rows) {
        case 16: return dispatch_epi<BN, 16>(epi, ma, mw, args, blocks, stream);
        case 64: return dispatch_epi<BN, 64>(epi, ma, mw, args, blocks, stream);
        case 256:
            if constexpr (BN == 256) return dispatch_epi<BN, 256>(epi, ma, mw, args, blocks, stream);
            return AIR_ERR_BAD_ARGUMENT;
        default: return dispatch_epi<BN, 128>(epi, ma, mw, args, blocks, stream);
    }
}

}  // namespace air

// a [M, K] bf16, w [N, K] bf16 (for epi 2: gate and up rows interleaved in blocks of bn / 2), K % 8 == 0.
// out as TcArgs.out.  bn: 32, 64, 128 or 256.  max_blocks: the number of SMs to use (0: all).
AIR_API int air_gemm_tc(const void* a, const void* w, void* out, int M, int N, int K, int bn, int epi, int splits,
                        int max_blocks, int* status, cudaStream_t stream) {
    using namespace air;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || splits < 1 || (splits > 1 && epi != EPI_PARTIAL) || ((uintptr_t)a & 15) ||
        ((uintptr_t)w & 15) || ((uintptr_t)out & 15))
        return AIR_ERR_BAD_ARGUMENT;
    if (epi == EPI_SILU && (bn < 64 || N % bn || (N / 2) % 8)) return AIR_ERR_BAD_ARGUMENT;
    if (epi != EPI_SILU && N % 4) return AIR_ERR_BAD_ARGUMENT;
    const int k_tiles = (K + TC_BK - 1) / TC_BK;
    // every part of the k range must hold at least one k-tile (an accumulator that no product wrote is not zero)
    if (splits > k_tiles || (long long)(splits - 1) * ((k_tiles + splits - 1) / splits) >= k_tiles)
        return AIR_ERR_BAD_ARGUMENT;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_blocks > 0 && max_blocks < sms) sms = max_blocks;
    // (256-row tiles where they still leave three quarters of the SMs a tile each)
    const bool tall = bn == 256 && M >= 512 && (long long)((M + 255) / 256) * ((N + 255) / 256) * 4 >= 3ll * sms;
    const int a_rows = tall ? 256 : M > 64 ? 128 : (M > 16 ? 64 : 16);
    const int tile_m = a_rows == 256 ? 256 : TC_BM;
    CUtensorMap ma, mw;
    int rc = make_map(&ma, a, M, K, a_rows);
    if (rc) return rc;
    rc = make_map(&mw, w, N, K, bn);
    if (rc) return rc;
    const long long tiles = (long long)((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn) * splits;
    const int blocks = (int)(tiles < sms ? tiles : sms);
    // With few rows the product is a stream of weights: while the predecessor runs, each block asks
    // its share of up to 40 MB of them into L2 (the L2 holds 126 MB).
    const int prefetch = M <= 64 ? (int)((40ll << 20) / blocks / (bn * TC_BK * 2)) : 0;
    TcArgs args{out, M, N, K, a_rows, splits, prefetch, status};
    switch (bn) {
        case 32: return dispatch_rows<32>(a_rows, epi, ma, mw, args, blocks, stream);
        case 64: return dispatch_rows<64>(a_rows, epi, ma, mw, args, blocks, stream);
        case 128: return dispatch_rows<128>(a_rows, epi, ma, mw, args, blocks, stream);
        case 256: return dispatch_rows<256>(a_rows, epi, ma, mw, args, blocks, stream);
        default: return AIR_ERR_BAD_ARGUMENT;
    }
}

AIR_API int air_trace_set_gemm_tc(unsigned long long* buffer) { return air::set_trace_here(buffer); }
