// bfloat16 matrix product for a few tokens (up to 64) on the fifth-generation tensor cores, with the
// WEIGHTS as the M side of tcgen05.mma: C[T,N] = X[T,K] * W[N,K]^T is computed as its transpose,
// 128 rows of W (the accumulator's lanes) by NT = 16, 32 or 64 tokens (its columns).
//
// gemm_tc.cu puts the tokens on the M side, where an instruction always works on 128 rows: with 8
// tokens a k step of a 256-wide tile takes 128 cycles of the tensor pipe for 8 useful rows, and once
// the weights are in shared memory ahead of time (the block was resident while its predecessor
// ran) those cycles are what a decode step waits for: about 2.6 us per product with ten k-blocks
// per block.  Here a k step takes the time of reading 128 x 16 weights from shared memory (about
// 32 cycles).
//
// One persistent block per SM, 192 threads, as in gemm_tc.cu: warp 0 issues TMA loads (a tile of
// HALVES x 128 rows of W and the NT-row tile of X per stage, 128-byte swizzle, no multicast), warp 1
// issues tcgen05.mma (M 128, N NT, K 16; per k step one per half of the W tile, sharing the tile of
// X) into one of two sets of accumulators, warps 2-5 read a finished accumulator (thread = output
// feature, columns = tokens) and write the result, coalesced over the features.
//   EPI_F32 / EPI_BF16  store C
//   EPI_SILU            HALVES = 2 and W holds, per 256 rows, 128 rows of the gate projection followed
//                       by the 128 rows of the up projection for the same outputs: silu(gate) * up
//   EPI_PARTIAL         the k range is split over `splits` blocks; each writes C[split][T][N] (float32)
// Rows of X beyond T and rows of W beyond N are zero-filled by TMA.
// Every wait on an mbarrier is bounded; on giving up the block sets *status = 4 (as gemm_tc.cu).
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace air {

constexpr int TS_BK = 64;
constexpr int TS_THREADS = 192;

enum { TS_F32 = 0, TS_BF16 = 1, TS_SILU = 2, TS_PARTIAL = 3 };   // as in gemm_tc.cu

struct TsArgs {
    void* out;          // F32/PARTIAL: float [splits][T][N]; BF16: bf16 [T][N]; SILU: bf16 [T][N/2]
    int T, N, K;
    int splits;
    int* status;
    // Optional scale per token, applied to the accumulators before the epilogue: rsqrt(sum over ss_tiles of
    // ss[tile][t] / K + eps), the RMSNorm scale of an input whose rows came as x * weight without it
    // (add_prenorm_kernel in elementwise.cu writes such rows and the sums of squares).  ss == nullptr: none.
    const float* ss;
    int ss_tiles;
    float eps;
};

__host__ __device__ constexpr int ts_stages(int nt, int halves) {
    return 196 * 1024 / ((halves * 128 + nt) * TS_BK * 2) > 24 ? 24 : 196 * 1024 / ((halves * 128 + nt) * TS_BK * 2);
}
__host__ __device__ constexpr int ts_tmem_cols(int nt, int halves) {
    return 2 * halves * nt < 32 ? 32 : 2 * halves * nt;      // 32, 64, 128 or 256: a power of two
}

template <int NT>
__device__ __forceinline__ void ts_load_row(uint32_t taddr, float (&v)[NT]) {
    if constexpr (NT == 16) {
        uint32_t r[16];
        tmem_ld16(taddr, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
    } else {
#pragma unroll
        for (int c = 0; c < NT; c += 32) {
            uint32_t r[32];
            tmem_ld32(taddr + c, r);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[c + i] = __uint_as_float(r[i]);
        }
    }
}

template <int NT, int EPI, int HALVES>
__global__ void __launch_bounds__(TS_THREADS, 1)
gemm_tc_small_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                     const TsArgs args) {
    static_assert(EPI != TS_SILU || HALVES == 2, "the activation needs the gate half and the up half of a tile");
    constexpr int HALF_W = 128 * TS_BK * 2;           // 16 KB: 128 rows of W, 64 of k
    constexpr int STAGE_W = HALVES * HALF_W;
    constexpr int STAGE_X = NT * TS_BK * 2;
    constexpr int STAGES = ts_stages(NT, HALVES);
    constexpr int ACC_COLS = HALVES * NT;
    constexpr int TMEM_COLS = ts_tmem_cols(NT, HALVES);
    constexpr int TILE_N = HALVES * 128;               // rows of W per tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sw = smem;
    uint8_t* sx = smem + STAGES * STAGE_W;
    uint64_t* bars = (uint64_t*)(sx + STAGES * STAGE_X);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* row_scale = (float*)(tmem_slot + 2);       // [NT]

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (args.N + TILE_N - 1) / TILE_N;
    const int k_tiles = (args.K + TS_BK - 1) / TS_BK;
    const int k_per = (k_tiles + args.splits - 1) / args.splits;
    const int total = n_tiles * args.splits;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------ producer
            const uint32_t bytes = (uint32_t)(STAGE_W + STAGE_X);
            uint32_t stage = 0, phase = 0;
            bool first = true;
            trace_point(TR_GEMM_TC + 100);   // when this block became resident
            for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x) {
                const int split = tile % args.splits;
                const int n0 = (tile / args.splits) * TILE_N;
                const int k_begin = split * k_per, k_end = min(k_tiles, k_begin + k_per);
                int kt = k_begin;
                if (first) {
                    // The weights are written by no kernel: the first stages' tiles of W are fetched
                    // while the predecessor in the stream may still be running; the tiles of X (its
                    // output) follow once it has completed.
                    first = false;
                    const int pre = min(STAGES, k_end - k_begin);
                    for (int i = 0; i < pre; ++i) {
                        mbar_expect_tx(&full[i], bytes);
                        tma_load_2d(sw + i * STAGE_W, &map_w, (k_begin + i) * TS_BK, n0, &full[i]);
                    }
                    // (Asking further k-tiles into L2 here, as gemm_tc.cu does, was measured to cost 1.7 % of a
                    // decode step with this kernel: the ring is deep, and the requests delay the loads of
                    // the small kernels that run meanwhile.)
                    pdl_wait();
                    trace_point(TR_GEMM_TC);
                    for (int i = 0; i < pre; ++i) tma_load_2d(sx + i * STAGE_X, &map_x, (k_begin + i) * TS_BK, 0, &full[i]);
                    kt = k_begin + pre;
                    if (pre == STAGES) phase = 1; else stage = pre;
                }
                for (; kt < k_end; ++kt) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;
                    mbar_expect_tx(&full[stage], bytes);
                    tma_load_2d(sw + stage * STAGE_W, &map_w, kt * TS_BK, n0, &full[stage]);
                    tma_load_2d(sx + stage * STAGE_X, &map_x, kt * TS_BK, 0, &full[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------- MMA issuer: the warp runs together, an
        // elected lane issues (see gemm_tc.cu)
        constexpr uint32_t idesc = umma_idesc(128, NT);
        const uint64_t dw0 = umma_desc(smem_u32(sw)), dx0 = umma_desc(smem_u32(sx));
        uint32_t stage = 0, phase = 0, it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok && !*abort_flag; tile += gridDim.x, ++it) {
            const int split = tile % args.splits;
            const int k_begin = split * k_per, k_end = min(k_tiles, k_begin + k_per);
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d = tmem_base + acc * ACC_COLS;
            for (int kt = k_begin; kt < k_end; ++kt) {
                // (a stage that is already there costs one try; the bounded loop only where the issuer has to wait)
                if (!mbar_try_wait(&full[stage], phase)) ok = __all_sync(0xffffffffu, mbar_wait(&full[stage], phase, abort_flag));
                if (!ok) break;
                tc_fence_after();
                const uint64_t dw = dw0 + (uint64_t)(stage * (STAGE_W >> 4));
                const uint64_t dx = dx0 + (uint64_t)(stage * (STAGE_X >> 4));
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < TS_BK / 16; ++k)
#pragma unroll
                        for (int hf = 0; hf < HALVES; ++hf)
                            umma_bf16(d + hf * NT, dw + (uint64_t)(hf * (HALF_W >> 4)) + 2 * k, dx + 2 * k, idesc,
                                      (kt > k_begin || k > 0) ? 1u : 0u);
                    umma_commit(&empty[stage]);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok && elect_one()) umma_commit(&acc_full[acc]);
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------- epilogue: warps 2..5, thread = feature
        pdl_wait();   // nothing is written before the predecessor has completed
        const int quarter = warp & 3;                     // the 32 lanes of tensor memory this warp may read
        const int r = quarter * 32 + lane;                // row of the tile's half
        if (args.ss) {
            // the tokens' norm scales, worked out while the weights stream: eight loads in flight at a time,
            // the sums added in the order of the tiles
            if (r < NT) {
                float total = 0.f;
                if (r < args.T) {
                    for (int base = 0; base < args.ss_tiles; base += 8) {
                        float part[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            part[i] = base + i < args.ss_tiles ? args.ss[(size_t)(base + i) * args.T + r] : 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) total += part[i];
                    }
                }
                row_scale[r] = r < args.T ? rsqrtf(total / (float)args.K + args.eps) : 0.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++it) {
            const int split = tile % args.splits;
            const int n0 = (tile / args.splits) * TILE_N;
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            if constexpr (EPI == TS_SILU) {
                float gate[NT], up[NT];
                ts_load_row<NT>(taddr, gate);
                ts_load_row<NT>(taddr + NT, up);
                if (args.ss) {
#pragma unroll
                    for (int t = 0; t < NT; ++t) { gate[t] *= row_scale[t]; up[t] *= row_scale[t]; }
                }
                const int col = n0 / 2 + r;
                if (col < args.N / 2) {
                    __nv_bfloat16* out = (__nv_bfloat16*)args.out + col;
#pragma unroll
                    for (int t = 0; t < NT; ++t)
                        if (t < args.T)
                            out[(size_t)t * (args.N / 2)] = __float2bfloat16_rn(gate[t] / (1.f + expf(-gate[t])) * up[t]);
                }
            } else {
#pragma unroll
                for (int hf = 0; hf < HALVES; ++hf) {
                    float v[NT];
                    ts_load_row<NT>(taddr + hf * NT, v);
                    if (args.ss) {
#pragma unroll
                        for (int t = 0; t < NT; ++t) v[t] *= row_scale[t];
                    }
                    const int col = n0 + hf * 128 + r;
                    if (col < args.N) {
                        if constexpr (EPI == TS_BF16) {
                            __nv_bfloat16* out = (__nv_bfloat16*)args.out + col;
#pragma unroll
                            for (int t = 0; t < NT; ++t)
                                if (t < args.T) out[(size_t)t * args.N] = __float2bfloat16_rn(v[t]);
                        } else {
                            float* out = (float*)args.out + (size_t)split * args.T * args.N + col;
#pragma unroll
                            for (int t = 0; t < NT; ++t)
                                if (t < args.T) out[(size_t)t * args.N] = v[t];
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
    }

    // ---------------------------------------------------------- leaving
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // copies that were issued may still be on their way: give them time before the block ends
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 4);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// A tensor map of a row-major bf16 matrix [rows, cols] with boxes of box_rows x 64 and 128-byte swizzle.
static int ts_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    return tensor_map_2d(map, base, rows, cols, box_rows);
}

template <int NT, int EPI, int HALVES>
static int ts_launch(const CUtensorMap& mw, const CUtensorMap& mx, const TsArgs& args, int blocks, cudaStream_t stream) {
    constexpr int STAGES = ts_stages(NT, HALVES);
    // always more than half of an SM's shared memory, so that two blocks never share an SM (and its
    // tensor memory)
    const size_t smem = 1024 + (size_t)STAGES * (HALVES * 128 + NT) * TS_BK * 2 + 16 * STAGES + 256 + 4 * NT;
    const size_t request = smem < 120 * 1024 ? 120 * 1024 : smem;
    auto kernel = gemm_tc_small_kernel<NT, EPI, HALVES>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)request);
    if (e != cudaSuccess) return (int)e;
    return launch(kernel, blocks, TS_THREADS, request, stream, mw, mx, args);
}

template <int NT, int HALVES>
static int ts_dispatch_epi(int epi, const CUtensorMap& mw, const CUtensorMap& mx, const TsArgs& args, int blocks,
                           cudaStream_t stream) {
    switch (epi) {
        case TS_F32: return ts_launch<NT, TS_F32, HALVES>(mw, mx, args, blocks, stream);
        case TS_BF16: return ts_launch<NT, TS_BF16, HALVES>(mw, mx, args, blocks, stream);
        case TS_SILU:
            if constexpr (HALVES == 2) return ts_launch<NT, TS_SILU, HALVES>(mw, mx, args, blocks, stream);
            return AIR_ERR_BAD_ARGUMENT;
        case TS_PARTIAL: return ts_launch<NT, TS_F32, HALVES>(mw, mx, args, blocks, stream);
        default: return AIR_ERR_BAD_ARGUMENT;
    }
}

template <int HALVES>
static int ts_dispatch_tokens(int nt, int epi, const CUtensorMap& mw, const CUtensorMap& mx, const TsArgs& args,
                              int blocks, cudaStream_t stream) {
    switch (nt) {
        case 16: return ts_dispatch_epi<16, HALVES>(epi, mw, mx, args, blocks, stream);
        case 32: return ts_dispatch_epi<32, HALVES>(epi, mw, mx, args, blocks, stream);
        default: return ts_dispatch_epi<64, HALVES>(epi, mw, mx, args, blocks, stream);
    }
}

}  // namespace air

// x [T, K] bf16 with T <= 64, w [N, K] bf16 (for epi 2: per 256 rows 128 of gate, then 128 of up), K % 8 == 0.
// out as TsArgs.out.  tile_rows: 128 or 256 rows of W per tile (256 for epi 2).  max_blocks: the number of
// SMs to use (0: all).
AIR_API int air_gemm_tc_small(const void* x, const void* w, void* out, int T, int N, int K, int tile_rows, int epi,
                              int splits, int max_blocks, int* status, const float* ss, int ss_tiles, float eps,
                              cudaStream_t stream) {
    using namespace air;
    if (T <= 0 || N <= 0) return 0;
    if (T > 64 || K <= 0 || K % 8 || splits < 1 || (splits > 1 && epi != TS_PARTIAL) || ((uintptr_t)x & 15) ||
        ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || (tile_rows != 128 && tile_rows != 256))
        return AIR_ERR_BAD_ARGUMENT;
    if (epi == TS_SILU && (tile_rows != 256 || N % 256)) return AIR_ERR_BAD_ARGUMENT;
    const int k_tiles = (K + TS_BK - 1) / TS_BK;
    // every part of the k range must hold at least one k-tile (an accumulator that no product wrote is not zero)
    if (splits > k_tiles || (long long)(splits - 1) * ((k_tiles + splits - 1) / splits) >= k_tiles)
        return AIR_ERR_BAD_ARGUMENT;
    const int nt = T > 32 ? 64 : (T > 16 ? 32 : 16);
    CUtensorMap mw, mx;
    int rc = ts_make_map(&mw, w, N, K, tile_rows);
    if (rc) return rc;
    rc = ts_make_map(&mx, x, T, K, nt);
    if (rc) return rc;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_blocks > 0 && max_blocks < sms) sms = max_blocks;
    const long long tiles = (long long)((N + tile_rows - 1) / tile_rows) * splits;
    const int blocks = (int)(tiles < sms ? tiles : sms);
    if (ss && ss_tiles < 1) return AIR_ERR_BAD_ARGUMENT;
    TsArgs args{out, T, N, K, splits, status, ss, ss_tiles, eps};
    if (tile_rows == 256) return ts_dispatch_tokens<2>(nt, epi, mw, mx, args, blocks, stream);
    return ts_dispatch_tokens<1>(nt, epi, mw, mx, args, blocks, stream);
}

AIR_API int air_trace_set_gemm_tc_small(unsigned long long* buffer) { return air::set_trace_here(buffer); }
