// Choosing the next token on the device: the lowest index of the maximum (greedy), or an
// index drawn from softmax(logits / temperature), optionally cut to the k largest logits and then
// to the shortest prefix of the descending order whose weights reach the share p (AIR's sampler,
// src/runtime/sampling.cpp:9-62: top-k after a stable descending sort, then top-p, at least one kept),
// with a uniform number that the host supplies for the row.  One block per row of logits [R, V]
// (float32).  The row is never sorted.  With a cut, the largest logits are found by a selection over
// the logits' bit patterns, one digit of 8 bits per pass with a histogram, which stops as soon as the
// digits so far leave no more than CANDIDATES indices; these are gathered into shared memory and
// sorted there (by logit, ties by index, as a stable sort leaves them), cut, and the draw walks them
// in that order, as AIR's does.  Where that is not enough (k above CANDIDATES, a share that the
// candidates do not reach, more ties than fit) the general path finds both cuts by the same kind of
// selection over the whole row and walks the kept indices in index order; so does a draw without a
// cut.  That gives AIR's distribution but, for the same uniform number, not the token that AIR's walk
// in descending order gives (the host sampler does that).  Weights are integers, exp((x - max) / T) *
// 2^36 cut off, so that every sum is exact and independent of the order in which it is taken: what is
// kept and what is drawn depends on the row, the options and the uniform number alone.
#include "common.cuh"

namespace air {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;
constexpr float MASS_ONE = 2147483648.f;         // 2^31: the largest logit's weight
constexpr int NO_TIE_LIMIT = 0x7fffffff;
constexpr int CANDIDATES = 2048;                 // two per thread
constexpr int COUNT_COLUMNS = 16;                // of a bin's counter: lanes l and l + 16 share one
typedef unsigned long long u64;

union SampleScratch {
    struct {
        union {
            uint32_t count[256][COUNT_COLUMNS];  // the candidates' selection: its histogram
            u64 upto[CANDIDATES];                // cumulative weights of the sorted candidates
        };
        u64 candidate[CANDIDATES];               // order_key << 32 | ~index: descending = by logit, ties by index
    } few;
    u64 hist[256][COUNT_COLUMNS];                // the general path's histogram
};

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// A float's bits as an unsigned number of the same order.
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The sum over the warp of values up to 2^31.
__device__ __forceinline__ u64 round_sum(u64 m) {
    const unsigned lo = __reduce_add_sync(0xffffffffu, (unsigned)(m & 0xffffu));
    const unsigned hi = __reduce_add_sync(0xffffffffu, (unsigned)(m >> 16));
    return lo + ((u64)hi << 16);
}

// temperature == nullptr or temperature[r] <= 0: greedy.  Otherwise the drawn index is the
// first kept i (in index order) with sum_{kept j<=i} w_j >= u * sum_{kept j} w_j, w_j = exp((x_j - max) / T).
// With slots and last_token the chosen index is also stored at last_token[slots[r]], where the
// embedding kernel of the next step finds it.
// A row whose maximum is not finite sets *status (AIR flags non-finite logits on the device,
// src/cuda/cuda_backend.cu:621-624).
//
// Each warp owns a run of consecutive indices and its lanes take them 32 at a time, so that loads are
// whole lines and "in index order" is (warp, round, lane): a tie's rank is the ties of earlier warps
// (one small sum), of earlier rounds (a running count) and of lower lanes (a ballot).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, const int* __restrict__ top_k, const float* __restrict__ top_p,
              int* __restrict__ out, const int* __restrict__ slots, int* __restrict__ last_token, int V,
              int* status) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float s_max;
    __shared__ int s_arg;
    __shared__ SampleScratch scratch;
    __shared__ int bin_count[256];
    __shared__ u64 bin_mass[256];
    __shared__ int s_candidates, s_gathered, s_keep;
    __shared__ u64 warp_mass[SAMPLE_WARPS];
    __shared__ int warp_ties[SAMPLE_WARPS];
    __shared__ uint32_t s_prefix;
    __shared__ u64 s_need;
    pdl_enter(TR_SAMPLE);
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * V;

    float v = -INFINITY;
    int idx = 0x7fffffff;
    bool bad = false;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float xi = x[i];
        if (!(fabsf(xi) <= 3.4e38f)) bad = true;
        argmax_combine(v, idx, xi, i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(v, idx, ov, oi);
    }
    if (__syncthreads_or(bad) && tid == 0 && status) atomicExch(status, 3);
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = sv[lane];
        idx = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_combine(v, idx, ov, oi);
        }
        if (lane == 0) {
            s_max = v;
            s_arg = idx == 0x7fffffff ? 0 : idx;
        }
    }
    __syncthreads();
    const float temp = temperature ? temperature[r] : 0.f;
    const int arg = s_arg;
    if (tid == 0) {                                  // the greedy answer; a draw below replaces it
        out[r] = arg;
        if (slots && last_token) last_token[slots[r]] = arg;
    }
    if (!(temp > 0.f)) return;

    const float inv_t = 1.f / temp, mx = s_max;
    auto mass_of = [&](float xi) { return (u64)__float2uint_rz(__expf((xi - mx) * inv_t) * MASS_ONE); };
    const int seg = ((V + SAMPLE_WARPS - 1) / SAMPLE_WARPS + 31) & ~31;
    const int seg_begin = min(V, warp * seg), seg_end = min(V, seg_begin + seg);
    const unsigned lower = (1u << lane) - 1u;

    // The kept set is {key > cut} and the first `ties` indices with key == cut.  Without a cut: everything.
    uint32_t cut = 0;
    int ties = NO_TIE_LIMIT;
    int ties_before = 0;          // indices with key == cut in the warps before this one

    // f(i, x_i, key_i, kept_i) for this warp's indices in index order; every lane calls f in every round
    // (kept_i is false beyond the end).
    auto each = [&](auto&& f) {
        int run = ties_before;
        float ahead[4];                               // the next four rounds' loads are in flight during these four
#pragma unroll
        for (int u = 0; u < 4; ++u) ahead[u] = seg_begin + 32 * u + lane < seg_end ? x[seg_begin + 32 * u + lane] : 0.f;
        for (int base = seg_begin; base < seg_end; base += 128) {
            float xs[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                xs[u] = ahead[u];
                ahead[u] = base + 128 + 32 * u + lane < seg_end ? x[base + 128 + 32 * u + lane] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (base + 32 * u >= seg_end) break;
                const int i = base + 32 * u + lane;
                const bool valid = i < seg_end;
                const float xi = xs[u];
                const uint32_t key = order_key(xi);
                const bool tie = valid && key == cut;
                const unsigned tb = __ballot_sync(0xffffffffu, tie);
                const bool in = valid && (key > cut || (tie && run + __popc(tb & lower) < ties));
                run += __popc(tb);
                f(i, xi, key, in);
            }
        }
    };
    auto count_ties_before = [&]() {                  // after `cut` changed
        int mine = 0;
        for (int base = seg_begin; base < seg_end; base += 32) {
            const int i = base + lane;
            mine += __popc(__ballot_sync(0xffffffffu, i < seg_end && order_key(x[min(i, seg_end - 1)]) == cut));
        }
        __syncthreads();
        if (lane == 0) warp_ties[warp] = mine;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_ties[w];
        ties_before = before;
    };
    // The largest key K with measure{kept i: key_i >= K} >= need, where the measure counts (weighted = false)
    // or adds weights; `need` must not exceed the measure of all that is kept.  Leaves in `need` what the
    // indices with key K have to supply.  One digit of 8 bits per pass, from the top.
    auto select = [&](bool weighted, u64& need) {
        uint32_t prefix = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 256 * COUNT_COLUMNS; i += SAMPLE_THREADS) (&scratch.hist[0][0])[i] = 0;
            if (tid == 0) { s_prefix = prefix << 8; s_need = need; }
            __syncthreads();
            each([&](int, float xi, uint32_t key, bool in) {
                if (in && (shift == 24 || (key >> (shift + 8)) == prefix))
                    atomicAdd(&scratch.hist[(key >> shift) & 255u][lane & (COUNT_COLUMNS - 1)],
                              weighted ? mass_of(xi) : 1ull);
            });
            __syncthreads();
            if (tid < 256) {
                u64 c = 0;
#pragma unroll
                for (int j = 0; j < COUNT_COLUMNS; ++j) c += scratch.hist[tid][j];
                bin_mass[tid] = c;
            }
            __syncthreads();
            if (warp == 0) {                          // lane l: bins 8 l .. 8 l + 7; the digit from the top
                u64 local = 0;
#pragma unroll
                for (int b = 0; b < 8; ++b) local += bin_mass[lane * 8 + b];
                u64 suffix = local;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const u64 n = __shfl_down_sync(0xffffffffu, suffix, o);
                    if (lane + o < 32) suffix += n;
                }
                const u64 above = suffix - local;
                if (above < need && need <= above + local) {
                    u64 cum = above;
                    for (int b = 7; b >= 0; --b) {
                        const u64 h = bin_mass[lane * 8 + b];
                        if (cum + h >= need) {
                            s_prefix = (prefix << 8) | (uint32_t)(lane * 8 + b);
                            s_need = need - cum;
                            break;
                        }
                        cum += h;
                    }
                }
            }
            __syncthreads();
            prefix = s_prefix;
            need = s_need;
            __syncthreads();
        }
        return prefix;
    };
    auto kept_mass = [&](u64& before, u64& total) {  // of the warps before this one, and of all
        u64 mine = 0;
        if (cut == 0 && ties == NO_TIE_LIMIT) {       // everything is kept
#pragma unroll 8
            for (int i = seg_begin + lane; i < seg_end; i += 32) mine += mass_of(x[i]);
        } else {
            each([&](int, float xi, uint32_t, bool in) { if (in) mine += mass_of(xi); });
        }
        mine = warp_sum_u64(mine);
        __syncthreads();
        if (lane == 0) warp_mass[warp] = mine;
        __syncthreads();
        before = 0;
        total = 0;
        for (int w = 0; w < SAMPLE_WARPS; ++w) {
            const u64 t = warp_mass[w];
            if (w < warp) before += t;
            total += t;
        }
        return mine;
    };

    const int k = top_k ? top_k[r] : 0;
    const float share = top_p ? top_p[r] : 1.f;
    const bool cut_k = k > 0 && k < V, cut_p = share < 1.f;

    // ---- with a cut: candidates in shared memory ----
    if ((cut_k || cut_p) && (!cut_k || k <= CANDIDATES)) {
        // The `want` largest or somewhat more: digits of the want-th largest key from the top, until the
        // indices at or above the digits so far are no more than CANDIDATES.
        const int want = cut_k ? k : min(V, CANDIDATES / 2);
        uint32_t prefix = 0;
        int need = want, shift = 24;
        u64 all_mass = 0;                             // without top-k the share is of the whole row's weight
        for (; shift >= 0; shift -= 8) {
            for (int i = tid; i < 256 * COUNT_COLUMNS; i += SAMPLE_THREADS) (&scratch.few.count[0][0])[i] = 0;
            if (tid == 0) { s_prefix = prefix << 8; s_need = (u64)need; s_candidates = CANDIDATES + 1; }
            __syncthreads();
            const bool weigh = shift == 24 && !cut_k;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float xi = x[i];
                const uint32_t key = order_key(xi);
                if (shift == 24 || (key >> (shift + 8)) == prefix)
                    atomicAdd(&scratch.few.count[(key >> shift) & 255u][lane & (COUNT_COLUMNS - 1)], 1u);
                if (weigh) all_mass += mass_of(xi);
            }
            if (weigh) {
                all_mass = warp_sum_u64(all_mass);
                if (lane == 0) warp_mass[warp] = all_mass;
            }
            __syncthreads();
            if (weigh) {
                all_mass = 0;
                for (int w = 0; w < SAMPLE_WARPS; ++w) all_mass += warp_mass[w];
            }
            if (tid < 256) {
                int c = 0;
#pragma unroll
                for (int j = 0; j < COUNT_COLUMNS; ++j) c += (int)scratch.few.count[tid][j];
                bin_count[tid] = c;
            }
            __syncthreads();
            if (warp == 0) {                          // lane l: bins 8 l .. 8 l + 7; the digit from the top
                int local = 0;
#pragma unroll
                for (int b = 0; b < 8; ++b) local += bin_count[lane * 8 + b];
                int suffix = local;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int n = __shfl_down_sync(0xffffffffu, suffix, o);
                    if (lane + o < 32) suffix += n;
                }
                const int above = suffix - local;
                if (above < need && need <= above + local) {
                    int cum = above;
                    for (int b = 7; b >= 0; --b) {
                        const int h = bin_count[lane * 8 + b];
                        if (cum + h >= need) {
                            s_prefix = (prefix << 8) | (uint32_t)(lane * 8 + b);
                            s_need = (u64)(need - cum);
                            // at or above this digit: above the digits so far, above this bin, and in it
                            s_candidates = (want - need) + cum + h;
                            break;
                        }
                        cum += h;
                    }
                }
            }
            __syncthreads();
            prefix = s_prefix;
            need = (int)s_need;
            const bool fits = s_candidates <= CANDIDATES;
            __syncthreads();
            if (fits) break;
        }
        if (shift >= 0) {
            // gather (in any order) and sort
            const int n = s_candidates;
            for (int i = tid; i < CANDIDATES; i += SAMPLE_THREADS) scratch.few.candidate[i] = 0;
            if (tid == 0) s_gathered = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const uint32_t key = order_key(x[i]);
                if ((key >> shift) >= prefix) {
                    const int at = atomicAdd(&s_gathered, 1);
                    if (at < CANDIDATES) scratch.few.candidate[at] = ((u64)key << 32) | (u64)(0xffffffffu - (uint32_t)i);
                }
            }
            int n2 = 64;
            while (n2 < n) n2 <<= 1;
            for (int size = 2; size <= n2; size <<= 1) {
                for (int stride = size >> 1; stride > 0; stride >>= 1) {
                    __syncthreads();
                    for (int t = tid; t < n2 / 2; t += SAMPLE_THREADS) {
                        const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                        const u64 a = scratch.few.candidate[lo], b = scratch.few.candidate[hi];
                        if ((a < b) == ((lo & size) == 0)) { scratch.few.candidate[lo] = b; scratch.few.candidate[hi] = a; }
                    }
                }
            }
            __syncthreads();
            // cumulative weights of the first n_k, two candidates per thread
            const int n_k = cut_k ? min(k, n) : n;
            const int j0 = 2 * tid, j1 = j0 + 1;
            const u64 m0 = j0 < n_k ? mass_of(key_value((uint32_t)(scratch.few.candidate[j0] >> 32))) : 0ull;
            const u64 m1 = j1 < n_k ? mass_of(key_value((uint32_t)(scratch.few.candidate[j1] >> 32))) : 0ull;
            u64 inc = m0 + m1;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const u64 t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            if (lane == 31) warp_mass[warp] = inc;
            __syncthreads();
            u64 before = 0;
            for (int w = 0; w < warp; ++w) before += warp_mass[w];
            scratch.few.upto[j0] = before + inc - m1;
            scratch.few.upto[j1] = before + inc;
            if (tid == 0) s_keep = -1;
            __syncthreads();
            const u64 kept_k = scratch.few.upto[n_k - 1];
            const u64 prev0 = j0 > 0 ? scratch.few.upto[j0 - 1] : 0ull, prev1 = scratch.few.upto[j0];
            int keep = n_k;
            bool enough = true;
            if (cut_p) {
                const u64 total = cut_k ? kept_k : all_mass;
                u64 reach = (u64)ceil((double)fmaxf(share, 0.f) * (double)total);
                reach = min(max(reach, 1ull), total);
                enough = kept_k >= reach;             // else the share lies beyond the candidates
                if (enough) {
                    if (j0 < n_k && prev0 < reach && reach <= scratch.few.upto[j0]) s_keep = j0 + 1;
                    if (j1 < n_k && prev1 < reach && reach <= scratch.few.upto[j1]) s_keep = j1 + 1;
                    __syncthreads();
                    keep = s_keep;
                }
            }
            if (enough && keep > 0) {
                const u64 total = scratch.few.upto[keep - 1];
                u64 target = (u64)ceil((double)uniform[r] * (double)total);
                target = min(max(target, 1ull), total);
                int chosen = -1;
                if (j0 < keep && prev0 < target && target <= scratch.few.upto[j0]) chosen = j0;
                if (j1 < keep && prev1 < target && target <= scratch.few.upto[j1]) chosen = j1;
                if (chosen >= 0) {
                    const int token = (int)(0xffffffffu - (uint32_t)(scratch.few.candidate[chosen] & 0xffffffffull));
                    out[r] = token;
                    if (slots && last_token) last_token[slots[r]] = token;
                }
                return;
            }
            __syncthreads();
        }
    }

    // ---- the general path: cuts over the whole row, the walk in index order ----
    if (cut_k) {
        u64 need = (u64)k;
        cut = select(false, need);
        ties = (int)need;                             // of the indices with the k-th largest logit: the first so many
        count_ties_before();
    }
    if (cut_p) {
        u64 before, total;
        kept_mass(before, total);
        u64 need = (u64)ceil((double)fmaxf(share, 0.f) * (double)total);
        need = min(max(need, 1ull), total);
        const uint32_t at = select(true, need);
        const u64 one = max(mass_of(key_value(at)), 1ull);
        int enough = (int)min((need + one - 1) / one, (u64)NO_TIE_LIMIT);
        enough = max(enough, 1);
        if (at == cut) enough = min(enough, ties);
        cut = at;
        ties = enough;
        count_ties_before();
    }

    // the draw: the warp in whose run the cumulative weight passes the target walks its run again
    u64 before, total;
    const u64 mine = kept_mass(before, total);
    u64 target = (u64)ceil((double)uniform[r] * (double)total);
    target = min(max(target, 1ull), total);
    if (!(before < target && target <= before + mine)) return;
    u64 cum = before;
    int chosen = -1;
    each([&](int i, float xi, uint32_t, bool in) {
        if (chosen >= 0) return;
        const u64 m = in ? mass_of(xi) : 0ull;
        const u64 round = round_sum(m);
        if (cum + round < target) { cum += round; return; }
        u64 upto = m;                                 // inclusive over the lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 n = __shfl_up_sync(0xffffffffu, upto, o);
            if (lane >= o) upto += n;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, m > 0 && cum + upto >= target);
        chosen = (i - lane) + __ffs(hit) - 1;         // hit is not empty: the round's sum reaches the target
    });
    if (lane == 0 && chosen >= 0) {
        out[r] = chosen;
        if (slots && last_token) last_token[slots[r]] = chosen;
    }
}

}  // namespace air

// top_k [R] int (0: off) and top_p [R] float (1: off) may be null.
AIR_API int air_sample(const float* logits, const float* temperature, const float* uniform, const int* top_k,
                       const float* top_p, int* out, const int* slots, int* last_token, int R, int V, int* status,
                       cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return AIR_ERR_BAD_ARGUMENT;
    return air::launch(air::sample_kernel, R, air::SAMPLE_THREADS, 0, stream, logits, temperature, uniform, top_k,
                       top_p, out, slots, last_token, V, status);
}

AIR_API int air_trace_set_sampling(unsigned long long* buffer) { return air::set_trace_here(buffer); }
