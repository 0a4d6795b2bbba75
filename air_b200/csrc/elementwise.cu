// Embedding gather, residual-add + RMSNorm, bias + rotary + cache write, SiLU*mul.
// All arithmetic is 32-bit; bfloat16 appears only where a value is read or stored.
#include "common.cuh"
#include "tma.cuh"

namespace air {

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32.  A negative id -(s+1) stands for "the token that
// was sampled last for state slot s": it is read from last_token[s], so a decoded token can
// be fed back without passing through the host.  A token outside the table sets *status and
// yields a row of zeros (the host checks ids first; this is the device's own guard).
template <typename TT>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 const int* __restrict__ last_token, float* __restrict__ out, int E, int V,
                                 float multiplier, int* status) {
    // The step's first kernel.  It lets its successors start only once ITS predecessors are done (the copy of the
    // step's batch, the update of the block tables): kernels further down the step read those before their own
    // wait on their predecessor (the decode attention's copy warp).
    pdl_wait();
    pdl_trigger();
    trace_point(TR_EMBED);
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && last_token) id = last_token[-id - 1];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0 && status) atomicExch(status, 1);
    const TT* row = table + (size_t)(ok ? id : 0) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x)
        out[(size_t)t * E + i] = ok ? (multiplier == 1.f ? to_float(row[i]) : to_float(row[i]) * multiplier) : 0.f;
}

// ---------------------------------------------------------------- h += delta
// h[t, i] += sum over parts of delta[part, t, i], the parts added in order (float32 stream; delta float32
// or bfloat16).  The norm kernel below does this sum on its way; this is the sum alone, for a norm of
// another kind that wants the stream complete before it starts.
template <typename TD>
__global__ void add_parts_kernel(float* __restrict__ h, const TD* __restrict__ delta, int parts, size_t n) {
    pdl_enter(TR_NORM);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float x = h[i];
        for (int p = 0; p < parts; ++p) x += to_float(delta[(size_t)p * n + i]);
        h[i] = x;
    }
}

// ---------------------------------------------------------------- add + the next norm's rows, short of their scale
// For few rows (a decode step).  h[t, i] += sum over parts of delta[part, t, i]; xg[t, i] = bfloat16(h[t, i] * w[i]);
// ss[chunk, t] = the sum of h[t, i]^2 over the chunk's PN_CHUNK columns.  The RMSNorm's scale per row,
// rsqrt(sum over chunks of ss / E + eps), is one number per row and commutes with the matrix product that takes
// xg: that product applies it to its accumulators (gemm_tc_small.cu), working it out from ss while its weights
// stream.  So no block here waits for a row's other blocks: a (row, chunk) is one block of PN_CHUNK / 4 threads
// that issues all its loads at once, and the kernel is as long as one round trip to L2, where the norm kernel above
// is a chain of a row's loads, a block-wide sum and a second pass (4 to 5 us at 8 rows of 3,584).
constexpr int PN_CHUNK = 512;
constexpr int PN_PARTS = 8;      // partial sums that a thread asks for at once
template <typename TD, typename TW>
__global__ void __launch_bounds__(PN_CHUNK / 4) add_prenorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                                   int parts, size_t part_stride,
                                                                   const TW* __restrict__ w,
                                                                   __nv_bfloat16* __restrict__ xg,
                                                                   float* __restrict__ ss, int T, int E) {
    __shared__ float scratch[32];
    pdl_enter(TR_NORM);
    const int t = blockIdx.y, chunk = blockIdx.x;
    const int i = chunk * PN_CHUNK + threadIdx.x * 4;
    const bool in = i < E;
    const size_t at = (size_t)t * E + i;
    float x[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f}, d[PN_PARTS][4];
    if (in) {
        load4(h + at, x);
        load4(w + i, wv);
#pragma unroll
        for (int p = 0; p < PN_PARTS; ++p)
            if (p < parts) load4(delta + p * part_stride + at, d[p]);
#pragma unroll
        for (int p = 0; p < PN_PARTS; ++p)
            if (p < parts) {
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] += d[p][j];
            }
        for (int p = PN_PARTS; p < parts; ++p) {
            float e[4];
            load4(delta + p * part_stride + at, e);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] += e[j];
        }
        if (parts > 0) store4(h + at, x);
        float y[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = x[j] * wv[j];
        store4(xg + at, y);
    }
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) sq += x[j] * x[j];
    const float total = block_sum(sq, scratch);
    if (threadIdx.x == 0) ss[(size_t)chunk * T + t] = total;
}

// ---------------------------------------------------------------- what follows the output matrix
// logits[r, v] = (logits[r, v] + bias[v]) * scale, then cap * tanh(. / cap) where cap > 0.  In place, float32.
__global__ void logits_post_kernel(float* __restrict__ logits, const float* __restrict__ bias, float scale, float cap,
                                   int V, size_t n) {
    pdl_enter(TR_CONVERT);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float x = logits[i];
        if (bias) x += bias[i % (size_t)V];
        x *= scale;
        if (cap > 0.f) x = cap * tanhf(x / cap);
        logits[i] = x;
    }
}

// ---------------------------------------------------------------- add + RMSNorm
// One block per row.  h (float32 residual stream) is updated in place with delta when
// rows == nullptr; with rows the kernel reads h[rows[r]] (+ delta[rows[r]]) and leaves h
// as it is.  out[r, i] = x_i * rsqrt(mean(x^2) + eps) * w_i, product order x*scale*w.
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const TW* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int E, float eps) {
    __shared__ float scratch[32];
    extern __shared__ float xrow[];
    pdl_enter(TR_NORM);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * E;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float x = h[src + i];
        if (delta) x += to_float(delta[src + i]);
        xrow[i] = x;
        ss += x * x;
    }
    const float total = block_sum(ss, scratch);
    const float scale = rsqrtf(total / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float x = xrow[i];
        if (!rows && delta) h[src + i] = x;
        out[(size_t)r * E + i] = from_float<TO>(x * scale * to_float(w[i]));
    }
}

// The same with four elements per access, for E % 4 == 0.  `parts` tensors of delta's shape,
// one after the other, are summed in order (the partial sums of a split product).  With few rows the
// kernel is a chain of latencies, so a thread first issues all of its loads (up to ELT_PARTS parts at
// once) and the block is as wide as the row (one access per thread where E <= 4096).
constexpr int ELT_PARTS = 8;
#ifndef NORM_REGS
#define NORM_REGS 56
#endif
template <typename TD, typename TW, typename TO>
__global__ void __maxnreg__(NORM_REGS) add_rmsnorm_vec4_kernel(float* __restrict__ h, const TD* __restrict__ delta, int parts,
                                        size_t part_stride, const TW* __restrict__ w, TO* __restrict__ out,
                                        const int* __restrict__ rows, int E, float eps) {
    __shared__ float scratch[32];
    extern __shared__ float xrow[];
    pdl_enter(TR_NORM);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * E;
    float ss = 0.f;
    const int i0 = threadIdx.x * 4;
    float w0[4] = {0.f, 0.f, 0.f, 0.f};
    if (i0 < E) load4(w + i0, w0);          // the weights of the thread's first elements, asked for with the rest
    for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
        float x[4], d[ELT_PARTS][4];
        load4(h + src + i, x);
#pragma unroll
        for (int p = 0; p < ELT_PARTS; ++p)
            if (p < parts) load4(delta + p * part_stride + src + i, d[p]);
#pragma unroll
        for (int p = 0; p < ELT_PARTS; ++p)
            if (p < parts) {
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] += d[p][j];
            }
        for (int p = ELT_PARTS; p < parts; ++p) {
            float e[4];
            load4(delta + p * part_stride + src + i, e);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] += e[j];
        }
        store4(xrow + i, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
    }
    const float total = block_sum(ss, scratch);
    const float scale = rsqrtf(total / (float)E + eps);
    for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
        float x[4], wv[4], y[4];
        load4(xrow + i, x);
        if (i == i0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = w0[j];
        } else {
            load4(w + i, wv);
        }
        if (!rows && parts > 0) store4(h + src + i, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = x[j] * scale * wv[j];
        store4(out + (size_t)r * E + i, y);
    }
}

// The same for many rows (a prompt portion), where the rows hide each other's latencies and a thread
// that holds fewer registers lets more of them run at a time.
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_vec4_many_kernel(float* __restrict__ h, const TD* __restrict__ delta, int parts,
                                        size_t part_stride, const TW* __restrict__ w, TO* __restrict__ out,
                                        const int* __restrict__ rows, int E, float eps) {
    __shared__ float scratch[32];
    extern __shared__ float xrow[];
    pdl_enter(TR_NORM);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * E;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
        float x[4];
        load4(h + src + i, x);
        for (int p = 0; p < parts; ++p) {
            float d[4];
            load4(delta + p * part_stride + src + i, d);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] += d[j];
        }
        store4(xrow + i, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
    }
    const float total = block_sum(ss, scratch);
    const float scale = rsqrtf(total / (float)E + eps);
    for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) {
        float x[4], wv[4], y[4];
        load4(xrow + i, x);
        load4(w + i, wv);
        if (!rows && parts > 0) store4(h + src + i, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = x[j] * scale * wv[j];
        store4(out + (size_t)r * E + i, y);
    }
}

// For many rows of moderate width: a row is held in the registers of a small block (up to NV vectors of four
// per thread), so that it is read once, there is one block-wide sum and many blocks fit on an SM.
template <typename TD, typename TW, typename TO, int NV>
__global__ void __launch_bounds__(256) add_rmsnorm_vec4_held_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                                    int parts, size_t part_stride,
                                                                    const TW* __restrict__ w, TO* __restrict__ out,
                                                                    const int* __restrict__ rows, int E, float eps) {
    __shared__ float scratch[NV * 8];
    pdl_enter(TR_NORM);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * E;
    float x[NV][4];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = (v * blockDim.x + threadIdx.x) * 4;
        if (i < E) load4(h + src + i, x[v]);
    }
    for (int p = 0; p < parts; ++p) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int i = (v * blockDim.x + threadIdx.x) * 4;
            if (i < E) {
                float d[4];
                load4(delta + p * part_stride + src + i, d);
#pragma unroll
                for (int j = 0; j < 4; ++j) x[v][j] += d[j];
            }
        }
    }
    // The sum of squares in the order of the kernel for few rows, so that a row's result does not depend on how
    // many rows are beside it (up to 4,096 wide, where that kernel has one vector per thread): four squares per
    // vector, a warp's 32 vectors by the shuffle tree, the warps one after the other.
    const int warps = blockDim.x >> 5;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = (v * blockDim.x + threadIdx.x) * 4;
        float sv = 0.f;
        if (i < E) {
#pragma unroll
            for (int j = 0; j < 4; ++j) sv += x[v][j] * x[v][j];
            if (!rows && parts > 0) store4(h + src + i, x[v]);
        }
        sv = warp_sum(sv);
        if ((threadIdx.x & 31) == 0) scratch[v * warps + (threadIdx.x >> 5)] = sv;
    }
    __syncthreads();
    float total = 0.f;
    for (int k = 0; k < (E / 4 + 31) / 32; ++k) total += scratch[k];
    const float scale = rsqrtf(total / (float)E + eps);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = (v * blockDim.x + threadIdx.x) * 4;
        if (i < E) {
            float wv[4], y[4];
            load4(w + i, wv);
#pragma unroll
            for (int j = 0; j < 4; ++j) y[j] = x[v][j] * scale * wv[j];
            store4(out + (size_t)r * E + i, y);
        }
    }
}

// Many rows and nothing to add (a prompt step whose products add into the stream themselves): the copy engine brings a
// block's row into shared memory with one instruction and no registers, so that a block is small, 14 rows of 3,584
// fit on an SM, and all rows of a prompt portion are on their way at once; the kernel that holds a row in registers
// runs 2,048 rows in two rounds of blocks (10.7 us against 5.3 for a copy of the same bytes; this kernel 8.5, and
// 11.4 against 15.1 from a cold L2).  The sum of squares is
// taken in the order of the kernel for few rows (see add_rmsnorm_vec4_held_kernel).  Should the copy never arrive
// (the wait is bounded), the block waits some more, so that the copy cannot land in a later block's memory, and
// reads the row with plain loads.
template <typename TW, typename TO>
__global__ void __launch_bounds__(128) add_rmsnorm_bulk_kernel(const float* __restrict__ h, const TW* __restrict__ w,
                                                               TO* __restrict__ out, const int* __restrict__ rows, int E,
                                                               float eps) {
    extern __shared__ __align__(16) float xrow[];
    __shared__ float scratch[64];
    __shared__ uint64_t bar;
    __shared__ int gave_up;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_enter(TR_NORM);
    const int r = blockIdx.x;
    const float* src = h + (size_t)(rows ? rows[r] : r) * E;
    if (threadIdx.x == 0) {
        mbar_expect_tx(&bar, (uint32_t)E * 4u);
        bulk_load(xrow, src, (uint32_t)E * 4u, &bar);
    }
    const float* x = xrow;
    if (!mbar_wait(&bar, 0, &gave_up)) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        x = src;
    }
    const int vectors = E / 4;
    for (int v = 0; v * 128 < vectors; ++v) {
        const int i = v * 128 + threadIdx.x;
        float sv = 0.f;
        if (i < vectors) {
            float t[4];
            load4(x + 4 * i, t);
#pragma unroll
            for (int j = 0; j < 4; ++j) sv += t[j] * t[j];
        }
        sv = warp_sum(sv);
        if ((threadIdx.x & 31) == 0) scratch[v * 4 + (threadIdx.x >> 5)] = sv;
    }
    __syncthreads();
    float total = 0.f;
    for (int k = 0; k < (vectors + 31) / 32; ++k) total += scratch[k];
    const float scale = rsqrtf(total / (float)E + eps);
    for (int i = threadIdx.x; i < vectors; i += 128) {
        float t[4], wv[4], y[4];
        load4(x + 4 * i, t);
        load4(w + 4 * i, wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = t[j] * scale * wv[j];
        store4(out + (size_t)r * E + 4 * i, y);
    }
}

// ---------------------------------------------------------------- bias + rotary + cache write
// qkv [T, (H + 2K) d] is the output of the fused projection.  For every token: add the
// bias, rotate the heads of q and k with the table's cos/sin of the token's position
// (pairs (i, i + rot/2) of the first `rot` elements of a head), store q to q_out [T, H, d]
// and k, v into the token's place in the pages: cache [page, 2, K, P, d].  token_seq[t] is the
// slot of the token's request = its row of block_table; a negative slot marks padding.
// table [positions, rot]: cos in the first rot/2 columns, sin in the second.
template <typename TI, typename TB, typename TO>
__global__ void qkv_rope_store_kernel(const TI* __restrict__ qkv, const TB* __restrict__ bias,
                                      const float* __restrict__ table, int rot,
                                      const int* __restrict__ positions, const int* __restrict__ token_seq,
                                      const int* __restrict__ block_table, int max_blocks,
                                      TO* __restrict__ q_out, TO* __restrict__ cache,
                                      int H, int K, int d, int P, int write_kv, int* status) {
    pdl_enter(TR_ROPE);
    const int t = blockIdx.x;
    const int slot = token_seq[t];
    if (slot < 0) return;  // padding
    const int pos = positions[t];
    const int width = (H + 2 * K) * d;
    const TI* in = qkv + (size_t)t * width;
    const int half = rot / 2;
    TO* kdst = nullptr;
    TO* vdst = nullptr;
    if (write_kv) {
        const int page = block_table[(size_t)slot * max_blocks + pos / P];
        if (page < 0) {
            if (threadIdx.x == 0 && status) atomicExch(status, 2);
        } else {
            kdst = cache + ((size_t)page * 2 * K * P + (size_t)(pos % P)) * d;
            vdst = kdst + (size_t)K * P * d;
        }
    }
    // one thread per (head, element below half or beyond the rotated part)
    const int per_head = d - half;  // pairs in [0, half) plus unrotated tail [rot, d)
    const int heads = H + 2 * K;
    for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
        const int head = idx / per_head;
        const int j = idx % per_head;
        const int base = head * d;
        const bool is_v = head >= H + K;
        if (!write_kv && head >= H) continue;
        float a, b = 0.f;
        bool pair = !is_v && j < half;
        int i0, i1 = 0;
        if (is_v) {
            // values are not rotated: this thread copies element j and, if any, j + per_head
            i0 = j;
            i1 = j + per_head;
            pair = i1 < d;
        } else if (j < half) {
            i0 = j;
            i1 = j + half;
        } else {
            i0 = j + half;  // tail element beyond the rotated part
        }
        a = to_float(in[base + i0]);
        if (bias) a += to_float(bias[base + i0]);
        if (pair) {
            b = to_float(in[base + i1]);
            if (bias) b += to_float(bias[base + i1]);
        }
        if (!is_v && j < half) {
            const float c = table[(size_t)pos * rot + j];
            const float s = table[(size_t)pos * rot + half + j];
            const float ra = a * c - b * s;
            const float rb = a * s + b * c;
            a = ra;
            b = rb;
        }
        if (head < H) {
            TO* dst = q_out + ((size_t)t * H + head) * d;
            dst[i0] = from_float<TO>(a);
            if (pair) dst[i1] = from_float<TO>(b);
        } else if (kdst) {
            const int kvh = is_v ? head - H - K : head - H;
            TO* dst = (is_v ? vdst : kdst) + (size_t)kvh * P * d;
            dst[i0] = from_float<TO>(a);
            if (pair) dst[i1] = from_float<TO>(b);
        }
    }
}

// The same for full rotation (rot == d) with four pairs per thread.  `parts` tensors of qkv's
// shape are summed in order (the partial sums of a split product).
constexpr int ROPE_PARTS = 4;      // partial sums that a thread asks for ahead of the index chain
constexpr int ROPE_THREADS = 640;
template <typename TI, typename TB, typename TO>
__global__ void __launch_bounds__(ROPE_THREADS) qkv_rope_store_vec4_kernel(const TI* __restrict__ qkv, int parts, size_t part_stride,
                                           const TB* __restrict__ bias, const float* __restrict__ table,
                                           const int* __restrict__ positions, const int* __restrict__ token_seq,
                                           const int* __restrict__ block_table, int max_blocks,
                                           TO* __restrict__ q_out, TO* __restrict__ cache,
                                           int H, int K, int d, int P, int write_kv, int* status) {
    pdl_enter(TR_ROPE);
    const int t = blockIdx.x;
    const int width = (H + 2 * K) * d, half = d / 2;
    const TI* in = qkv + (size_t)t * width;
    const int per_head = half / 4;
    const int heads = write_kv ? H + 2 * K : H;
    // With few tokens the kernel is a chain of latencies: the first item's partial sums are asked
    // for before the token's slot, position and page are looked up (a padding token's row exists too).
    float pa[ROPE_PARTS][4], pb[ROPE_PARTS][4];
    const int first = threadIdx.x;
    if (first < heads * per_head) {
        const int base = (first / per_head) * d, j = (first % per_head) * 4;
#pragma unroll
        for (int p = 0; p < ROPE_PARTS; ++p)
            if (p < parts) {
                load4(in + p * part_stride + base + j, pa[p]);
                load4(in + p * part_stride + base + half + j, pb[p]);
            }
    }
    const int slot = token_seq[t];
    const int pos = positions[t];
    if (slot < 0) return;
    TO* kdst = nullptr;
    TO* vdst = nullptr;
    if (write_kv) {
        const int page = block_table[(size_t)slot * max_blocks + pos / P];
        if (page < 0) {
            if (threadIdx.x == 0 && status) atomicExch(status, 2);
        } else {
            kdst = cache + ((size_t)page * 2 * K * P + (size_t)(pos % P)) * d;
            vdst = kdst + (size_t)K * P * d;
        }
    }
    const float* cs = table + (size_t)pos * d;
    for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
        const int head = idx / per_head, j = (idx % per_head) * 4;
        const int base = head * d;
        float a[4], b[4];
        if (idx == first) {
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] = pa[0][e]; b[e] = pb[0][e]; }
#pragma unroll
            for (int p = 1; p < ROPE_PARTS; ++p)
                if (p < parts) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) { a[e] += pa[p][e]; b[e] += pb[p][e]; }
                }
        } else {
            load4(in + base + j, a);
            load4(in + base + half + j, b);
        }
        for (int p = (idx == first ? ROPE_PARTS : 1); p < parts; ++p) {
            float x[4], y[4];
            load4(in + p * part_stride + base + j, x);
            load4(in + p * part_stride + base + half + j, y);
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] += x[e]; b[e] += y[e]; }
        }
        if (bias) {
            float x[4], y[4];
            load4(bias + base + j, x);
            load4(bias + base + half + j, y);
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] += x[e]; b[e] += y[e]; }
        }
        const bool is_v = head >= H + K;
        if (!is_v) {
            float c[4], sn[4];
            load4(cs + j, c);
            load4(cs + half + j, sn);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float ra = a[e] * c[e] - b[e] * sn[e], rb = a[e] * sn[e] + b[e] * c[e];
                a[e] = ra;
                b[e] = rb;
            }
        }
        TO* dst;
        if (head < H) dst = q_out + ((size_t)t * H + head) * d;
        else if (!kdst) continue;
        else dst = (is_v ? vdst + (size_t)(head - H - K) * P * d : kdst + (size_t)(head - H) * P * d);
        store4(dst + j, a);
        store4(dst + half + j, b);
    }
}

// The same for many tokens (a prompt portion): plain loops, fewer registers, 256 threads.
template <typename TI, typename TB, typename TO>
__global__ void qkv_rope_store_vec4_many_kernel(const TI* __restrict__ qkv, int parts, size_t part_stride,
                                           const TB* __restrict__ bias, const float* __restrict__ table,
                                           const int* __restrict__ positions, const int* __restrict__ token_seq,
                                           const int* __restrict__ block_table, int max_blocks,
                                           TO* __restrict__ q_out, TO* __restrict__ cache,
                                           int H, int K, int d, int P, int write_kv, int* status) {
    pdl_enter(TR_ROPE);
    const int t = blockIdx.x;
    const int slot = token_seq[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int width = (H + 2 * K) * d, half = d / 2;
    const TI* in = qkv + (size_t)t * width;
    TO* kdst = nullptr;
    TO* vdst = nullptr;
    if (write_kv) {
        const int page = block_table[(size_t)slot * max_blocks + pos / P];
        if (page < 0) {
            if (threadIdx.x == 0 && status) atomicExch(status, 2);
        } else {
            kdst = cache + ((size_t)page * 2 * K * P + (size_t)(pos % P)) * d;
            vdst = kdst + (size_t)K * P * d;
        }
    }
    const int per_head = half / 4;
    const int heads = write_kv ? H + 2 * K : H;
    const float* cs = table + (size_t)pos * d;
    for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
        const int head = idx / per_head, j = (idx % per_head) * 4;
        const int base = head * d;
        float a[4], b[4];
        load4(in + base + j, a);
        load4(in + base + half + j, b);
        for (int p = 1; p < parts; ++p) {
            float x[4], y[4];
            load4(in + p * part_stride + base + j, x);
            load4(in + p * part_stride + base + half + j, y);
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] += x[e]; b[e] += y[e]; }
        }
        if (bias) {
            float x[4], y[4];
            load4(bias + base + j, x);
            load4(bias + base + half + j, y);
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] += x[e]; b[e] += y[e]; }
        }
        const bool is_v = head >= H + K;
        if (!is_v) {
            float c[4], sn[4];
            load4(cs + j, c);
            load4(cs + half + j, sn);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float ra = a[e] * c[e] - b[e] * sn[e], rb = a[e] * sn[e] + b[e] * c[e];
                a[e] = ra;
                b[e] = rb;
            }
        }
        TO* dst;
        if (head < H) dst = q_out + ((size_t)t * H + head) * d;
        else if (!kdst) continue;
        else dst = (is_v ? vdst + (size_t)(head - H - K) * P * d : kdst + (size_t)(head - H) * P * d);
        store4(dst + j, a);
        store4(dst + half + j, b);
    }
}

// ---------------------------------------------------------------- SiLU(gate) * up
// in [T, 2I]: blocks of `block` gate columns and `block` up columns in turn (block = I: all gate
// columns, then all up columns).  out [T, I].
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ in, TO* __restrict__ out, int I, int block, size_t total) {
    pdl_enter(TR_SILU);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx % I);
        const size_t at = t * 2 * I + (size_t)(i / block) * 2 * block + i % block;
        const float g = to_float(in[at]);
        const float u = to_float(in[at + block]);
        out[idx] = from_float<TO>(g / (1.f + expf(-g)) * u);
    }
}

template <typename TI, typename TO>
__global__ void silu_mul_vec4_kernel(const TI* __restrict__ in, TO* __restrict__ out, int I, int block,
                                     size_t total4) {
    pdl_enter(TR_SILU);
    const int I4 = I / 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I4;
        const int i = (int)(idx % I4) * 4;
        const size_t at = t * 2 * I + (size_t)(i / block) * 2 * block + i % block;
        float g[4], u[4], y[4];
        load4(in + at, g);
        load4(in + at + block, u);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = g[e] / (1.f + expf(-g[e])) * u[e];
        store4(out + t * I + i, y);
    }
}

// Eight bfloat16 at a time (16-byte accesses), for I % 8 == 0 and block % 8 == 0.
__global__ void __launch_bounds__(256, 4) silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ in,
                                                                 __nv_bfloat16* __restrict__ out, int I, int block,
                                                                 size_t total8) {
    // A thread takes two groups of eight outputs, a block's width apart, and asks for its four 16-byte loads before
    // it computes (with one group per thread a block lived for one round trip to memory: 544 rows of 18,944 took
    // 14.6 us, a copy of the same bytes 8.9; four groups per thread needed 86 registers and took 22 us).  The
    // index arithmetic is 32-bit where the sizes allow, and 1 / (1 + e^-g) is the fast division of the fast
    // exponential: their errors are far below the rounding of the result to bfloat16.
    pdl_enter(TR_SILU);
    const int I8 = I / 8;
    constexpr int PER = 2;
    const bool narrow = total8 < (1ull << 31);
    for (size_t first = (size_t)blockIdx.x * blockDim.x * PER + threadIdx.x; first < total8;
         first += (size_t)gridDim.x * blockDim.x * PER) {
        uint4 gv[PER], uv[PER];
        size_t to[PER];
        bool live[PER];
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const size_t idx = first + (size_t)k * blockDim.x;
            live[k] = idx < total8;
            if (live[k]) {
                const size_t t = narrow ? (size_t)((uint32_t)idx / (uint32_t)I8) : idx / I8;
                const int i = (int)(idx - t * I8) * 8;
                const size_t at = t * 2 * I + (size_t)(i / block) * 2 * block + i % block;
                gv[k] = *reinterpret_cast<const uint4*>(in + at);
                uv[k] = *reinterpret_cast<const uint4*>(in + at + block);
                to[k] = t * I + i;
            }
        }
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            if (live[k]) {
                const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv[k]);
                const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv[k]);
                uint4 ov;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
                    o2[e] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x,
                                                  __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
                }
                *reinterpret_cast<uint4*>(out + to[k]) = ov;
            }
        }
    }
}

// ---------------------------------------------------------------- block table updates
// updates [n, 3]: (slot, block, page) -> table[slot, block] = page
__global__ void table_update_kernel(int* __restrict__ table, const int* __restrict__ updates, int n, int W) {
    pdl_enter(TR_TABLE);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) table[(size_t)updates[3 * i] * W + updates[3 * i + 1]] = updates[3 * i + 2];
}

// ---------------------------------------------------------------- conversions
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    pdl_enter(TR_CONVERT);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<TO>(to_float(in[i]));
}

}  // namespace air

using namespace air;

AIR_API int air_embedding(const void* table, int table_dtype, const int* ids, const int* last_token, float* out,
                          int T, int E, int V, float multiplier, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    AIR_DISPATCH(table_dtype, TT, return launch(embedding_kernel<TT>, T, 256, 0, stream, (const TT*)table, ids,
                                                last_token, out, E, V, multiplier, status));
    return 0;
}

AIR_API int air_add_parts(float* h, const void* delta, int delta_dtype, int parts, long long n, cudaStream_t stream) {
    if (n <= 0 || parts <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    AIR_DISPATCH(delta_dtype, TD, return launch(add_parts_kernel<TD>, blocks, 256, 0, stream, h, (const TD*)delta,
                                                parts, (size_t)n));
    return 0;
}

// h [T, E] float32 (in and out); delta: `parts` tensors [T, E] one after the other (null: none); w [E]; xg [T, E]
// bfloat16; ss [ceil(E / 512), T] float32.  E % 4 == 0, T <= 65535.
AIR_API int air_add_prenorm(float* h, const void* delta, int delta_dtype, int parts, const void* w, int w_dtype,
                            void* xg, float* ss, int T, int E, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E % 4 || T > 65535 || !h || !w || !xg || !ss) return AIR_ERR_BAD_ARGUMENT;
    if (!delta) parts = 0;
    const dim3 grid((E + PN_CHUNK - 1) / PN_CHUNK, T);
    const size_t stride = (size_t)T * E;
    AIR_DISPATCH(delta ? delta_dtype : AIR_F32, TD, AIR_DISPATCH(w_dtype, TW, {
        return launch(add_prenorm_kernel<TD, TW>, grid, PN_CHUNK / 4, 0, stream, h, (const TD*)delta, parts, stride,
                      (const TW*)w, (__nv_bfloat16*)xg, ss, T, E);
    }));
    return 0;
}

AIR_API int air_logits_post(float* logits, const float* bias, float scale, float cap, int R, int V,
                            cudaStream_t stream) {
    const long long n = (long long)R * V;
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    return launch(logits_post_kernel, blocks, 256, 0, stream, logits, bias, scale, cap, V, (size_t)n);
}

// delta: `parts` tensors [rows of h, E] one after the other (parts = 0 or delta = null: none).
AIR_API int air_add_rmsnorm(float* h, const void* delta, int delta_dtype, int parts, const void* w, int w_dtype,
                            void* out, int out_dtype, const int* rows, int R, int E, long long h_rows, float eps,
                            cudaStream_t stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)E * sizeof(float);
    if (smem > 200 * 1024 || parts < 0) return AIR_ERR_BAD_ARGUMENT;
    if (!delta) parts = 0;
    int threads = E >= 2048 ? 512 : 256;
    AIR_DISPATCH(delta_dtype, TD, AIR_DISPATCH(w_dtype, TW, AIR_DISPATCH(out_dtype, TO, {
        if (E % 4 == 0) {
            // (from a thousand rows on: with fewer, all blocks run in one round either way and the copy engine's
            // longer way to the first byte shows: 544 rows 5.7 against 4.8 us)
            if (R >= 1024 && E <= 8192 && parts == 0 && ((uintptr_t)h & 15) == 0)
                return launch(add_rmsnorm_bulk_kernel<TW, TO>, R, 128, smem, stream, (const float*)h, (const TW*)w,
                              (TO*)out, rows, E, eps);
            if (R > 64 && E <= 8192) {
                // many rows: each held in the registers of 128 threads (up to 4,096 wide) or 256
                const int held = E <= 4096 ? 128 : 256;
                return launch(add_rmsnorm_vec4_held_kernel<TD, TW, TO, 8>, R, held, 0, stream, h, (const TD*)delta, parts,
                              (size_t)h_rows * E, (const TW*)w, (TO*)out, rows, E, eps);
            }
            if (R <= 64) threads = min(1024, max(128, (E / 4 + 31) / 32 * 32));   // few rows: one access per thread
            auto kernel = R <= 64 ? add_rmsnorm_vec4_kernel<TD, TW, TO> : add_rmsnorm_vec4_many_kernel<TD, TW, TO>;
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            return launch(kernel, R, threads, smem, stream, h, (const TD*)delta, parts, (size_t)h_rows * E,
                          (const TW*)w, (TO*)out, rows, E, eps);
        } else {
            if (parts > 1) return AIR_ERR_BAD_ARGUMENT;
            auto kernel = add_rmsnorm_kernel<TD, TW, TO>;
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            return launch(kernel, R, threads, smem, stream, h, parts ? (const TD*)delta : nullptr, (const TW*)w,
                          (TO*)out, rows, E, eps);
        }
    })));
    return (int)cudaGetLastError();
}

AIR_API int air_qkv_rope_store(const void* qkv, int in_dtype, int parts, const void* bias, int bias_dtype,
                               const float* table, int rot, const int* positions, const int* token_seq,
                               const int* block_table, int max_blocks, void* q_out, void* cache,
                               int out_dtype, int T, int H, int K, int d, int P, int write_kv,
                               int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || parts < 1) return AIR_ERR_BAD_ARGUMENT;
    AIR_DISPATCH(in_dtype, TI, AIR_DISPATCH(bias_dtype, TB, AIR_DISPATCH(out_dtype, TO, {
        if (rot == d && d % 8 == 0) {
            // few tokens: one item per thread, so that every load of the block is in flight at once
            const int items = (write_kv ? H + 2 * K : H) * (d / 8);
            // (from a thousand tokens on, blocks of 128 threads: sixteen to an SM, so that 2,048 tokens run in one round of
            // blocks, 9.7 against 11.7 us; with fewer tokens the wider block is faster, 4.2 against 5.1 us at 544)
            const int threads = T <= 64 ? min(ROPE_THREADS, max(128, (items + 31) / 32 * 32)) : (T >= 1024 ? 128 : 256);
            return launch(T <= 64 ? qkv_rope_store_vec4_kernel<TI, TB, TO> : qkv_rope_store_vec4_many_kernel<TI, TB, TO>, T,
                          threads, 0, stream, (const TI*)qkv, parts,
                          (size_t)T * (H + 2 * K) * d, (const TB*)bias, table, positions, token_seq, block_table,
                          max_blocks, (TO*)q_out, (TO*)cache, H, K, d, P, write_kv, status);
        } else {
            if (parts != 1) return AIR_ERR_BAD_ARGUMENT;
            return launch(qkv_rope_store_kernel<TI, TB, TO>, T, 256, 0, stream, (const TI*)qkv, (const TB*)bias,
                          table, rot, positions, token_seq, block_table, max_blocks, (TO*)q_out, (TO*)cache, H, K, d,
                          P, write_kv, status);
        }
    })));
    return (int)cudaGetLastError();
}

AIR_API int air_silu_mul(const void* in, int in_dtype, void* out, int out_dtype, int T, int I, int block,
                         cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (block <= 0 || I % block) return AIR_ERR_BAD_ARGUMENT;
    if (in_dtype == AIR_BF16 && out_dtype == AIR_BF16 && I % 8 == 0 && block % 8 == 0) {
        const size_t n = total / 8;
        const size_t want = (n + 511) / 512;               // 256 threads, two groups each
        const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
        return launch(silu_mul_bf16x8_kernel, blocks, 256, 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, I,
                      block, n);
    }
    AIR_DISPATCH(in_dtype, TI, AIR_DISPATCH(out_dtype, TO, {
        if (I % 4 == 0 && block % 4 == 0) {
            const size_t n = total / 4;
            const int blocks = (int)((n + 255) / 256 < 148 * 32 ? (n + 255) / 256 : 148 * 32);
            return launch(silu_mul_vec4_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)in, (TO*)out, I, block, n);
        } else {
            const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
            return launch(silu_mul_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)in, (TO*)out, I, block, total);
        }
    }));
    return (int)cudaGetLastError();
}

AIR_API int air_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                        cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    AIR_DISPATCH(in_dtype, TI, AIR_DISPATCH(out_dtype, TO, {
        return launch(convert_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)in, (TO*)out, (size_t)n);
    }));
    return (int)cudaGetLastError();
}

AIR_API int air_table_update(int* table, const int* updates, int n, int W, cudaStream_t stream) {
    if (n <= 0) return 0;
    return launch(table_update_kernel, (n + 127) / 128, 128, 0, stream, table, updates, n, W);
}

// 1: kernels are launched so that they may overlap the tail of their predecessor (the default);
// 0: plain stream order.
AIR_API void air_set_pdl(int on) { air::pdl_enabled() = on ? 1 : 0; }

namespace air {
int& pdl_enabled() {
    static int enabled = 1;
    return enabled;
}
}  // namespace air

AIR_API int air_trace_set_elementwise(unsigned long long* buffer) { return air::set_trace_here(buffer); }
