// Shared helpers of the sm_100a kernels: element types, conversions, reductions and the
// dispatch from a run-time dtype code to a template argument.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define AIR_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with air_b200/csrc/ops.py
#define AIR_F32 0
#define AIR_BF16 1

// error codes returned by the launchers (0 and CUDA's own codes apart)
#define AIR_ERR_BAD_ARGUMENT 100001

namespace air {

// Programmatic dependent launch.  Every kernel of this library is launched with the attribute
// that lets it become resident while its predecessor in the stream is still running, and every
// kernel begins with pdl_enter(): it first tells the scheduler that its own successor may be
// launched, then waits until its predecessor has completed and its writes are visible.  Whatever
// a kernel does before pdl_enter() (setting up barriers, fetching weights, which no kernel
// writes) overlaps the predecessor's tail.  Without the attribute both instructions do nothing.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Optional timeline: when a trace buffer is set (air_set_trace), block 0 of every kernel appends
// (kernel id, %globaltimer) once it has passed the wait on its predecessor.  Slot 0 counts entries.
static __device__ unsigned long long* g_trace = nullptr;
__device__ __forceinline__ void trace_point(int id) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long* t = g_trace;
        if (t) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            const unsigned long long i = atomicAdd(t, 1ull);
            if (i < 16384) {
                t[1 + 2 * i] = (unsigned long long)id;
                t[2 + 2 * i] = now;
            }
        }
    }
}
enum TraceId { TR_EMBED = 1, TR_NORM, TR_ROPE, TR_SILU, TR_CONVERT, TR_TABLE, TR_ATT_REF, TR_ATT_DECODE, TR_ATT_COMBINE,
               TR_ATT_PREFILL, TR_GEMM_F32, TR_GEMM_TC, TR_SAMPLE };

__device__ __forceinline__ void pdl_enter(int id = 0) {
    pdl_trigger();
    pdl_wait();
    trace_point(id);
}

// Every translation unit has its own copy of g_trace; this sets the copy of the unit that calls it.
inline int set_trace_here(unsigned long long* buffer) {
    return (int)cudaMemcpyToSymbol(g_trace, &buffer, sizeof(buffer));
}

// 1: launches carry the programmatic-serialization attribute (set by air_set_pdl).
int& pdl_enabled();

template <typename... KArgs, typename... Args>
inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Four consecutive elements at once (the address must be aligned to four elements).
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on the block size, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = 0.f;
    for (int i = 0; i < warps; ++i) total += scratch[i];
    return total;
}

}  // namespace air

// Calls `body` with `T` bound to the element type of dtype code `code`.
#define AIR_DISPATCH(code, T, ...)                                     \
    do {                                                               \
        if ((code) == AIR_F32) { using T = float; __VA_ARGS__; }       \
        else if ((code) == AIR_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return AIR_ERR_BAD_ARGUMENT;                              \
    } while (0)
