// Shared helpers of the tinyinfer_b200 kernels (sm_100a).
// Every launcher is an extern "C" function taking raw device pointers and a stream; it returns 0
// or a non-zero code and leaves a message for ti_last_error(). Nothing here allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define TI_API extern "C" __attribute__((visibility("default")))

enum TiDtype : int { TI_F32 = 0, TI_BF16 = 1 };

// Host side: message of the last failed call of this thread (one buffer per library).
void ti_set_error(const char* fmt, ...);
void ti_count_launch(int n = 1);

#define TI_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            ti_set_error(__VA_ARGS__);        \
            return -1;                        \
        }                                     \
    } while (0)

#define TI_CHECK_LAUNCH(name)                                                   \
    do {                                                                        \
        cudaError_t e__ = cudaGetLastError();                                   \
        if (e__ != cudaSuccess) {                                               \
            ti_set_error("%s: %s", name, cudaGetErrorString(e__));              \
            return (int)e__;                                                    \
        }                                                                       \
        ti_count_launch();                                                      \
    } while (0)

// Programmatic dependent launch: every kernel of this package waits for the kernels before it in
// the stream with ti_grid_wait() before it touches anything they wrote (and before it writes
// anything), and lets the kernel after it start its own prologue early with
// ti_grid_launch_dependents(). Launched without the attribute, both are no-ops.
__device__ __forceinline__ void ti_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ti_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool ti_pdl_enabled();

// Launches `kernel` with the programmatic-stream-serialization attribute (unless switched off by
// TINYINFER_B200_PDL=0): it may begin while the previous kernel of the stream drains.
template <typename... KArgs, typename... Args>
cudaError_t ti_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ti_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same without the attribute: the kernel starts when the stream's earlier work has ended, on an empty machine,
// so its blocks are dealt evenly to the SMs. For a long kernel of few blocks whose warps wait on latency: started
// early, its blocks land wherever the kernel before frees room first, several on one SM, and stay there.
template <typename... KArgs, typename... Args>
cudaError_t ti_launch_alone(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}

// Scores that level off smoothly: s -> cap * tanh(s / cap). P is an attention kernel's parameter block with scale_log2
// (the softmax scale times log2 e), cap_log2 (cap * log2 e; 0: no cap) and cap_arg (scale / cap). The result is in log2
// units, like raw * scale_log2; a masked score (-inf) stays -inf. These are the bfloat16 tensor-core kernels, whose
// softmax is bound by the transcendental unit: the tanh is the unit's own instruction (one more trip a score, relative
// error 2^-11, below the rounding of the bfloat16 probabilities); from an exponential and a division it was three trips
// a score and the prompt kernel 2.5 times its uncapped time.
// CAP is a template parameter of the kernels, so that the kernels of models without a cap are the code they were.
__device__ __forceinline__ float ti_tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <bool CAP, typename P> __device__ __forceinline__ float ti_score_log2(const P& p, float raw) {
    if constexpr (CAP) {
        if (raw == -INFINITY) return -INFINITY;
        return p.cap_log2 * ti_tanh_approx(raw * p.cap_arg);
    } else {
        return raw * p.scale_log2;
    }
}
// The exponent of a probability, score - m_use, in log2 units.
template <bool CAP, typename P> __device__ __forceinline__ float ti_prob_log2(const P& p, float raw, float m_use) {
    if constexpr (CAP) return ti_score_log2<true>(p, raw) - m_use;
    else return fmaf(raw, p.scale_log2, -m_use);
}
#define TI_SET_SCORE_CAP(p, scale, softcap)                                                        \
    do {                                                                                           \
        (p).cap_log2 = (softcap) > 0.f ? (softcap) * 1.4426950408889634f : 0.f;                     \
        (p).cap_arg = (softcap) > 0.f ? (scale) / (softcap) : 0.f;                                  \
    } while (0)

// A softmax sink and an output factor that may differ from head to head. P is an attention kernel's parameter block with
// sink_log2 / head_sinks (float32 natural-log logits per query head, or null) and out_scale / gate (bfloat16 rows of
// ld_gate elements, first column gate_off, one logit per (token, query head), or null: the output is also multiplied by
// sigmoid(gate)).
template <typename P> __device__ __forceinline__ float ti_sink_log2(const P& p, int head) {
    return p.head_sinks ? p.head_sinks[head] * 1.4426950408889634f : p.sink_log2;
}
template <typename P> __device__ __forceinline__ float ti_head_out_scale(const P& p, size_t row, int head) {
    if (!p.gate) return p.out_scale;
    const float z = __bfloat162float(p.gate[row * p.ld_gate + p.gate_off + head]);
    return p.out_scale / (1.f + expf(-z));
}
