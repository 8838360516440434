// A residual that is several float32 streams instead of one ("hyper-connections": Zhu et al., 2024). The streams
// are X [S][T][W] float32. A sublayer reads one mixture of them and writes back into all of them:
//     u = sum_s c_in[s] X[s]                    h = w * u * rsqrt(mean(u^2) + eps)   (the sublayer's input)
//     X[t] <- sum_s c_mix[s][t] X[s] + c_out[t] * y        (all streams at once from the old ones; y = sublayer(h))
// One kernel does a sublayer's write-back AND the next sublayer's read: streams_step first applies the update
// that the sublayer before left pending (if any), in place, then mixes and norms with the next sublayer's
// coefficients (if any). A block owns a token's row of every stream; the sums and the norm are float32, the
// rounding of h to the compute dtype is the only one. With S = 1, c_in = c_mix = c_out = 1 this is the ordinary
// pre-norm residual kept in float32.
//   streams_embed : X[s][t] = table[id[t]] * scale for every s
//   streams_step  : as above; `rows` picks the tokens to work on (the rows whose logits are wanted)
//   gelu, scale   : the feed-forward's activation on a stored tensor, and a constant factor on float32 logits
//   soft_cap      : x <- cap * tanh(x / cap) on float32 logits
#include "common.cuh"

constexpr int HS_MAX_STREAMS = 8;

template <typename T>
__global__ void streams_embed_kernel(float* __restrict__ X, const T* __restrict__ table, const int* __restrict__ ids,
                                     int num_tokens, int width, int vocab, int streams, float scale) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ok ? to_f32(src[i]) * scale : 0.f;
        for (int s = 0; s < streams; ++s) X[((size_t)s * num_tokens + t) * width + i] = v;
    }
}

TI_API int ti_streams_embed(float* X, const void* table, const int* ids, int num_tokens, int width, int vocab, int streams,
                            float scale, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && width > 0 && vocab > 0 && streams >= 1 && streams <= HS_MAX_STREAMS,
               "streams_embed: bad sizes (1..%d streams)", HS_MAX_STREAMS);
    if (num_tokens == 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == TI_F32)
        ti_launch(streams_embed_kernel<float>, num_tokens, threads, 0, stream, X, (const float*)table, ids, num_tokens, width, vocab, streams, scale);
    else if (dtype == TI_BF16)
        ti_launch(streams_embed_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, X, (const __nv_bfloat16*)table, ids, num_tokens, width, vocab, streams, scale);
    else TI_REQUIRE(false, "streams_embed: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("streams_embed");
    return 0;
}

// VEC neighbouring features at a time: 16-byte loads and stores of the float32 streams where rows allow it.
template <int VEC> struct HsVec;
template <> struct HsVec<1> {
    static __device__ __forceinline__ void load(const float* p, float* v) { v[0] = *p; }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) { v[0] = __bfloat162float(*p); }
    static __device__ __forceinline__ void store(float* p, const float* v) { *p = v[0]; }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) { *p = __float2bfloat16_rn(v[0]); }
};
template <> struct HsVec<4> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        uint2 u;
        *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

// TY: what the pending sublayer output y is stored in; TH: what h is stored in.
// NS: the most streams this instance is unrolled for (the arrays below live in registers).
template <typename TY, typename TH, int VEC, int NS>
__global__ void __launch_bounds__(VEC == 4 ? 256 : 512) streams_step_kernel(float* __restrict__ X, const TY* __restrict__ y, const float* __restrict__ c_mix,
                                    const float* __restrict__ c_out, const float* __restrict__ c_in,
                                    const float* __restrict__ norm_w, float eps, TH* __restrict__ h,
                                    const int* __restrict__ rows, int num_tokens, int width, int streams,
                                    const float* __restrict__ upd_w, float upd_eps) {
    extern __shared__ float urow[];
    __shared__ float red[33];
    __shared__ float mix[HS_MAX_STREAMS * HS_MAX_STREAMS], cout_s[HS_MAX_STREAMS], cin_s[HS_MAX_STREAMS];
    ti_grid_launch_dependents();
    if (threadIdx.x < streams * streams && y) mix[threadIdx.x] = c_mix[threadIdx.x];      // weights: not written by a kernel
    if (threadIdx.x < streams) {
        if (y) cout_s[threadIdx.x] = c_out[threadIdx.x];
        if (h) cin_s[threadIdx.x] = c_in[threadIdx.x];
    }
    ti_grid_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float y_inv = 1.f;
    if (y && upd_w) {                 // the update passes an RMS norm of its own first: its row's mean square
        float sy = 0.f;
        for (int i = threadIdx.x * VEC; i < width; i += blockDim.x * VEC) {
            float yv[VEC];
            HsVec<VEC>::load(y + (size_t)t * width + i, yv);
#pragma unroll
            for (int e = 0; e < VEC; ++e) sy += yv[e] * yv[e];
        }
        y_inv = rsqrtf(block_sum(sy, red) / (float)width + upd_eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < width; i += blockDim.x * VEC) {
        float x[NS][VEC];
#pragma unroll
        for (int s = 0; s < NS; ++s)
            if (s < streams) HsVec<VEC>::load(X + ((size_t)s * num_tokens + t) * width + i, x[s]);
        if (y) {
            float yv[VEC], fresh[NS][VEC];
            HsVec<VEC>::load(y + (size_t)t * width + i, yv);
            if (upd_w) {
                float uw[VEC];
                HsVec<VEC>::load(upd_w + i, uw);
#pragma unroll
                for (int e = 0; e < VEC; ++e) yv[e] = uw[e] * yv[e] * y_inv;
            }
#pragma unroll
            for (int to = 0; to < NS; ++to) {
                if (to < streams) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        float acc = 0.f;
#pragma unroll
                        for (int s = 0; s < NS; ++s)
                            if (s < streams) acc = fmaf(mix[s * streams + to], x[s][e], acc);
                        fresh[to][e] = fmaf(cout_s[to], yv[e], acc);
                    }
                }
            }
#pragma unroll
            for (int s = 0; s < NS; ++s)
                if (s < streams) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) x[s][e] = fresh[s][e];
                    HsVec<VEC>::store(X + ((size_t)s * num_tokens + t) * width + i, fresh[s]);
                }
        }
        if (h) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < NS; ++s)
                    if (s < streams) u = fmaf(cin_s[s], x[s][e], u);
                urow[i + e] = u;
                ss += u * u;
            }
        }
    }
    if (!h) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x * VEC; i < width; i += blockDim.x * VEC) {
        float w[VEC], o[VEC];
        HsVec<VEC>::load(norm_w + i, w);
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = w[e] * urow[i + e] * inv;
        HsVec<VEC>::store(h + (size_t)r * width + i, o);
    }
}

// y (may be null: nothing pending) with c_mix [S][S] (indexed [from][to]) and c_out [S]; h (may be null: only the
// update) with c_in [S] and norm_w [W]. rows (may be null): the tokens to work on; h then has one row per entry.
// upd_w (may be null; float32 [W]) with upd_eps: y is replaced by upd_w * y * rsqrt(mean(y^2) + upd_eps) before it is
// applied (a norm on a sublayer's output).
TI_API int ti_streams_step(float* X, const void* y, const float* c_mix, const float* c_out, const float* c_in,
                           const float* norm_w, float eps, void* h, const int* rows, int num_rows, int num_tokens, int width,
                           int streams, int y_dtype, int h_dtype, const float* upd_w, float upd_eps, cudaStream_t stream) {
    TI_REQUIRE(num_rows >= 0 && num_tokens >= 0 && width > 0 && streams >= 1 && streams <= HS_MAX_STREAMS,
               "streams_step: bad sizes (1..%d streams)", HS_MAX_STREAMS);
    TI_REQUIRE(width <= 48 * 1024 / 4, "streams_step: rows of %d features do not fit shared memory", width);
    TI_REQUIRE(!y || (c_mix && c_out), "streams_step: an update needs its coefficients");
    TI_REQUIRE(!h || (c_in && norm_w), "streams_step: a read needs its coefficients and the norm's weight");
    if (num_rows == 0 || (!y && !h)) return 0;
    const bool wide = width % 4 == 0 && ((uintptr_t)X | (uintptr_t)y | (uintptr_t)h | (uintptr_t)norm_w | (uintptr_t)upd_w) % 16 == 0 &&
                      ((size_t)num_tokens * width) % 4 == 0;
    int threads = 64;
    while (threads < (wide ? 256 : 512) && threads * 4 < width) threads <<= 1;
    const size_t smem = h ? (size_t)width * sizeof(float) : 0;
    typedef __nv_bfloat16 B;
#define TI_STEP_N(TY, TH, VEC, NS)                                                                                        \
    ti_launch(streams_step_kernel<TY, TH, VEC, NS>, num_rows, threads, smem, stream, X, (const TY*)y, c_mix, c_out, c_in, \
              norm_w, eps, (TH*)h, rows, num_tokens, width, streams, upd_w, upd_eps)
#define TI_STEP_V(TY, TH, VEC)                             \
    do {                                                   \
        if (streams == 1) TI_STEP_N(TY, TH, VEC, 1);       \
        else if (streams == 2) TI_STEP_N(TY, TH, VEC, 2);  \
        else if (streams <= 4) TI_STEP_N(TY, TH, VEC, 4);  \
        else TI_STEP_N(TY, TH, VEC, HS_MAX_STREAMS);       \
    } while (0)
#define TI_STEP(TY, TH)                    \
    do {                                   \
        if (wide) TI_STEP_V(TY, TH, 4);    \
        else TI_STEP_V(TY, TH, 1);         \
    } while (0)
    if (y_dtype == TI_F32 && h_dtype == TI_F32) TI_STEP(float, float);
    else if (y_dtype == TI_F32 && h_dtype == TI_BF16) TI_STEP(float, B);
    else if (y_dtype == TI_BF16 && h_dtype == TI_BF16) TI_STEP(B, B);
    else if (y_dtype == TI_BF16 && h_dtype == TI_F32) TI_STEP(B, float);
    else TI_REQUIRE(false, "streams_step: unknown dtypes %d, %d", y_dtype, h_dtype);
#undef TI_STEP
#undef TI_STEP_V
#undef TI_STEP_N
    TI_CHECK_LAUNCH("streams_step");
    return 0;
}

// ------------------------------------------------------------------ activation and scaling
// kind 0: the exact gelu 0.5 z (1 + erf(z / sqrt 2)); 1: its tanh form. In place or not; float32 arithmetic.
__device__ __forceinline__ float gelu_of(float z, int kind) {
    return kind == 0 ? 0.5f * z * (1.f + erff(z * 0.70710678118654752f))
                     : 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// 16 bytes a thread a trip where the tensors start on 16-byte boundaries; what is left at the end one by one.
template <typename T>
__global__ void gelu_kernel(T* __restrict__ out, const T* __restrict__ x, size_t n, int kind, int wide) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    constexpr int VEC = 16 / sizeof(T);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t groups = wide ? n / VEC : 0;
    for (size_t gi = first; gi < groups; gi += stride) {
        uint4 raw = reinterpret_cast<const uint4*>(x)[gi];
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int j = 0; j < VEC; ++j) e[j] = from_f32<T>(gelu_of(to_f32(e[j]), kind));
        reinterpret_cast<uint4*>(out)[gi] = raw;
    }
    for (size_t i = groups * VEC + first; i < n; i += stride) out[i] = from_f32<T>(gelu_of(to_f32(x[i]), kind));
}

TI_API int ti_gelu(void* out, const void* x, long long n, int kind, int dtype, cudaStream_t stream) {
    TI_REQUIRE(n >= 0 && (kind == 0 || kind == 1), "gelu: bad arguments");
    if (n == 0) return 0;
    const int threads = 256;
    const int wide = ((uintptr_t)out | (uintptr_t)x) % 16 == 0;
    const long long want = (n / (dtype == TI_F32 ? 4 : 8) + threads - 1) / threads + 1;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == TI_F32)
        ti_launch(gelu_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)x, (size_t)n, kind, wide);
    else if (dtype == TI_BF16)
        ti_launch(gelu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, (size_t)n, kind, wide);
    else TI_REQUIRE(false, "gelu: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("gelu");
    return 0;
}

__global__ void scale_kernel(float* __restrict__ x, size_t n, float factor) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] *= factor;
}

TI_API int ti_scale(float* x, long long n, float factor, cudaStream_t stream) {
    TI_REQUIRE(n >= 0, "scale: bad size");
    if (n == 0) return 0;
    const long long want = (n + 255) / 256;
    ti_launch(scale_kernel, (int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream, x, (size_t)n, factor);
    TI_CHECK_LAUNCH("scale");
    return 0;
}

__global__ void soft_cap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = cap * tanhf(x[i] * inv_cap);
}

// x <- cap * tanh(x / cap) in place (float32): logits that level off smoothly at +-cap.
TI_API int ti_soft_cap(float* x, long long n, float cap, cudaStream_t stream) {
    TI_REQUIRE(n >= 0 && cap > 0.f, "soft_cap: bad arguments");
    if (n == 0) return 0;
    const long long want = (n + 255) / 256;
    ti_launch(soft_cap_kernel, (int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream, x, (size_t)n, cap, 1.f / cap);
    TI_CHECK_LAUNCH("soft_cap");
    return 0;
}
