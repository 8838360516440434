// Short causal convolutions over time with their per-request history, and softmax attention over pages whose
// rows hold a token's key and value side by side (so keys and values may differ in size).
//
// A convolution of `taps` taps reads the current token and the taps - 1 before it. Inputs of earlier steps come
// from the request's state slot: `hist` float32 [taps - 1][width], oldest first, zero when the request starts
// (which is "zeros before the start"). The slots lie `slot_stride` floats apart, so the history may be a slice of
// a larger per-request state.
//   short_conv        : out[t][c] = act(bias[c] + sum_j w[j][c] * in[t - (taps - 1 - j)][c]),  act: none or silu
//                       (the weights lie tap by tap, [taps][channels], so that neighbouring channels are neighbours)
//   conv_qkv_append   : the same on the packed rows [q | k | v] of an attention layer, without bias or activation;
//                       q is multiplied by its position's temperature 1 + coef * ln(floor((p + 1) / every) + 1)
//                       and stored as [T][Hq][d]; k and v go to the token's row of its page: [k (d) | v (dv)], or,
//                       where keys and values have the same size, to the two planes [keys][values] of the cache
//   conv_state_update : the step's last taps - 1 inputs of every request become its history
//   attention_rows    : causal attention of q over such pages, float32 arithmetic, any sizes; optionally the
//                       softmax denominator holds one more term exp(sink) that has no value ("sink")
// Everything is computed in float32 from the stored operands; each result is rounded once.
#include "common.cuh"

constexpr int SC_MAX_TAPS = 16;

template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ in, int ld_in, int col, int t, int local,
                                         const float* __restrict__ hist, int width, int c,
                                         const float* __restrict__ w, int taps) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {                       // column taps - 1 meets the current token
        const int back = taps - 1 - j;
        const float v = local - back >= 0 ? to_f32(in[(size_t)(t - back) * ld_in + col])
                                          : hist[(size_t)(taps - 1 + local - back) * width + c];
        acc = fmaf(w[(size_t)j * width + c], v, acc);
    }
    return acc;
}

// A step in which every request brings ONE token: the thread that made the token's output is the only one that
// read this channel's history, so it may also move the history on by one (oldest out, the token's input in).
__device__ __forceinline__ void conv_shift_history(float* __restrict__ hist, int width, int c, int taps, float newest) {
    float kept[SC_MAX_TAPS];
    for (int j = 1; j < taps - 1; ++j) kept[j] = hist[(size_t)j * width + c];
    for (int j = 1; j < taps - 1; ++j) hist[(size_t)(j - 1) * width + c] = kept[j];
    hist[(size_t)(taps - 2) * width + c] = newest;
}

// ------------------------------------------------------------------ sixteen bytes of channels a thread
// The *_vec kernels do the same as short_conv_kernel and conv_qkv_append_kernel for rows whose pieces (q, k, v, a
// head) all start on 16-byte boundaries: a thread takes V = 16 / sizeof(T) neighbouring channels, one load per tap, one store.
template <typename T, int V>
__device__ __forceinline__ void load_row(const T* __restrict__ p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = to_f32(e[i]);
}
template <typename T, int V>
__device__ __forceinline__ void store_row(T* __restrict__ p, const float* v) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < V; ++i) e[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// acc[i] = sum_j w[j][c0 + i] * in(t - (taps - 1 - j))[c0 + i]; newest[i]: the current token's own input.
template <typename T, int V>
__device__ __forceinline__ void conv_at_vec(const T* __restrict__ in, int ld_in, int col0, int t, int local,
                                            const float* __restrict__ hist, int width, int c0,
                                            const float* __restrict__ w, int taps, float* acc, float* newest) {
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        float v[V];
        if (local - back >= 0) {
            load_row<T, V>(in + (size_t)(t - back) * ld_in + col0, v);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) v[i] = hist[(size_t)(taps - 1 + local - back) * width + c0 + i];
        }
        float wj[V];
        if (w) {
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                const float4 f = *reinterpret_cast<const float4*>(w + (size_t)j * width + c0 + i);
                wj[i] = f.x; wj[i + 1] = f.y; wj[i + 2] = f.z; wj[i + 3] = f.w;
            }
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(w ? wj[i] : 1.f, v[i], acc[i]);
        if (back == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i) newest[i] = v[i];
        }
    }
}

template <typename T>
__global__ void short_conv_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int ld_in, int in_off,
                                      const float* __restrict__ state, long long slot_stride, const float* __restrict__ w,
                                      const float* __restrict__ bias, const int* __restrict__ token_seq,
                                      const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int width,
                                      int taps, int act, int shift_history) {
    constexpr int V = 16 / sizeof(T);
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.y;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (c0 >= width) return;
    const int seq = token_seq[t];
    const int local = t - cu_seqlens[seq];
    const float* hist = state + (size_t)state_slots[seq] * slot_stride;
    float acc[V], newest[V];
    conv_at_vec<T, V>(in, ld_in, in_off + c0, t, local, hist, width, c0, w, taps, acc, newest);
    if (shift_history && taps > 1) {
#pragma unroll
        for (int i = 0; i < V; ++i) conv_shift_history(const_cast<float*>(hist), width, c0 + i, taps, newest[i]);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
        if (bias) acc[i] += bias[c0 + i];
        if (act == 1) acc[i] = acc[i] / (1.f + expf(-acc[i]));
    }
    store_row<T, V>(out + (size_t)t * width + c0, acc);
}

template <typename T>
__global__ void conv_qkv_append_vec_kernel(T* __restrict__ q_out, T* __restrict__ cache, const T* __restrict__ qkv,
                                           int ld_in, int in_off, const float* __restrict__ state, long long slot_stride,
                                           const float* __restrict__ w, int taps, float temp_coef, int temp_every,
                                           const int* __restrict__ positions, const int* __restrict__ token_seq,
                                           const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                           const int* __restrict__ block_table, int max_blocks, int hq, int hkv, int d,
                                           int dv, int page_size, int num_pages, int row_stride, long long v_off,
                                           int shift_history, int* __restrict__ status) {
    constexpr int V = 16 / sizeof(T);
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.y;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int cq = hq * d, ck = hkv * d, width = cq + ck + hkv * dv;
    if (c0 >= width) return;
    const int seq = token_seq[t];
    const int local = t - cu_seqlens[seq];
    const float* hist = taps > 1 ? state + (size_t)state_slots[seq] * slot_stride : nullptr;
    float acc[V], newest[V];
    conv_at_vec<T, V>(qkv, ld_in, in_off + c0, t, local, hist, width, c0, w, taps, acc, newest);
    if (shift_history && taps > 1) {
#pragma unroll
        for (int i = 0; i < V; ++i) conv_shift_history(const_cast<float*>(hist), width, c0 + i, taps, newest[i]);
    }
    const int pos = positions[t];
    if (c0 < cq) {
        if (temp_every > 0) {
            const float f = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] *= f;
        }
        store_row<T, V>(q_out + (size_t)t * cq + c0, acc);
        return;
    }
    if (!cache) return;
    const int logical = pos / page_size;
    const int page = logical < max_blocks ? block_table[(size_t)seq * max_blocks + logical] : -1;
    if (page < 0 || page >= num_pages) {
        if (status) atomicExch(status, 1);                 // a token without a page
        return;
    }
    int head;
    long long off;
    if (c0 < cq + ck) { head = (c0 - cq) / d; off = (c0 - cq) % d; }
    else { head = (c0 - cq - ck) / dv; off = v_off + (c0 - cq - ck) % dv; }
    store_row<T, V>(cache + (((size_t)page * hkv + head) * page_size + pos % page_size) * row_stride + off, acc);
}

template <typename T>
__global__ void short_conv_kernel(T* __restrict__ out, const T* __restrict__ in, int ld_in, int in_off,
                                  const float* __restrict__ state, long long slot_stride, const float* __restrict__ w,
                                  const float* __restrict__ bias, const int* __restrict__ token_seq,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int width,
                                  int taps, int act, int shift_history) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int seq = token_seq[t];
    const int local = t - cu_seqlens[seq];
    const float* hist = state + (size_t)state_slots[seq] * slot_stride;
    float v = conv_at(in, ld_in, in_off + c, t, local, hist, width, c, w, taps);
    if (shift_history && taps > 1)
        conv_shift_history(const_cast<float*>(hist), width, c, taps, to_f32(in[(size_t)t * ld_in + in_off + c]));
    if (bias) v += bias[c];
    if (act == 1) v = v / (1.f + expf(-v));
    out[(size_t)t * width + c] = from_f32<T>(v);
}

// shift_history: every request of the step brings one token, and the kernel also moves the histories on (otherwise
// conv_state_update does, afterwards).
TI_API int ti_short_conv(void* out, const void* in, int ld_in, int in_off, float* state, long long slot_stride,
                         const float* w, const float* bias, const int* token_seq, const int* cu_seqlens,
                         const int* state_slots, int num_tokens, int width, int taps, int act, int shift_history, int dtype,
                         cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && width > 0 && taps >= 1 && taps <= SC_MAX_TAPS, "short_conv: bad sizes (taps 1..%d)", SC_MAX_TAPS);
    TI_REQUIRE(num_tokens <= 65535, "short_conv: more than 65535 tokens in one step");
    TI_REQUIRE(act == 0 || act == 1, "short_conv: unknown activation %d", act);
    if (num_tokens == 0) return 0;
    // sixteen bytes of channels a thread where every piece allows it and the step has tokens enough to fill the machine so
    const int vec = dtype == TI_F32 ? 4 : 8;
    if (num_tokens >= 64 && width % vec == 0 && ld_in % vec == 0 && in_off % vec == 0 && ((uintptr_t)out | (uintptr_t)in | (uintptr_t)w) % 16 == 0) {
        dim3 vgrid((width / vec + 127) / 128, num_tokens);
        if (dtype == TI_F32)
            ti_launch(short_conv_vec_kernel<float>, vgrid, 128, 0, stream, (float*)out, (const float*)in, ld_in, in_off,
                      (const float*)state, slot_stride, w, bias, token_seq, cu_seqlens, state_slots, width, taps, act, shift_history);
        else if (dtype == TI_BF16)
            ti_launch(short_conv_vec_kernel<__nv_bfloat16>, vgrid, 128, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)in,
                      ld_in, in_off, (const float*)state, slot_stride, w, bias, token_seq, cu_seqlens, state_slots, width, taps,
                      act, shift_history);
        else TI_REQUIRE(false, "short_conv: unknown dtype %d", dtype);
        TI_CHECK_LAUNCH("short_conv");
        return 0;
    }
    dim3 grid((width + 127) / 128, num_tokens);
    if (dtype == TI_F32)
        ti_launch(short_conv_kernel<float>, grid, 128, 0, stream, (float*)out, (const float*)in, ld_in, in_off, (const float*)state, slot_stride,
                  w, bias, token_seq, cu_seqlens, state_slots, width, taps, act, shift_history);
    else if (dtype == TI_BF16)
        ti_launch(short_conv_kernel<__nv_bfloat16>, grid, 128, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)in, ld_in,
                  in_off, (const float*)state, slot_stride, w, bias, token_seq, cu_seqlens, state_slots, width, taps, act, shift_history);
    else TI_REQUIRE(false, "short_conv: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("short_conv");
    return 0;
}

// One thread per (request, channel): reads the taps - 1 values that will be the history (from the step's rows,
// or, where the step was shorter than that, from the old history) and only then writes them.
template <typename T>
__global__ void conv_state_update_kernel(float* __restrict__ state, long long slot_stride, const T* __restrict__ in,
                                         int ld_in, int in_off, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ state_slots, int width, int taps) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int row0 = cu_seqlens[seq], n = cu_seqlens[seq + 1] - row0;
    float* hist = state + (size_t)state_slots[seq] * slot_stride;
    const int keep = taps - 1;
    float fresh[SC_MAX_TAPS];
    for (int j = 0; j < keep; ++j) {
        const int idx = n - keep + j;                      // the step's row that becomes entry j
        fresh[j] = idx >= 0 ? to_f32(in[(size_t)(row0 + idx) * ld_in + in_off + c]) : hist[(size_t)(keep + idx) * width + c];
    }
    for (int j = 0; j < keep; ++j) hist[(size_t)j * width + c] = fresh[j];
}

TI_API int ti_conv_state_update(float* state, long long slot_stride, const void* in, int ld_in, int in_off,
                                const int* cu_seqlens, const int* state_slots, int num_seqs, int width, int taps, int dtype,
                                cudaStream_t stream) {
    TI_REQUIRE(num_seqs >= 0 && width > 0 && taps >= 1 && taps <= SC_MAX_TAPS, "conv_state_update: bad sizes");
    TI_REQUIRE(num_seqs <= 65535, "conv_state_update: too many requests");
    if (num_seqs == 0 || taps == 1) return 0;
    dim3 grid((width + 127) / 128, num_seqs);
    if (dtype == TI_F32)
        ti_launch(conv_state_update_kernel<float>, grid, 128, 0, stream, state, slot_stride, (const float*)in, ld_in, in_off,
                  cu_seqlens, state_slots, width, taps);
    else if (dtype == TI_BF16)
        ti_launch(conv_state_update_kernel<__nv_bfloat16>, grid, 128, 0, stream, state, slot_stride, (const __nv_bfloat16*)in,
                  ld_in, in_off, cu_seqlens, state_slots, width, taps);
    else TI_REQUIRE(false, "conv_state_update: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("conv_state_update");
    return 0;
}

template <typename T>
__global__ void conv_qkv_append_kernel(T* __restrict__ q_out, T* __restrict__ cache, const T* __restrict__ qkv, int ld_in,
                                       int in_off, const float* __restrict__ state, long long slot_stride, const float* __restrict__ w,
                                       int taps, float temp_coef, int temp_every, const int* __restrict__ positions,
                                       const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                                       const int* __restrict__ state_slots, const int* __restrict__ block_table,
                                       int max_blocks, int hq, int hkv, int d, int dv, int page_size, int num_pages,
                                       int row_stride, long long v_off, int shift_history, int* __restrict__ status) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int cq = hq * d, ck = hkv * d, width = cq + ck + hkv * dv;
    if (c >= width) return;
    const int seq = token_seq[t];
    const int local = t - cu_seqlens[seq];
    const float* hist = taps > 1 ? state + (size_t)state_slots[seq] * slot_stride : nullptr;
    float v = taps > 1 ? conv_at(qkv, ld_in, in_off + c, t, local, hist, width, c, w, taps)
                       : (w ? w[c] : 1.f) * to_f32(qkv[(size_t)t * ld_in + in_off + c]);     // one tap: [1][width]
    if (shift_history && taps > 1)
        conv_shift_history(const_cast<float*>(hist), width, c, taps, to_f32(qkv[(size_t)t * ld_in + in_off + c]));
    const int pos = positions[t];
    if (c < cq) {
        if (temp_every > 0) v *= 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
        q_out[(size_t)t * cq + c] = from_f32<T>(v);
        return;
    }
    if (!cache) return;
    const int logical = pos / page_size;
    const int page = logical < max_blocks ? block_table[(size_t)seq * max_blocks + logical] : -1;
    if (page < 0 || page >= num_pages) {
        if (status) atomicExch(status, 1);                 // a token without a page
        return;
    }
    int head;
    long long off;
    if (c < cq + ck) { head = (c - cq) / d; off = (c - cq) % d; }
    else { head = (c - cq - ck) / dv; off = v_off + (c - cq - ck) % dv; }
    cache[(((size_t)page * hkv + head) * page_size + pos % page_size) * row_stride + off] = from_f32<T>(v);
}

// w: float32 [taps][width] over the packed channels (may be null with taps == 1: no convolution at all).
// planes 1: cache [pages][hkv][page_size][d + dv]; planes 2 (d == dv): [2][pages][hkv][page_size][d].
// shift_history: as in ti_short_conv. The packed rows are columns [in_off, in_off + width) of rows of ld_in elements.
TI_API int ti_conv_qkv_append(void* q_out, void* cache, const void* qkv, int ld_in, int in_off, float* state, long long slot_stride,
                              const float* w, int taps, float temp_coef, int temp_every, const int* positions,
                              const int* token_seq, const int* cu_seqlens, const int* state_slots, const int* block_table,
                              int max_blocks, int num_tokens, int hq, int hkv, int d, int dv, int page_size, int num_pages,
                              int planes, int shift_history, int* status, int dtype, cudaStream_t stream) {
    TI_REQUIRE(planes == 1 || (planes == 2 && d == dv), "conv_qkv_append: two planes need keys and values of one size");
    const int row_stride = planes == 2 ? d : d + dv;
    const long long v_off = planes == 2 ? (long long)num_pages * hkv * page_size * d : d;
    TI_REQUIRE(num_tokens >= 0 && hq > 0 && hkv > 0 && d > 0 && dv > 0 && taps >= 1 && taps <= SC_MAX_TAPS,
               "conv_qkv_append: bad sizes (taps 1..%d)", SC_MAX_TAPS);
    TI_REQUIRE(taps == 1 || (w && state), "conv_qkv_append: a convolution needs its weights and the history");
    TI_REQUIRE(num_tokens <= 65535, "conv_qkv_append: more than 65535 tokens in one step");
    TI_REQUIRE(temp_every >= 0 && page_size > 0, "conv_qkv_append: bad constants");
    if (num_tokens == 0) return 0;
    const int width = hq * d + hkv * (d + dv);
    const int vec = dtype == TI_F32 ? 4 : 8;
    TI_REQUIRE(in_off >= 0 && ld_in >= in_off + width, "conv_qkv_append: the packed rows do not fit their tensor's rows");
    if (num_tokens >= 64 && d % vec == 0 && dv % vec == 0 && ld_in % vec == 0 && in_off % vec == 0 && ((uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)qkv | (uintptr_t)w) % 16 == 0) {
        dim3 vgrid((width / vec + 127) / 128, num_tokens);
        if (dtype == TI_F32)
            ti_launch(conv_qkv_append_vec_kernel<float>, vgrid, 128, 0, stream, (float*)q_out, (float*)cache, (const float*)qkv,
                      ld_in, in_off, (const float*)state, slot_stride, w, taps, temp_coef, temp_every, positions, token_seq, cu_seqlens,
                      state_slots, block_table, max_blocks, hq, hkv, d, dv, page_size, num_pages, row_stride, v_off,
                      shift_history, status);
        else if (dtype == TI_BF16)
            ti_launch(conv_qkv_append_vec_kernel<__nv_bfloat16>, vgrid, 128, 0, stream, (__nv_bfloat16*)q_out,
                      (__nv_bfloat16*)cache, (const __nv_bfloat16*)qkv, ld_in, in_off, (const float*)state, slot_stride, w, taps,
                      temp_coef, temp_every, positions, token_seq, cu_seqlens, state_slots, block_table, max_blocks, hq, hkv, d, dv,
                      page_size, num_pages, row_stride, v_off, shift_history, status);
        else TI_REQUIRE(false, "conv_qkv_append: unknown dtype %d", dtype);
        TI_CHECK_LAUNCH("conv_qkv_append");
        return 0;
    }
    dim3 grid((width + 127) / 128, num_tokens);
    if (dtype == TI_F32)
        ti_launch(conv_qkv_append_kernel<float>, grid, 128, 0, stream, (float*)q_out, (float*)cache, (const float*)qkv, ld_in, in_off,
                  (const float*)state,
                  slot_stride, w, taps, temp_coef, temp_every, positions, token_seq, cu_seqlens, state_slots, block_table,
                  max_blocks, hq, hkv, d, dv, page_size, num_pages, row_stride, v_off, shift_history, status);
    else if (dtype == TI_BF16)
        ti_launch(conv_qkv_append_kernel<__nv_bfloat16>, grid, 128, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache,
                  (const __nv_bfloat16*)qkv, ld_in, in_off, (const float*)state, slot_stride, w, taps, temp_coef, temp_every, positions, token_seq,
                  cu_seqlens, state_slots, block_table, max_blocks, hq, hkv, d, dv, page_size, num_pages, row_stride, v_off,
                  shift_history, status);
    else TI_REQUIRE(false, "conv_qkv_append: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("conv_qkv_append");
    return 0;
}

// ------------------------------------------------------------------ attention over [k | v] rows, float32 arithmetic
// One block per (token, query head). The running maximum starts at the sink's logit and the running sum at 1 when
// there is a sink: the sink is a key without a value.
constexpr int AR_THREADS = 128;
constexpr int AR_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(AR_THREADS) attention_rows_kernel(
    T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ positions,
    const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks, int hq, int hkv, int d, int dv,
    int page_size, int num_pages, int row, long long v_off, float scale, int window, int has_sink, float sink,
    const float* __restrict__ head_sinks, const T* __restrict__ gate, int ld_gate, int gate_off,
    float out_scale, float softcap, int* __restrict__ status) {
    __shared__ float qs[AR_MAX_D];
    __shared__ float p[AR_THREADS];
    __shared__ long long row_off[AR_THREADS];
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int tid = threadIdx.x;
    const int h = blockIdx.x, t = blockIdx.y;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int kvh = h / (hq / hkv);
    const int* table = block_table + (size_t)token_seq[t] * max_blocks;
    const T* qrow = q + ((size_t)t * hq + h) * d;
    for (int i = tid; i < d; i += AR_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();

    float acc0 = 0.f, acc1 = 0.f;
    if (head_sinks) { has_sink = 1; sink = head_sinks[h]; }            // a learned sink per query head
    if (gate) {                                                          // a sigmoid gate per (token, query head)
        const float z = to_f32(gate[(size_t)t * ld_gate + gate_off + h]);
        out_scale *= 1.f / (1.f + expf(-z));
    }
    float m = has_sink ? sink : -INFINITY, l = has_sink ? 1.f : 0.f;
    for (int tile0 = lo; tile0 <= pos; tile0 += AR_THREADS) {
        const int j = tile0 + tid;
        float s = -INFINITY;
        long long off = -1;
        if (j <= pos) {
            const int logical = j / page_size;
            const int page = logical < max_blocks ? table[logical] : -1;
            if (page >= 0 && page < num_pages) {
                off = (((long long)page * hkv + kvh) * page_size + j % page_size) * row;
                const T* krow = cache + off;
                float dot = 0.f;
                for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
                s = dot * scale;
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);      // scores level off smoothly at +-softcap
            } else if (status) {
                atomicExch(status, 2);                 // a visible key without a page
            }
        }
        const float tile_max = block_max(s, red);
        const float m_new = fmaxf(m, tile_max);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
        p[tid] = pj;
        row_off[tid] = off;
        const float tile_sum = block_sum(pj, red);      // also orders the writes of p and row_off
        l = l * corr + tile_sum;
        acc0 *= corr;
        acc1 *= corr;
        m = m_new;
        const int n = min(AR_THREADS, pos + 1 - tile0);
        if (tid < dv) {
            for (int jj = 0; jj < n; ++jj) {
                const long long o = row_off[jj];
                if (o < 0) continue;
                const float pv = p[jj];
                acc0 = fmaf(pv, to_f32(cache[o + v_off + tid]), acc0);
                if (tid + AR_THREADS < dv) acc1 = fmaf(pv, to_f32(cache[o + v_off + tid + AR_THREADS]), acc1);
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)t * hq + h) * dv;
    const float inv = l > 0.f ? out_scale / l : 0.f;
    if (tid < dv) orow[tid] = from_f32<T>(acc0 * inv);
    if (tid + AR_THREADS < dv) orow[tid + AR_THREADS] = from_f32<T>(acc1 * inv);
}

// planes 1: cache [pages][hkv][page_size][d + dv]; planes 2 (d == dv): [2][pages][hkv][page_size][d].
// out: [T][hq * dv], multiplied by out_scale before its one rounding. head_sinks (float32 [hq], or null): a sink's
// logit per query head in place of the one `sink`; gate (compute dtype, rows of ld_gate, first column gate_off, or
// null): the output of (token, head) is also multiplied by sigmoid(gate[token][head]). softcap > 0: a score s becomes
// softcap * tanh(s / softcap) before the softmax.
TI_API int ti_attention_rows(void* out, const void* q, const void* cache, const int* positions, const int* token_seq,
                             const int* block_table, int max_blocks, int num_tokens, int hq, int hkv, int d, int dv,
                             int page_size, int num_pages, int planes, float scale, int window, int has_sink, float sink,
                             const float* head_sinks, const void* gate, int ld_gate, int gate_off,
                             float out_scale, float softcap, int* status, int dtype, cudaStream_t stream) {
    TI_REQUIRE(planes == 1 || (planes == 2 && d == dv), "attention_rows: two planes need keys and values of one size");
    const int row = planes == 2 ? d : d + dv;
    const long long v_off = planes == 2 ? (long long)num_pages * hkv * page_size * d : d;
    TI_REQUIRE(d > 0 && d <= AR_MAX_D && dv > 0 && dv <= AR_MAX_D, "attention_rows: head sizes %d / %d not in 1..%d", d, dv, AR_MAX_D);
    TI_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, "attention_rows: %d query heads do not group over %d kv heads", hq, hkv);
    TI_REQUIRE(page_size > 0 && num_tokens >= 0 && window >= 0 && softcap >= 0.f, "attention_rows: bad sizes");
    TI_REQUIRE(num_tokens <= 65535, "attention_rows: more than 65535 tokens in one step");
    if (num_tokens == 0) return 0;
    dim3 grid(hq, num_tokens);
    if (dtype == TI_F32)
        ti_launch(attention_rows_kernel<float>, grid, AR_THREADS, 0, stream, (float*)out, (const float*)q, (const float*)cache,
                  positions, token_seq, block_table, max_blocks, hq, hkv, d, dv, page_size, num_pages, row, v_off, scale, window,
                  has_sink, sink, head_sinks, (const float*)gate, ld_gate, gate_off, out_scale, softcap, status);
    else if (dtype == TI_BF16)
        ti_launch(attention_rows_kernel<__nv_bfloat16>, grid, AR_THREADS, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)cache, positions, token_seq, block_table, max_blocks, hq, hkv, d, dv, page_size,
                  num_pages, row, v_off, scale, window, has_sink, sink, head_sinks, (const __nv_bfloat16*)gate, ld_gate, gate_off,
                  out_scale, softcap, status);
    else TI_REQUIRE(false, "attention_rows: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("attention_rows");
    return 0;
}
