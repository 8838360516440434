// Per-head norm and rotary rotation of packed rows [q | k | v] whose pieces may differ in size, for mixers that
// are not served by the fused kernel of the plain decoder (rope_append.cu): keys and values of different sizes,
// rows that hold more than q, k and v, layers that only have queries, and mixers that keep no pages at all.
//   in  : rows of ld_in elements, first column in_off: Hq heads of d query features, then (has_kv) Hkv heads of d key
//         features and Hkv heads of dv value features
//   q, k: optional RMS norm over the head with a plain weight, then the rotation of the first rotary_dim features
//         (same rotation data as rope_append.cu: inverse frequencies or a table of cosines and sines, half-split or
//         interleaved pairs; rot_factor multiplies every cosine and sine), then a constant factor (q_scale, k_scale);
//         v passes unchanged. norm_after != 0: the RMS norm comes AFTER the rotation instead, with the weight or, if
//         there is none, without one (x / rms(x))
//   out : q goes to out[t][head * d] (rows of ld_out). With a cache, k and v go to the token's place in its page:
//         planes 2 (d == dv): [2][pages][Hkv][page][d]; planes 1: rows [k (d) | v (dv)]. Without a cache and with
//         has_kv, k and v follow q in the row of out: [q | k | v], so that a recurrent mixer reads them from there.
// One warp a (token, head); float32 arithmetic, one rounding at the store. OutT may be float32 for a bfloat16 input:
// what enters a float32 recurrence is then never rounded after its rotation.
#include "common.cuh"

constexpr int HR_WARPS = 4;
constexpr int HR_MAX_D = 512;

struct HeadRotationArgs {
    void* out; int ld_out;
    void* cache; int planes; long long v_plane_off;
    const void* in; int ld_in, in_off;
    const float *q_w, *k_w; float eps;
    const float *inv_freq, *table; int table_positions, interleaved, rotary_dim;
    float q_scale, k_scale, rot_factor; int norm_after;
    const int *positions, *token_seq, *block_table; int max_blocks;
    int hq, hkv, d, dv, has_kv, page_size, num_pages;
    int* status;
};

template <typename T, typename OutT>
__global__ void __launch_bounds__(HR_WARPS * 32) head_rotation_kernel(HeadRotationArgs a) {
    __shared__ float buf[HR_WARPS][HR_MAX_D];
    __shared__ float turned[HR_WARPS][HR_MAX_D];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x * HR_WARPS + warp;
    const int t = blockIdx.y;
    const int heads_total = a.hq + (a.has_kv ? 2 * a.hkv : 0);
    if (head >= heads_total) return;
    const bool is_q = head < a.hq;
    const bool is_k = !is_q && head < a.hq + a.hkv;
    const int size = (is_q || is_k) ? a.d : a.dv;
    const int col = is_q ? head * a.d : is_k ? a.hq * a.d + (head - a.hq) * a.d
                                             : (a.hq + a.hkv) * a.d + (head - a.hq - a.hkv) * a.dv;
    const T* src = (const T*)a.in + (size_t)t * a.ld_in + a.in_off + col;
    float* x = buf[warp];
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) {
        const float v = to_f32(src[i]);
        x[i] = v;
        ss += v * v;
    }
    const float* w = is_q ? a.q_w : (is_k ? a.k_w : nullptr);
    const bool norm_last = a.norm_after && (is_q || is_k);
    if (w != nullptr && !norm_last) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)size + a.eps);
        for (int i = lane; i < size; i += 32) x[i] = w[i] * x[i] * inv;
    }
    __syncwarp();
    const int pos = a.positions[t];
    const bool rotate = (is_q || is_k) && (a.inv_freq != nullptr || a.table != nullptr) && a.rotary_dim > 0;
    if (rotate && a.table != nullptr && (pos < 0 || pos >= a.table_positions)) {
        if (lane == 0 && a.status) atomicExch(a.status, 4);          // a position the table does not reach
        return;
    }
    const float factor = is_q ? a.q_scale : is_k ? a.k_scale : 1.f;
    T* cdst = nullptr;
    OutT* odst = nullptr;
    if (is_q || a.cache == nullptr) {
        odst = (OutT*)a.out + (size_t)t * a.ld_out + col;
    } else {
        const int logical = pos / a.page_size;
        const int page = logical < a.max_blocks ? a.block_table[(size_t)a.token_seq[t] * a.max_blocks + logical] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (lane == 0 && a.status) atomicExch(a.status, 1);      // a token without a page: never write
            return;
        }
        const int kvh = is_k ? head - a.hq : head - a.hq - a.hkv;
        const size_t place = ((size_t)page * a.hkv + kvh) * a.page_size + pos % a.page_size;
        if (a.planes == 2) cdst = (T*)a.cache + (is_k ? 0 : a.v_plane_off) + place * a.d;
        else cdst = (T*)a.cache + place * (a.d + a.dv) + (is_k ? 0 : a.d);
    }
    const int half = a.rotary_dim >> 1;
    const float pos_f = (float)pos;
    float* y = turned[warp];
    float ss_after = 0.f;
    for (int i = lane; i < size; i += 32) {
        float o = x[i];
        if (rotate && i < a.rotary_dim) {
            const int j = a.interleaved ? (i >> 1) : (i < half ? i : i - half);
            const bool first = a.interleaved ? !(i & 1) : i < half;
            const int other = a.interleaved ? (i ^ 1) : (i < half ? i + half : i - half);
            float s, c;
            if (a.table != nullptr) {
                c = a.table[(size_t)pos * a.rotary_dim + j];
                s = a.table[(size_t)pos * a.rotary_dim + half + j];
            } else {
                sincosf(pos_f * a.inv_freq[j], &s, &c);
            }
            c *= a.rot_factor;
            s *= a.rot_factor;
            o = first ? x[i] * c - x[other] * s : x[i] * c + x[other] * s;
        }
        y[i] = o;                                   // read back by this lane alone
        ss_after += o * o;
    }
    float inv_after = 1.f;
    if (norm_last) inv_after = rsqrtf(warp_sum(ss_after) / (float)size + a.eps);
    for (int i = lane; i < size; i += 32) {
        float o = y[i];
        if (norm_last) o = (w != nullptr ? w[i] : 1.f) * o * inv_after;
        o *= factor;
        if (cdst) cdst[i] = from_f32<T>(o);
        else odst[i] = from_f32<OutT>(o);
    }
}

// dtype: of `in` and of the cache; out_f32 != 0: `out` is float32 whatever the dtype.
TI_API int ti_head_rotation(void* out, int ld_out, void* cache, int planes, const void* in, int ld_in, int in_off,
                            const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq,
                            const float* cos_sin_table, int table_positions, int interleaved, int rotary_dim, float rot_factor, float q_scale,
                            float k_scale, const int* positions, const int* token_seq, const int* block_table,
                            int max_blocks, int num_tokens, int hq, int hkv, int d, int dv, int has_kv, int page_size,
                            int num_pages, int* status, int out_f32, int norm_after, int dtype, cudaStream_t stream) {
    TI_REQUIRE(d > 0 && d <= HR_MAX_D && dv > 0 && dv <= HR_MAX_D, "head_rotation: head sizes %d / %d not in 1..%d", d, dv, HR_MAX_D);
    TI_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
               "head_rotation: rotary_dim %d must be even and at most the head size %d", rotary_dim, d);
    TI_REQUIRE(hq > 0 && hkv >= 0 && num_tokens >= 0, "head_rotation: bad sizes");
    TI_REQUIRE(inv_freq == nullptr || cos_sin_table == nullptr, "head_rotation: inverse frequencies or a table, not both");
    TI_REQUIRE(cos_sin_table == nullptr || table_positions > 0, "head_rotation: a table needs its number of positions");
    TI_REQUIRE(cache == nullptr || (has_kv && (planes == 1 || (planes == 2 && d == dv)) && page_size > 0 && block_table),
               "head_rotation: a cache of two planes needs keys and values of one size");
    TI_REQUIRE(num_tokens <= 65535, "head_rotation: more than 65535 tokens in one step");
    if (num_tokens == 0) return 0;
    HeadRotationArgs a = {out, ld_out, cache, planes, (long long)num_pages * hkv * page_size * d, in, ld_in, in_off,
                          q_norm_w, k_norm_w, eps, inv_freq, cos_sin_table, table_positions, interleaved, rotary_dim,
                          q_scale, k_scale, rot_factor, norm_after ? 1 : 0, positions, token_seq, block_table, max_blocks, hq, hkv, d, dv, has_kv ? 1 : 0,
                          page_size, num_pages, status};
    const int heads_total = hq + (has_kv ? 2 * hkv : 0);
    dim3 grid((heads_total + HR_WARPS - 1) / HR_WARPS, num_tokens);
    if (dtype == TI_F32) ti_launch(head_rotation_kernel<float, float>, grid, HR_WARPS * 32, 0, stream, a);
    else if (dtype == TI_BF16 && out_f32) ti_launch(head_rotation_kernel<__nv_bfloat16, float>, grid, HR_WARPS * 32, 0, stream, a);
    else if (dtype == TI_BF16) ti_launch(head_rotation_kernel<__nv_bfloat16, __nv_bfloat16>, grid, HR_WARPS * 32, 0, stream, a);
    else TI_REQUIRE(false, "head_rotation: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("head_rotation");
    return 0;
}
