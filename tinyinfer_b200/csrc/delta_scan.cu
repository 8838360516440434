// The gated delta rule with a decay per head and key channel ("Gated Delta Networks", Yang, Kautz and Hatamizadeh, 2024,
// with the decay made channel-wise). Per head, S is dk x dv, float32, kept per request in a state slot (stored
// transposed, [H][dv][dk], as linear_scan.cu keeps its states), zero when the request starts. For every token, in order:
//     S <- diag(g) S            u = beta * (v - S^T k)            S <- S + k u^T            o = S^T q
// so the read-out sees the token's own write. Two kernels, all in float32:
//   delta_prepare_kernel, a block a token and head, makes what does not depend on the state, once for all columns:
//     q, k   : the group's rows divided by sqrt(sum(x^2) + unit_eps), q also times q_scale; and their product k.q
//     g      : exp(-exp(A_log[h]) * softplus(a[t][h][c] + dt_bias[h][c]))        a: float32 rows (a projection's output)
//     beta   : sigmoid(b[t][h])                                                    b: float32 rows
//     v      : widened to float32
//   delta_scan_kernel walks a request's tokens in order. The columns of S are independent of one another, and the
//   update of a column is not a composition of diagonal maps (the transition I - beta k k^T is a full matrix), so
//   the parallelism is requests x heads x value columns. A block is one request x one head x a few columns; a thread
//   holds KPT neighbouring rows of one column, a column's rows are spread over KP lanes. With D = diag(g) S, the
//   read-out is o = D^T q + u (k.q): both sums over the rows, D^T k and D^T q, are taken in one pass and meet in
//   one round of shuffles, and only S <- D + k u^T is carried to the next token. Chunks of tokens come into shared
//   memory by cp.async, the next chunk while the current one is walked.
#include "common.cuh"

constexpr int DS_MAX_WARPS = 4;
constexpr int DP_THREADS = 128;

__device__ __forceinline__ float ds_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

struct DeltaWork {                // float32, one row per token of the step
    float *q, *k;                 // [T][groups * dk]
    float* g;                     // [T][heads * dk]
    float* v;                     // [T][heads * dv]
    float *kq, *beta;             // [T][groups], [T][heads]
};

struct DeltaPrepArgs {
    DeltaWork w;
    const void *q, *k, *v;        // rows of ld_* elements, first column *_off; q and k: [groups][dk], v: [H][dv]
    int ld_q, q_off, ld_k, k_off, ld_v, v_off;
    const float* a;               // float32 rows of ld_a, first column a_off: [H][dk]
    int ld_a, a_off;
    const float* b;               // float32 rows of ld_b, first column b_off: [H]
    int ld_b, b_off;
    const float *a_log, *dt_bias; // [H], [H * dk]
    float q_scale, unit_eps;
    int heads, groups, dk, dv;
};

template <typename T>
__global__ void __launch_bounds__(DP_THREADS) delta_prepare_kernel(DeltaPrepArgs a) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per_group = a.heads / a.groups;
    if (warp == 0 && h % per_group == 0) {               // unit vectors: the first head of a group makes them
        const int g = h / per_group;
        const T* q = (const T*)a.q + (size_t)t * a.ld_q + a.q_off + g * a.dk;
        const T* k = (const T*)a.k + (size_t)t * a.ld_k + a.k_off + g * a.dk;
        float ssq = 0.f, ssk = 0.f, sqk = 0.f;
        for (int c = lane; c < a.dk; c += 32) {
            const float qv = to_f32(q[c]), kv = to_f32(k[c]);
            ssq = fmaf(qv, qv, ssq);
            ssk = fmaf(kv, kv, ssk);
        }
        ssq = warp_sum(ssq);
        ssk = warp_sum(ssk);
        const float fq = a.q_scale / sqrtf(ssq + a.unit_eps), fk = 1.f / sqrtf(ssk + a.unit_eps);
        for (int c = lane; c < a.dk; c += 32) {
            const float qv = to_f32(q[c]) * fq, kv = to_f32(k[c]) * fk;
            a.w.q[((size_t)t * a.groups + g) * a.dk + c] = qv;
            a.w.k[((size_t)t * a.groups + g) * a.dk + c] = kv;
            sqk = fmaf(qv, kv, sqk);
        }
        sqk = warp_sum(sqk);
        if (lane == 0) a.w.kq[(size_t)t * a.groups + g] = sqk;
    }
    const float rate = expf(a.a_log[h]);
    for (int c = tid; c < a.dk; c += DP_THREADS) {
        const float z = a.a[(size_t)t * a.ld_a + a.a_off + h * a.dk + c] + (a.dt_bias ? a.dt_bias[h * a.dk + c] : 0.f);
        a.w.g[((size_t)t * a.heads + h) * a.dk + c] = expf(-rate * ds_softplus(z));
    }
    const T* v = (const T*)a.v + (size_t)t * a.ld_v + a.v_off + h * a.dv;
    for (int c = tid; c < a.dv; c += DP_THREADS) a.w.v[((size_t)t * a.heads + h) * a.dv + c] = to_f32(v[c]);
    if (tid == 0) a.w.beta[(size_t)t * a.heads + h] = 1.f / (1.f + expf(-a.b[(size_t)t * a.ld_b + a.b_off + h]));
}

__device__ __forceinline__ void ds_copy16(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ds_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ds_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ds_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct DeltaScanArgs {
    DeltaWork w;
    float* y;                     // [T][H * dv]
    float* state;                 // slot s at state + s * slot_stride: [H][dv][dk]
    long long slot_stride;
    const int *cu_seqlens, *state_slots;
    int heads, groups, dk, dv, chunk;
    int vec_k, vec_v;             // rows of dk floats, and a block's columns of v, move in 16-byte pieces
};

template <int KPT, int KP>
__global__ void __launch_bounds__(DS_MAX_WARPS * 32) delta_scan_kernel(DeltaScanArgs a) {
    extern __shared__ __align__(16) float smem[];
    constexpr int PITCH = KPT + 4;                       // floats from one lane part's rows to the next: no two lanes in a bank
    constexpr int trow = KP * PITCH;
    constexpr int cols_per_warp = 32 / KP;
    const int threads = blockDim.x, warps = threads >> 5;
    const int cpb = warps * cols_per_warp;
    const int col_blocks = (a.dv + cpb - 1) / cpb;
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks;
    const int seq = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kpart = lane % KP;
    const int lcol = warp * cols_per_warp + lane / KP;
    const int col = cb * cpb + lcol;
    const bool col_ok = col < a.dv;
    const int g = h / (a.heads / a.groups);
    const int buf_floats = (a.chunk * (3 * trow + cpb + 2) + 3) & ~3;
    for (int e = tid; e < 2 * buf_floats; e += threads) smem[e] = 0.f;   // the rows past dk stay zero
    // which pieces of a token's rows this thread fetches: piece p_first (and every `threads`-th after it) of the
    // tokens tt_first, tt_first + tt_step, ...; with more threads than pieces, several tokens side by side
    const int step = a.vec_k ? 4 : 1, pieces = (a.dk + step - 1) / step;
    const bool wide = threads >= pieces;
    const int tt_step = wide ? threads / pieces : 1;
    const int tt_first = wide ? tid / pieces : 0;
    const int p_first = wide ? tid % pieces : tid;
    const int vstep = a.vec_v ? 4 : 1, vpieces = cpb / vstep;
    __syncthreads();
    ti_grid_wait();
    const int row0 = a.cu_seqlens[seq], row1 = a.cu_seqlens[seq + 1];
    float* srow = a.state + (size_t)a.state_slots[seq] * a.slot_stride + ((size_t)h * a.dv + (col_ok ? col : 0)) * a.dk;
    float S[KPT];
#pragma unroll
    for (int r = 0; r < KPT; ++r) S[r] = (col_ok && kpart * KPT + r < a.dk) ? srow[kpart * KPT + r] : 0.f;

    // a chunk's tokens t0 .. t0 + n - 1 into one of the two buffers
    auto fetch = [&](int t0, int n, float* buf) {
        float* sq = buf;
        float* sk = sq + (size_t)a.chunk * trow;
        float* sg = sk + (size_t)a.chunk * trow;
        float* sv = sg + (size_t)a.chunk * trow;         // [chunk][cpb]
        float* sb = sv + (size_t)a.chunk * cpb;          // [chunk]
        float* sx = sb + a.chunk;                        // [chunk]: k.q
        if (tt_first < tt_step) {
            const size_t ld_qk = (size_t)a.groups * a.dk, ld_g = (size_t)a.heads * a.dk;
            for (int p = p_first; p < pieces; p += threads) {
                const int idx = p * step;
                int at = tt_first * trow + (idx / KPT) * PITCH + idx % KPT;
                const float* gq = a.w.q + ((size_t)(t0 + tt_first) * a.groups + g) * a.dk + idx;
                const float* gk = a.w.k + ((size_t)(t0 + tt_first) * a.groups + g) * a.dk + idx;
                const float* gg = a.w.g + ((size_t)(t0 + tt_first) * a.heads + h) * a.dk + idx;
                for (int tt = tt_first; tt < n; tt += tt_step) {
                    if (a.vec_k) { ds_copy16(sq + at, gq); ds_copy16(sk + at, gk); ds_copy16(sg + at, gg); }
                    else { ds_copy4(sq + at, gq); ds_copy4(sk + at, gk); ds_copy4(sg + at, gg); }
                    at += tt_step * trow;
                    gq += tt_step * ld_qk;
                    gk += tt_step * ld_qk;
                    gg += tt_step * ld_g;
                }
            }
        }
        for (int e = tid; e < n * vpieces; e += threads) {
            const int tt = e / vpieces, c = (e % vpieces) * vstep;
            if (cb * cpb + c >= a.dv) continue;
            const float* gv = a.w.v + ((size_t)(t0 + tt) * a.heads + h) * a.dv + cb * cpb + c;
            if (a.vec_v) ds_copy16(sv + tt * cpb + c, gv);
            else ds_copy4(sv + tt * cpb + c, gv);
        }
        for (int tt = tid; tt < n; tt += threads) {
            ds_copy4(sb + tt, a.w.beta + (size_t)(t0 + tt) * a.heads + h);
            ds_copy4(sx + tt, a.w.kq + (size_t)(t0 + tt) * a.groups + g);
        }
    };

    if (row0 < row1) fetch(row0, min(a.chunk, row1 - row0), smem);
    ds_commit();
    int which = 0;
    for (int t0 = row0; t0 < row1; t0 += a.chunk, which ^= 1) {
        const int n = min(a.chunk, row1 - t0);
        if (t0 + a.chunk < row1) fetch(t0 + a.chunk, min(a.chunk, row1 - t0 - a.chunk), smem + (which ^ 1) * buf_floats);
        ds_commit();
        ds_wait<1>();                                    // this chunk has landed; the next one may still be on its way
        __syncthreads();
        const float* sq = smem + which * buf_floats;
        const float* sk = sq + (size_t)a.chunk * trow;
        const float* sg = sk + (size_t)a.chunk * trow;
        const float* sv = sg + (size_t)a.chunk * trow;
        const float* sb = sv + (size_t)a.chunk * cpb;
        const float* sx = sb + a.chunk;
        for (int tt = 0; tt < n; ++tt) {
            const float vv = sv[tt * cpb + lcol], beta = sb[tt], kq = sx[tt];
            const float4* pq = reinterpret_cast<const float4*>(sq + (size_t)tt * trow + kpart * PITCH);
            const float4* pk = reinterpret_cast<const float4*>(sk + (size_t)tt * trow + kpart * PITCH);
            const float4* pg = reinterpret_cast<const float4*>(sg + (size_t)tt * trow + kpart * PITCH);
            float kr[KPT];
            float dk0 = 0.f, dk1 = 0.f, dq0 = 0.f, dq1 = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < KPT / 4; ++r4) {
                const float4 gv = pg[r4], kv = pk[r4], qv = pq[r4];
                const float gr[4] = {gv.x, gv.y, gv.z, gv.w}, qr[4] = {qv.x, qv.y, qv.z, qv.w};
                kr[r4 * 4] = kv.x; kr[r4 * 4 + 1] = kv.y; kr[r4 * 4 + 2] = kv.z; kr[r4 * 4 + 3] = kv.w;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = r4 * 4 + j;
                    S[r] *= gr[j];
                    if (j & 1) { dk1 = fmaf(S[r], kr[r], dk1); dq1 = fmaf(S[r], qr[j], dq1); }
                    else { dk0 = fmaf(S[r], kr[r], dk0); dq0 = fmaf(S[r], qr[j], dq0); }
                }
            }
            float dot = dk0 + dk1, oq = dq0 + dq1;
#pragma unroll
            for (int off = 1; off < KP; off <<= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, off);
                oq += __shfl_xor_sync(0xffffffffu, oq, off);
            }
            const float u = beta * (vv - dot);
#pragma unroll
            for (int r = 0; r < KPT; ++r) S[r] = fmaf(kr[r], u, S[r]);
            if (kpart == 0 && col_ok) a.y[(size_t)(t0 + tt) * a.heads * a.dv + h * a.dv + col] = fmaf(u, kq, oq);
        }
        __syncthreads();                                 // the chunk has been read: its buffer may be filled again
    }
    ds_wait<0>();
    ti_grid_launch_dependents();                         // only now: the walk is long, and the next kernel's blocks would sit on the SMs through it
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < KPT; ++r)
            if (kpart * KPT + r < a.dk) srow[kpart * KPT + r] = S[r];
    }
}

static inline size_t ds_round4(size_t n) { return (n + 3) & ~(size_t)3; }

// floats of workspace for a step of t tokens: every part starts on a 16-byte boundary
static inline size_t ds_workspace(size_t t, int heads, int groups, int dk, int dv) {
    return 2 * ds_round4(t * groups * dk) + ds_round4(t * heads * dk) + ds_round4(t * heads * dv) + ds_round4(t * groups) +
           ds_round4(t * heads);
}

// y float32 [T][heads * dv]; q, k, v in the compute dtype; a, b float32; work: work_floats floats, 16-byte
// aligned, at least T * (2 groups dk + heads (dk + dv + 1) + groups) + 24 of them. A request's tokens of the step are cu_seqlens[i] .. cu_seqlens[i + 1] - 1; its state is slot
// state_slots[i].
TI_API int ti_delta_scan(float* y, float* state, long long slot_stride, const void* q, int ld_q, int q_off, const void* k,
                         int ld_k, int k_off, const void* v, int ld_v, int v_off, const float* a, int ld_a, int a_off,
                         const float* b, int ld_b, int b_off, const float* a_log, const float* dt_bias, float q_scale,
                         float unit_eps, const int* cu_seqlens, const int* state_slots, int num_seqs, int num_tokens,
                         int heads, int groups, int dk, int dv, float* work, long long work_floats, int dtype,
                         cudaStream_t stream) {
    TI_REQUIRE(num_seqs >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && dk > 0 && dv > 0, "delta_scan: bad sizes");
    TI_REQUIRE(dk <= 1024, "delta_scan: %d key channels a head (at most 1024)", dk);
    TI_REQUIRE(a && b && a_log, "delta_scan: the decay's and the step's tensors are needed");
    TI_REQUIRE(num_seqs <= 65535, "delta_scan: too many requests");
    TI_REQUIRE(dtype == TI_F32 || dtype == TI_BF16, "delta_scan: unknown dtype %d", dtype);
    if (num_seqs == 0 || num_tokens == 0) return 0;
    const size_t t = (size_t)num_tokens;
    TI_REQUIRE(work && ((uintptr_t)work & 15) == 0, "delta_scan: the workspace must be 16-byte aligned");
    TI_REQUIRE(work_floats >= (long long)ds_workspace(t, heads, groups, dk, dv), "delta_scan: the workspace is too small");
    DeltaWork w;
    w.q = work;
    w.k = w.q + ds_round4(t * groups * dk);
    w.g = w.k + ds_round4(t * groups * dk);
    w.v = w.g + ds_round4(t * heads * dk);
    w.kq = w.v + ds_round4(t * heads * dv);
    w.beta = w.kq + ds_round4(t * groups);
    DeltaPrepArgs prep = {w, q, k, v, ld_q, q_off, ld_k, k_off, ld_v, v_off, a, ld_a, a_off, b, ld_b, b_off,
                          a_log, dt_bias, q_scale, unit_eps, heads, groups, dk, dv};
    TI_REQUIRE(heads <= 65535, "delta_scan: too many heads");
    if (dtype == TI_F32) ti_launch(delta_prepare_kernel<float>, dim3(num_tokens, heads), DP_THREADS, 0, stream, prep);
    else ti_launch(delta_prepare_kernel<__nv_bfloat16>, dim3(num_tokens, heads), DP_THREADS, 0, stream, prep);
    TI_CHECK_LAUNCH("delta_prepare");

    int kp = 1;
    const int rows = 8;                                  // most rows of a column that a lane holds
    while (kp < 32 && (dk + kp - 1) / kp > rows) kp <<= 1;
    const int per_lane = (dk + kp - 1) / kp;
    const int kpt = per_lane <= 4 ? 4 : per_lane <= 8 ? 8 : per_lane <= 16 ? 16 : 32;
    // few columns a block when the step has few (request, head) pairs, so that every SM has a block; many columns a
    // block otherwise, as every block fetches the head's q, k and g for itself
    int warps = DS_MAX_WARPS;
    while (warps > 1 && (long long)num_seqs * heads * ((dv + warps * (32 / kp) - 1) / (warps * (32 / kp))) < 148) warps >>= 1;
    const int trow = kp * (kpt + 4), cpb = warps * (32 / kp);
    // two buffers of `chunk` tokens within the 48 KB that need no opt-in; a step of single tokens stages no more than one
    int chunk = 16;
    while (chunk > 1 && 2 * ds_round4((size_t)chunk * (3 * trow + cpb + 2)) * sizeof(float) > 44 * 1024) chunk >>= 1;
    if (num_tokens == num_seqs) chunk = 1;
    const size_t smem = 2 * ds_round4((size_t)chunk * (3 * trow + cpb + 2)) * sizeof(float);
    DeltaScanArgs args = {w, y, state, slot_stride, cu_seqlens, state_slots, heads, groups, dk, dv, chunk,
                          dk % 4 == 0, dv % 4 == 0 && cpb % 4 == 0};
    dim3 grid(heads * ((dv + cpb - 1) / cpb), num_seqs);
    // a walk of many tokens starts alone (see ti_launch_alone); a step of single tokens is short and starts early
    const bool alone = num_tokens != num_seqs;
    bool launched = false;
#define TI_DSCAN(KPT, KP)                                                                         \
    if (!launched && kpt == KPT && kp == KP) {                                                    \
        if (alone) ti_launch_alone(delta_scan_kernel<KPT, KP>, grid, warps * 32, smem, stream, args); \
        else ti_launch(delta_scan_kernel<KPT, KP>, grid, warps * 32, smem, stream, args);         \
        launched = true;                                                                          \
    }
#define TI_DSCAN_ROWS(KPT) TI_DSCAN(KPT, 1) TI_DSCAN(KPT, 2) TI_DSCAN(KPT, 4) TI_DSCAN(KPT, 8) TI_DSCAN(KPT, 16) TI_DSCAN(KPT, 32)
    TI_DSCAN_ROWS(4) TI_DSCAN_ROWS(8) TI_DSCAN_ROWS(16) TI_DSCAN(32, 32)
#undef TI_DSCAN_ROWS
#undef TI_DSCAN
    TI_REQUIRE(launched, "delta_scan: no kernel for %d rows a lane over %d lanes", kpt, kp);
    TI_CHECK_LAUNCH("delta_scan");
    return 0;
}
