// The gated delta rule with a decay per head and key channel ("Gated Delta Networks", Yang, Kautz and Hatamizadeh, 2024,
// with the decay made channel-wise). Per head, S is dk x dv, float32, kept per request in a state slot (stored
// transposed, [H][dv][dk], as linear_scan.cu keeps its states), zero when the request starts. For every token, in order:
//     S <- diag(g) S            u = beta * (v - S^T k)            S <- S + k u^T            o = S^T q
// so the read-out sees the token's own write. What the kernel makes from the model's tensors while it stages a chunk
// of tokens in shared memory, all in float32:
//     q, k   : the head's (or its group's) rows divided by sqrt(sum(x^2) + unit_eps), q also times q_scale
//     g      : exp(-exp(A_log[h]) * softplus(a[t][h][c] + dt_bias[h][c]))        a: float32 rows (a projection's output)
//     beta   : sigmoid(b[t][h])                                                    b: float32 rows
// The columns of S are independent of one another, and the update of a column is not a composition of diagonal maps
// (the transition I - beta k k^T is a full matrix), so a request's tokens are walked in order and the parallelism is
// requests x heads x value columns. A block is one request x one head x a few columns; a thread holds KPT neighbouring
// rows of one column, a column's rows are spread over KP lanes whose partial sums of S^T k and of S^T q meet by shuffles.
#include "common.cuh"

constexpr int DS_MAX_WARPS = 4;

__device__ __forceinline__ float ds_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

struct DeltaScanArgs {
    float* y;                     // [T][H * dv]
    float* state;                 // slot s at state + s * slot_stride: [H][dv][dk]
    long long slot_stride;
    const void *q, *k, *v;        // rows of ld_* elements, first column *_off; q and k: [groups][dk], v: [H][dv]
    int ld_q, q_off, ld_k, k_off, ld_v, v_off;
    const float* a;               // float32 rows of ld_a, first column a_off: [H][dk]
    int ld_a, a_off;
    const float* b;               // float32 rows of ld_b, first column b_off: [H]
    int ld_b, b_off;
    const float *a_log, *dt_bias; // [H], [H * dk]
    float q_scale, unit_eps;
    const int *cu_seqlens, *state_slots;
    int heads, groups, dk, dv, kp, chunk;
};

template <typename T, int KPT>
__global__ void __launch_bounds__(DS_MAX_WARPS * 32) delta_scan_kernel(DeltaScanArgs a) {
    extern __shared__ float smem[];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int KP = a.kp, dkp = KP * KPT;
    constexpr int PITCH = KPT + 4;                       // floats from one lane part's rows to the next: no two lanes in a bank
    const int trow = KP * PITCH;
    const int threads = blockDim.x, warps = threads >> 5;
    const int cols_per_warp = 32 / KP, cols_per_block = warps * cols_per_warp;
    const int col_blocks = (a.dv + cols_per_block - 1) / cols_per_block;
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks;
    const int seq = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kpart = lane % KP;
    const int col = cb * cols_per_block + warp * cols_per_warp + lane / KP;
    const bool col_ok = col < a.dv;
    const int g = h / (a.heads / a.groups);
    const int row0 = a.cu_seqlens[seq], row1 = a.cu_seqlens[seq + 1];
    float* sq = smem;                                    // [chunk][KP][PITCH]
    float* sk = sq + (size_t)a.chunk * trow;
    float* sa = sk + (size_t)a.chunk * trow;
    float* sv = sa + (size_t)a.chunk * trow;             // [chunk][cols_per_block]
    float* sb = sv + (size_t)a.chunk * cols_per_block;   // [chunk]
    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    float* srow = a.state + (size_t)a.state_slots[seq] * a.slot_stride + ((size_t)h * a.dv + (col_ok ? col : 0)) * a.dk;
    float S[KPT];
#pragma unroll
    for (int r = 0; r < KPT; ++r) S[r] = (col_ok && kpart * KPT + r < a.dk) ? srow[kpart * KPT + r] : 0.f;
    const float rate = expf(a.a_log[h]);

    for (int t0 = row0; t0 < row1; t0 += a.chunk) {
        const int n = min(a.chunk, row1 - t0);
        __syncthreads();                                 // the chunk before has been read
        for (int e = tid; e < n * dkp; e += threads) {
            const int tt = e / dkp, idx = e % dkp, t = t0 + tt;
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (idx < a.dk) {
                qv = to_f32(q[(size_t)t * a.ld_q + a.q_off + g * a.dk + idx]);
                kv = to_f32(k[(size_t)t * a.ld_k + a.k_off + g * a.dk + idx]);
                const float z = a.a[(size_t)t * a.ld_a + a.a_off + h * a.dk + idx] + (a.dt_bias ? a.dt_bias[h * a.dk + idx] : 0.f);
                av = expf(-rate * ds_softplus(z));
            }
            const int at = tt * trow + (idx / KPT) * PITCH + idx % KPT;
            sq[at] = qv;
            sk[at] = kv;
            sa[at] = av;
        }
        for (int e = tid; e < n * cols_per_block; e += threads) {
            const int tt = e / cols_per_block, c = cb * cols_per_block + e % cols_per_block;
            sv[e] = c < a.dv ? to_f32(v[(size_t)(t0 + tt) * a.ld_v + a.v_off + h * a.dv + c]) : 0.f;
        }
        for (int tt = tid; tt < n; tt += threads) {
            const float z = a.b[(size_t)(t0 + tt) * a.ld_b + a.b_off + h];
            sb[tt] = 1.f / (1.f + expf(-z));
        }
        __syncthreads();
        for (int tt = warp; tt < n; tt += warps) {       // unit vectors: a warp a token
            float ssq = 0.f, ssk = 0.f;
            for (int idx = lane; idx < a.dk; idx += 32) {
                const int at = tt * trow + (idx / KPT) * PITCH + idx % KPT;
                ssq = fmaf(sq[at], sq[at], ssq);
                ssk = fmaf(sk[at], sk[at], ssk);
            }
            ssq = warp_sum(ssq);
            ssk = warp_sum(ssk);
            const float fq = a.q_scale / sqrtf(ssq + a.unit_eps), fk = 1.f / sqrtf(ssk + a.unit_eps);
            for (int idx = lane; idx < a.dk; idx += 32) {
                const int at = tt * trow + (idx / KPT) * PITCH + idx % KPT;
                sq[at] *= fq;
                sk[at] *= fk;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vv = sv[tt * cols_per_block + warp * cols_per_warp + lane / KP];
            const float beta = sb[tt];
            const float4* pq = reinterpret_cast<const float4*>(sq + (size_t)tt * trow + kpart * PITCH);
            const float4* pk = reinterpret_cast<const float4*>(sk + (size_t)tt * trow + kpart * PITCH);
            const float4* pa = reinterpret_cast<const float4*>(sa + (size_t)tt * trow + kpart * PITCH);
            float kr[KPT];
            float dot = 0.f, dot2 = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < KPT / 4; ++r4) {
                const float4 av = pa[r4], kv = pk[r4];
                const float ar[4] = {av.x, av.y, av.z, av.w};
                kr[r4 * 4] = kv.x; kr[r4 * 4 + 1] = kv.y; kr[r4 * 4 + 2] = kv.z; kr[r4 * 4 + 3] = kv.w;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = r4 * 4 + j;
                    S[r] *= ar[j];
                    if (j & 1) dot2 = fmaf(S[r], kr[r], dot2);
                    else dot = fmaf(S[r], kr[r], dot);
                }
            }
            dot += dot2;
            for (int off = 1; off < KP; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
            const float u = beta * (vv - dot);
            float o = 0.f, o2 = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < KPT / 4; ++r4) {
                const float4 qv = pq[r4];
                const float qr[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = r4 * 4 + j;
                    S[r] = fmaf(kr[r], u, S[r]);
                    if (j & 1) o2 = fmaf(S[r], qr[j], o2);
                    else o = fmaf(S[r], qr[j], o);
                }
            }
            o += o2;
            for (int off = 1; off < KP; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (kpart == 0 && col_ok) a.y[(size_t)(t0 + tt) * a.heads * a.dv + h * a.dv + col] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < KPT; ++r)
            if (kpart * KPT + r < a.dk) srow[kpart * KPT + r] = S[r];
    }
}

// y float32 [T][heads * dv]; q, k, v in the compute dtype; a, b float32. A request's tokens of the step are
// cu_seqlens[i] .. cu_seqlens[i + 1] - 1; its state is slot state_slots[i].
TI_API int ti_delta_scan(float* y, float* state, long long slot_stride, const void* q, int ld_q, int q_off, const void* k,
                         int ld_k, int k_off, const void* v, int ld_v, int v_off, const float* a, int ld_a, int a_off,
                         const float* b, int ld_b, int b_off, const float* a_log, const float* dt_bias, float q_scale,
                         float unit_eps, const int* cu_seqlens, const int* state_slots, int num_seqs, int num_tokens,
                         int heads, int groups, int dk, int dv, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_seqs >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && dk > 0 && dv > 0, "delta_scan: bad sizes");
    TI_REQUIRE(dk <= 1024, "delta_scan: %d key channels a head (at most 1024)", dk);
    TI_REQUIRE(a && b && a_log, "delta_scan: the decay's and the step's tensors are needed");
    TI_REQUIRE(num_seqs <= 65535, "delta_scan: too many requests");
    if (num_seqs == 0 || num_tokens == 0) return 0;
    int kp = 1;
    while (kp < 32 && (dk + kp - 1) / kp > 16) kp <<= 1;
    const int per_lane = (dk + kp - 1) / kp;
    const int kpt = per_lane <= 4 ? 4 : per_lane <= 8 ? 8 : per_lane <= 16 ? 16 : 32;
    // few columns a block when the step has few (request, head) pairs, so that more SMs have a block
    int warps = DS_MAX_WARPS;
    while (warps > 1 && (long long)num_seqs * heads * ((dv + warps * (32 / kp) - 1) / (warps * (32 / kp))) < 2 * 148) warps >>= 1;
    const int trow = kp * (kpt + 4), cols_per_block = warps * (32 / kp);
    int chunk = 16;
    while (chunk > 1 && (size_t)chunk * (3 * trow + cols_per_block + 1) * sizeof(float) > 40 * 1024) chunk >>= 1;
    const size_t smem = (size_t)chunk * (3 * trow + cols_per_block + 1) * sizeof(float);
    DeltaScanArgs args = {y, state, slot_stride, q, k, v, ld_q, q_off, ld_k, k_off, ld_v, v_off, a, ld_a, a_off, b, ld_b, b_off,
                          a_log, dt_bias, q_scale, unit_eps, cu_seqlens, state_slots, heads, groups, dk, dv, kp, chunk};
    dim3 grid(heads * ((dv + cols_per_block - 1) / cols_per_block), num_seqs);
    typedef __nv_bfloat16 B;
#define TI_DSCAN(KPT)                                                                                          \
    do {                                                                                                       \
        if (dtype == TI_F32) ti_launch(delta_scan_kernel<float, KPT>, grid, warps * 32, smem, stream, args);   \
        else ti_launch(delta_scan_kernel<B, KPT>, grid, warps * 32, smem, stream, args);                       \
    } while (0)
    TI_REQUIRE(dtype == TI_F32 || dtype == TI_BF16, "delta_scan: unknown dtype %d", dtype);
    if (kpt == 4) TI_DSCAN(4);
    else if (kpt == 8) TI_DSCAN(8);
    else if (kpt == 16) TI_DSCAN(16);
    else TI_DSCAN(32);
#undef TI_DSCAN
    TI_CHECK_LAUNCH("delta_scan");
    return 0;
}
