// Linear attention with a decaying matrix state per head, for every mixer of the form
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          o_t = S_t^T q_t (+ skip_h * v_t)
// S is dk x dv per head, float32, kept per request in a state slot (stored transposed, [H][dv][dk], so that a thread's
// share of a column is contiguous), zero when the request starts. The decay a_t acts on the rows of S (the key
// channels) and is either one number per key channel or one per head. How it is made from the model's tensors:
//   gate 0 (raw)          a = gate                                      gate: float32 [T][H * dk] or [T][H]
//   gate 1 (sigmoid power) a = sigmoid(gate)^(1 / tau) = exp(logsigmoid(gate) / tau), per key channel
//   gate 2 (step size)     dt = softplus(gate + dt_bias[h]), a = exp(-exp(A_log[h]) * dt) per head, and k_t is
//                          multiplied by dt (a discretised state-space model: "Transformers are SSMs", Dao and Gu, 2024)
// For long portions a small kernel makes the decays (and the keys' factors) of the step once, float32 [T][H * dk] or
// [T][H], and the scan reads them like any other operand; short steps make them while staging.
// Decays, their logarithms, softplus, exponentials, the state and the outputs are float32; q, k and v are read in
// the compute dtype from wherever they lie (row length and first column given), several heads may share one
// group of q and k.
//
// A block is one request x one head x a few columns of S; a thread holds KPT neighbouring rows of one column, the rows
// of a column are spread over KP lanes (row = lane part * KPT + r), whose partial sums of o meet by shuffles; a thread
// reads its rows of q, k and the decay from shared memory four at a time (the parts lie KPT + 4 floats apart, so the
// lanes' 16-byte reads fall into different banks). The step's
// tokens of the request are walked in order; q, k and the decays of a few tokens at a time are staged in shared
// memory by the whole block.
//
// Long portions are cut into stretches that run side by side (grid z), since the recurrence composes: a stretch is
// (A, B) = (the product of its decays, its own scan from a zero state). Pass 1 scans every stretch from zero, writes
// the outputs that its own tokens give, leaves (A, B) and, per token, q times the product of the decays so far; a fold
// walks a request's stretches in order, S <- A S + B, leaves each stretch's true starting state where its B was and
// the request's new state in its slot; pass 2 adds to every output what the state at the stretch's start gives it,
// o_t += (q_t * D_t)^T S_start with D_t the product of the stretch's decays up to t: a plain product, no recurrence.
// Four thirds of the arithmetic, as many times the blocks as there are stretches.
//
//   gated_group_norm : out = scale * w * n(y) * act(gate)  or  scale * w * n(y * act(gate)),  n: every group of
//                      `group` features divided by its root mean square (float32), act silu or sigmoid, one rounding
#include "common.cuh"

enum { LS_GATE_RAW = 0, LS_GATE_SIGMOID_POW = 1, LS_GATE_STEP = 2 };
constexpr int LS_WARPS = 4;

__device__ __forceinline__ float ls_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float ls_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct LinearScanArgs {
    float* y;                 // [T][H * dv]
    float* state;             // slot s at state + s * slot_stride: [H][dv][dk]
    long long slot_stride;
    const void *q, *k, *v;    // rows of ld_* elements, first column *_off; q and k: [groups][dk], v: [H][dv]
    int ld_q, q_off, ld_k, k_off, ld_v, v_off;
    const float* decay;       // float32 rows of ld_decay, first column decay_off: [H][dk] (per channel) or [H]
    int ld_decay, decay_off, per_channel;
    const float* kscale;      // float32 [T][H] or null: a factor on the keys of a head
    int gate_mode;            // not LS_GATE_RAW: `decay` holds the gate's values and the decays are made while staging
    float inv_tau;            // (short steps: a kernel of its own for them would cost more than repeating them a few times)
    const float *a_log, *dt_bias;
    const float* skip;        // [H] or null
    float q_scale;
    const int *cu_seqlens, *state_slots;
    int heads, groups, dk, dv, kp, chunk;
    int wide_state;           // the rows of a state start on 16-byte boundaries: a thread moves its rows four at a time
    int stretches;            // > 1: grid z is the stretch; part_b [request][stretch][H][dv][dk], part_a [request][stretch][H][dk]
    float *part_b, *part_a;
    float* qd;                // [T][H][dk]: q times the product of the decays from the stretch's start to the token
};

// MODE 0: from the slot's state to the slot's state, with outputs; 1: a stretch from zero, with the outputs its own
// tokens give, leaves (A, B) and qd; 2: adds what the state at the stretch's start gives every output.
template <typename T, int KPT, int MODE>
__global__ void __launch_bounds__(LS_WARPS * 32, KPT <= 16 ? 7 : 1) linear_scan_kernel(LinearScanArgs a) {      // seven blocks an SM: what the stretches are counted for
    extern __shared__ float smem[];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int KP = a.kp, dkp = KP * KPT;                 // dk rounded up to what the lanes hold
    constexpr int PITCH = KPT + 4;                       // floats from one lane part's rows to the next in shared memory
    const int trow = KP * PITCH;                         // floats a token takes in each of sq, sk, sa
    const int cols_per_warp = 32 / KP, cols_per_block = LS_WARPS * cols_per_warp;
    const int col_blocks = (a.dv + cols_per_block - 1) / cols_per_block;
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks;
    const int seq = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kpart = lane % KP;
    const int col = cb * cols_per_block + warp * cols_per_warp + lane / KP;
    const bool col_ok = col < a.dv;
    const int g = h / (a.heads / a.groups);
    int row0 = a.cu_seqlens[seq], row1 = a.cu_seqlens[seq + 1];
    if (MODE != 0) {                                     // this block's stretch of the request's tokens
        const int n = row1 - row0, len = (n + a.stretches - 1) / a.stretches;
        const int first = row0 + min(n, (int)blockIdx.z * len);
        row1 = row0 + min(n, ((int)blockIdx.z + 1) * len);
        row0 = first;
    }
    float* sq = smem;                                    // [chunk][KP][PITCH]
    float* sk = sq + (size_t)a.chunk * trow;
    float* sa = sk + (size_t)a.chunk * trow;
    float* sv = sa + (size_t)a.chunk * trow;             // [chunk][cols_per_block]
    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;

    const size_t in_head = ((size_t)h * a.dv + (col_ok ? col : 0)) * a.dk;
    float* srow = MODE == 0 ? a.state + (size_t)a.state_slots[seq] * a.slot_stride + in_head
                            : a.part_b + ((size_t)seq * a.stretches + blockIdx.z) * a.heads * a.dv * a.dk + in_head;
    float S[KPT];
    // Mode 1, the block of a head's first columns: thread i (and i + 128, ...) carries the product D of key channel i's
    // decays from the stretch's start, chunk by chunk, and writes q * D for every token; at the end D is the stretch's A.
    constexpr int DPT = 8;                               // 1,024 key channels over 128 threads
    float D[MODE == 1 ? DPT : 1];
    if (MODE == 1) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) D[i] = 1.f;
    }
#pragma unroll
    for (int r = 0; r < KPT; ++r) S[r] = 0.f;
    if (MODE != 1 && col_ok) {
        if (a.wide_state) {
#pragma unroll
            for (int r = 0; r < KPT; r += 4) {
                if (kpart * KPT + r < a.dk) {            // dk is a multiple of 4: the four are inside or outside together
                    const float4 f = *reinterpret_cast<const float4*>(srow + kpart * KPT + r);
                    S[r] = f.x; S[r + 1] = f.y; S[r + 2] = f.z; S[r + 3] = f.w;
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < KPT; ++r)
                if (kpart * KPT + r < a.dk) S[r] = srow[kpart * KPT + r];
        }
    }
    const float skip = a.skip ? a.skip[h] : 0.f;
    const float rate = a.gate_mode == LS_GATE_STEP ? expf(a.a_log[h]) : 0.f;
    const float dt_bias = a.gate_mode == LS_GATE_STEP && a.dt_bias ? a.dt_bias[h] : 0.f;

    for (int t0 = row0; t0 < row1; t0 += a.chunk) {
        const int n = min(a.chunk, row1 - t0);
        __syncthreads();                                 // the chunk before has been read
        // Several elements a thread a trip, all their loads issued before the first is used: a trip that waits for its
        // three loads before it starts the next one is what a chunk's time went into. (Eight a trip where only qd is
        // read; four elsewhere: the registers they take are blocks an SM.)
        constexpr int U = MODE == 2 ? 8 : 4;
        for (int e0 = tid; e0 < n * dkp; e0 += LS_WARPS * 32 * U) {
            float qv[U], kv[U], av[U], ks[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = e0 + u * LS_WARPS * 32;
                const int tt = e / dkp, idx = e % dkp, t = t0 + tt;
                qv[u] = 0.f; kv[u] = 0.f; av[u] = 1.f; ks[u] = 1.f;
                if (e < n * dkp && idx < a.dk) {
                    if (MODE == 2) {
                        qv[u] = a.qd[((size_t)t * a.heads + h) * a.dk + idx];
                    } else {
                        qv[u] = to_f32(q[(size_t)t * a.ld_q + a.q_off + g * a.dk + idx]);
                        kv[u] = to_f32(k[(size_t)t * a.ld_k + a.k_off + g * a.dk + idx]);
                        if (a.kscale) ks[u] = a.kscale[(size_t)t * a.heads + h];
                        av[u] = a.decay[(size_t)t * a.ld_decay + a.decay_off + (a.per_channel ? h * a.dk + idx : h)];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = e0 + u * LS_WARPS * 32;
                if (e >= n * dkp) continue;
                const int tt = e / dkp, idx = e % dkp;
                float qs = qv[u], kk = kv[u] * ks[u], aa = av[u];
                if (MODE != 2 && idx < a.dk) {
                    qs *= a.q_scale;
                    if (a.gate_mode == LS_GATE_SIGMOID_POW) {
                        aa = expf(ls_logsigmoid(aa) * a.inv_tau);
                    } else if (a.gate_mode == LS_GATE_STEP) {
                        const float dt = ls_softplus(aa + dt_bias);
                        aa = expf(-rate * dt);
                        kk *= dt;
                    }
                }
                const int at = tt * trow + (idx / KPT) * PITCH + idx % KPT;
                sq[at] = qs;
                if (MODE != 2) {
                    sk[at] = kk;
                    sa[at] = aa;
                }
            }
        }
        // the values' columns of this block; in mode 2 the outputs so far, which the state's share is added to
        for (int e0 = tid; e0 < n * cols_per_block; e0 += LS_WARPS * 32 * 4) {
            float got[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = e0 + u * LS_WARPS * 32;
                const int tt = e / cols_per_block, c = cb * cols_per_block + e % cols_per_block;
                got[u] = 0.f;
                if (e < n * cols_per_block && c < a.dv)
                    got[u] = MODE == 2 ? a.y[(size_t)(t0 + tt) * a.heads * a.dv + h * a.dv + c]
                                       : to_f32(v[(size_t)(t0 + tt) * a.ld_v + a.v_off + h * a.dv + c]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = e0 + u * LS_WARPS * 32;
                if (e < n * cols_per_block) sv[e] = got[u];
            }
        }
        __syncthreads();
        if (MODE == 1 && cb == 0) {
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                const int idx = tid + i * LS_WARPS * 32;
                if (idx < a.dk) {
                    const int at0 = (idx / KPT) * PITCH + idx % KPT;
                    float d = D[MODE == 1 ? i : 0];
                    for (int tt = 0; tt < n; ++tt) {
                        d *= sa[tt * trow + at0];
                        a.qd[((size_t)(t0 + tt) * a.heads + h) * a.dk + idx] = sq[tt * trow + at0] * d;
                    }
                    D[MODE == 1 ? i : 0] = d;
                }
            }
        }
        for (int tt = 0; tt < n; ++tt) {
            const float vv = sv[tt * cols_per_block + warp * cols_per_warp + lane / KP];     // mode 2: the output so far
            const float4* pq = reinterpret_cast<const float4*>(sq + (size_t)tt * trow + kpart * PITCH);
            const float4* pk = reinterpret_cast<const float4*>(sk + (size_t)tt * trow + kpart * PITCH);
            const float4* pa = reinterpret_cast<const float4*>(sa + (size_t)tt * trow + kpart * PITCH);
            float o = 0.f, o2 = 0.f;
#pragma unroll
            for (int r4 = 0; r4 < KPT / 4; ++r4) {
                const float4 qv = pq[r4];
                const float qr[4] = {qv.x, qv.y, qv.z, qv.w};
                if (MODE == 2) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (j & 1) o2 = fmaf(S[r4 * 4 + j], qr[j], o2);
                        else o = fmaf(S[r4 * 4 + j], qr[j], o);
                    }
                    continue;
                }
                const float4 av = pa[r4], kv = pk[r4];
                const float ar[4] = {av.x, av.y, av.z, av.w}, kr[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = r4 * 4 + j;
                    S[r] = fmaf(ar[j], S[r], kr[j] * vv);
                    if (j & 1) o2 = fmaf(S[r], qr[j], o2);
                    else o = fmaf(S[r], qr[j], o);
                }
            }
            o += o2;
            for (int off = 1; off < KP; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (kpart == 0 && col_ok) {
                float* dst = a.y + (size_t)(t0 + tt) * a.heads * a.dv + h * a.dv + col;
                *dst = MODE == 2 ? vv + o : fmaf(skip, vv, o);
            }
        }
    }
    if (MODE == 2) return;
    if (col_ok) {
        if (a.wide_state) {
#pragma unroll
            for (int r = 0; r < KPT; r += 4)
                if (kpart * KPT + r < a.dk)
                    *reinterpret_cast<float4*>(srow + kpart * KPT + r) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
        } else {
#pragma unroll
            for (int r = 0; r < KPT; ++r)
                if (kpart * KPT + r < a.dk) srow[kpart * KPT + r] = S[r];
        }
    }
    if (MODE == 1 && cb == 0) {                          // the stretch's product of decays, once a head
        float* arow = a.part_a + (((size_t)seq * a.stretches + blockIdx.z) * a.heads + h) * a.dk;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int idx = tid + i * LS_WARPS * 32;
            if (idx < a.dk) arow[idx] = D[MODE == 1 ? i : 0];
        }
    }
}

// A request's stretches in order: S <- A S + B. Each stretch's B becomes the state it starts from; the slot gets
// the state after the last. One thread per element of a request's states.
__global__ void linear_scan_fold_kernel(float* __restrict__ state, long long slot_stride, float* __restrict__ part_b,
                                        const float* __restrict__ part_a, const int* __restrict__ state_slots,
                                        int stretches, int heads, int dk, int dv) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int per = heads * dv * dk;
    const int e = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
    if (e >= per) return;
    const int idx = e % dk, h = e / (dv * dk);
    float* slot = state + (size_t)state_slots[seq] * slot_stride;
    float S = slot[e];
    for (int k0 = 0; k0 < stretches; k0 += 8) {          // eight stretches' loads in flight at once
        float b[8], a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const size_t part = (size_t)seq * stretches + min(k0 + j, stretches - 1);
            b[j] = part_b[part * per + e];
            a[j] = part_a[(part * heads + h) * dk + idx];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (k0 + j < stretches) {
                part_b[((size_t)seq * stretches + k0 + j) * per + e] = S;
                S = fmaf(a[j], S, b[j]);
            }
        }
    }
    slot[e] = S;
}

// The decays of a step from the model's tensors: one thread per (token, head[, key channel]).
__global__ void scan_gate_kernel(float* __restrict__ decay, float* __restrict__ kscale, const float* __restrict__ gate,
                                 int ld_gate, int gate_off, int mode, float inv_tau, const float* __restrict__ a_log,
                                 const float* __restrict__ dt_bias, int heads, int per_head, size_t n) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const size_t t = e / ((size_t)heads * per_head);
    const int c = (int)(e % ((size_t)heads * per_head)), h = c / per_head;
    const float gv = gate[t * ld_gate + gate_off + c];
    if (mode == LS_GATE_SIGMOID_POW) {
        decay[e] = expf(ls_logsigmoid(gv) * inv_tau);
    } else {
        const float dt = ls_softplus(gv + (dt_bias ? dt_bias[h] : 0.f));
        decay[e] = expf(-expf(a_log[h]) * dt);
        kscale[e] = dt;
    }
}

TI_API long long ti_linear_scan_scratch_floats(int num_seqs, int num_tokens, int heads, int dk, int dv, int stretches) {
    return stretches > 1 ? (long long)num_seqs * stretches * heads * dk * (dv + 1) + (long long)num_tokens * heads * dk : 0;
}

// gate_mode 0: `gate` holds the decays themselves. Otherwise they are made first, into `gate_out` (float32, as many
// entries as the gate has per step: num_tokens x heads (x dk if per channel); gate mode 2 needs as many again behind
// them for the keys' factors).
TI_API int ti_linear_scan(float* y, float* state, long long slot_stride, const void* q, int ld_q, int q_off, const void* k,
                          int ld_k, int k_off, const void* v, int ld_v, int v_off, const float* gate, int ld_gate,
                          int gate_off, int gate_mode, int gate_per_channel, float tau, const float* a_log,
                          const float* dt_bias, const float* skip, float q_scale, const int* cu_seqlens,
                          const int* state_slots, int num_seqs, int num_tokens, int heads, int groups, int dk, int dv,
                          int stretches, float* scratch, long long scratch_floats, float* gate_out, int dtype,
                          cudaStream_t stream) {
    TI_REQUIRE(num_seqs >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && dk > 0 && dv > 0, "linear_scan: bad sizes");
    TI_REQUIRE(dk <= 1024, "linear_scan: %d key channels a head (at most 1024)", dk);
    TI_REQUIRE(gate_mode >= 0 && gate_mode <= 2 && gate, "linear_scan: unknown gate %d", gate_mode);
    TI_REQUIRE(gate_mode != LS_GATE_STEP || (a_log && !gate_per_channel), "linear_scan: the step-size gate is one number a head and needs A_log");
    TI_REQUIRE(gate_mode != LS_GATE_SIGMOID_POW || tau > 0.f, "linear_scan: tau must be positive");
    TI_REQUIRE(num_seqs <= 65535, "linear_scan: too many requests");
    TI_REQUIRE(stretches >= 1 && stretches <= 1024, "linear_scan: %d stretches", stretches);
    TI_REQUIRE(stretches == 1 || (scratch && scratch_floats >= ti_linear_scan_scratch_floats(num_seqs, num_tokens, heads, dk, dv, stretches)),
               "linear_scan: %d stretches need %lld floats of scratch", stretches,
               ti_linear_scan_scratch_floats(num_seqs, num_tokens, heads, dk, dv, stretches));
    TI_REQUIRE(gate_mode == LS_GATE_RAW || stretches == 1 || gate_out, "linear_scan: the decays need a place to be made in");
    if (num_seqs == 0 || num_tokens == 0) return 0;
    const float* decay = gate;
    const float* kscale = nullptr;
    int ld_decay = ld_gate, decay_off = gate_off;
    const bool gate_apart = gate_mode != LS_GATE_RAW && stretches > 1;      // long portions: the decays are made once
    if (gate_apart) {
        const int per_head = gate_per_channel ? dk : 1;
        const size_t n = (size_t)num_tokens * heads * per_head;
        ti_launch(scan_gate_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, gate_out, gate_out + n, gate, ld_gate, gate_off,
                  gate_mode, gate_mode == LS_GATE_SIGMOID_POW ? 1.f / tau : 0.f, a_log, dt_bias, heads, per_head, n);
        TI_CHECK_LAUNCH("linear_scan (decays)");
        decay = gate_out;
        ld_decay = heads * per_head;
        decay_off = 0;
        if (gate_mode == LS_GATE_STEP) kscale = gate_out + n;
    }
    // rows of a column over KP lanes, KPT rows a lane: the fewest lanes that keep a lane's share at 16 rows or fewer
    int kp = 1;
    while (kp < 32 && (dk + kp - 1) / kp > 16) kp <<= 1;
    const int per_lane = (dk + kp - 1) / kp;
    const int kpt = per_lane <= 4 ? 4 : per_lane <= 8 ? 8 : per_lane <= 16 ? 16 : 32;
    const int trow = kp * (kpt + 4), cols_per_block = LS_WARPS * (32 / kp);     // a token's floats in shared memory, padded
    int chunk = 16;          // more would be fewer barriers, and fewer blocks an SM (shared memory): measured slower
    while (chunk > 1 && (size_t)chunk * (3 * trow + cols_per_block) * sizeof(float) > 40 * 1024) chunk >>= 1;
    const size_t smem = (size_t)chunk * (3 * trow + cols_per_block) * sizeof(float);
    LinearScanArgs a = {y, state, slot_stride, q, k, v, ld_q, q_off, ld_k, k_off, ld_v, v_off, decay, ld_decay, decay_off,
                        gate_per_channel, kscale, gate_apart ? LS_GATE_RAW : gate_mode,
                        gate_mode == LS_GATE_SIGMOID_POW ? 1.f / tau : 0.f, a_log, dt_bias, skip, q_scale, cu_seqlens, state_slots,
                        heads, groups, dk, dv, kp, chunk,
                        dk % 4 == 0 && slot_stride % 4 == 0 && ((uintptr_t)state | (uintptr_t)scratch) % 16 == 0, stretches, scratch,
                        scratch ? scratch + (long long)num_seqs * stretches * heads * dk * dv : nullptr,
                        scratch ? scratch + (long long)num_seqs * stretches * heads * dk * (dv + 1) : nullptr};
    dim3 grid(heads * ((dv + cols_per_block - 1) / cols_per_block), num_seqs, stretches);
    typedef __nv_bfloat16 B;
#define TI_SCAN(KPT, MODE)                                                                                          \
    do {                                                                                                            \
        if (dtype == TI_F32) ti_launch(linear_scan_kernel<float, KPT, MODE>, grid, LS_WARPS * 32, smem, stream, a); \
        else ti_launch(linear_scan_kernel<B, KPT, MODE>, grid, LS_WARPS * 32, smem, stream, a);                     \
    } while (0)
#define TI_SCAN_PASS(MODE)             \
    do {                               \
        if (kpt == 4) TI_SCAN(4, MODE);        \
        else if (kpt == 8) TI_SCAN(8, MODE);   \
        else if (kpt == 16) TI_SCAN(16, MODE); \
        else TI_SCAN(32, MODE);                \
    } while (0)
    TI_REQUIRE(dtype == TI_F32 || dtype == TI_BF16, "linear_scan: unknown dtype %d", dtype);
    if (stretches == 1) {
        TI_SCAN_PASS(0);
        TI_CHECK_LAUNCH("linear_scan");
        return 0;
    }
    TI_SCAN_PASS(1);
    TI_CHECK_LAUNCH("linear_scan (stretches from zero)");
    const int per = heads * dv * dk;
    ti_launch(linear_scan_fold_kernel, dim3((per + 255) / 256, num_seqs), 256, 0, stream, state, slot_stride, a.part_b,
              (const float*)a.part_a, state_slots, stretches, heads, dk, dv);
    TI_CHECK_LAUNCH("linear_scan (fold)");
    TI_SCAN_PASS(2);
    TI_CHECK_LAUNCH("linear_scan (what the stretches' starts give)");
#undef TI_SCAN_PASS
#undef TI_SCAN
    return 0;
}

// One block per (token, group). gate_first: the gate multiplies y before the norm; otherwise after it.
template <typename T>
__global__ void gated_group_norm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ gate,
                                        int ld_gate, int gate_off, const float* __restrict__ w, int w_len, int width,
                                        int group, float eps, int gate_first, float out_scale, int gate_sigmoid) {
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x, g0 = blockIdx.y * group;
    const float* yrow = y + (size_t)t * width + g0;
    const T* grow = gate ? gate + (size_t)t * ld_gate + gate_off + g0 : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = yrow[i];
        if (gate_first && grow) {
            const float z = to_f32(grow[i]);
            v *= (gate_sigmoid ? 1.f : z) / (1.f + expf(-z));
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)group + eps) * out_scale;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = yrow[i];
        float gz = 1.f;
        if (grow) {
            const float z = to_f32(grow[i]);
            gz = (gate_sigmoid ? 1.f : z) / (1.f + expf(-z));
        }
        if (gate_first) v *= gz;
        v = v * inv * w[(g0 + i) % w_len];
        if (!gate_first) v *= gz;
        out[(size_t)t * width + g0 + i] = from_f32<T>(v);
    }
}

// The same with a warp per (token, group) and four neighbouring features a lane a trip (groups of a multiple of four
// features up to 512, rows on 16-byte boundaries): y and the gate are read once and kept in registers, no block-wide
// barrier, 16-byte loads of y, one store per four features.
template <typename T>
__global__ void gated_group_norm_warp_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ gate,
                                             int ld_gate, int gate_off, const float* __restrict__ w, int w_len, int width,
                                             int group, float eps, int gate_first, float out_scale, long long num_groups,
                                             int wide_rows, int gate_sigmoid) {
    constexpr int TRIPS = 4;                             // 4 trips x 32 lanes x 4 features = 512
    ti_grid_launch_dependents();
    ti_grid_wait();
    const long long gi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gi >= num_groups) return;
    const int lane = threadIdx.x & 31, per_row = width / group;
    const long long t = gi / per_row;
    const int g0 = (int)(gi % per_row) * group;
    const float* yrow = y + (size_t)t * width + g0;
    const T* grow = gate ? gate + (size_t)t * ld_gate + gate_off + g0 : nullptr;
    float v[TRIPS][4], gz[TRIPS][4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < TRIPS; ++k) {
        const int i = k * 128 + lane * 4;
        if (i < group) {
            const float4 f = *reinterpret_cast<const float4*>(yrow + i);
            v[k][0] = f.x; v[k][1] = f.y; v[k][2] = f.z; v[k][3] = f.w;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float z = grow ? to_f32(grow[i + e]) : 0.f;
                gz[k][e] = grow ? (gate_sigmoid ? 1.f : z) / (1.f + expf(-z)) : 1.f;
                if (gate_first) v[k][e] *= gz[k][e];
                ss += v[k][e] * v[k][e];
            }
        }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)group + eps) * out_scale;
#pragma unroll
    for (int k = 0; k < TRIPS; ++k) {
        const int i = k * 128 + lane * 4;
        if (i < group) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = v[k][e] * inv * w[(g0 + i + e) % w_len];
                o[e] = gate_first ? x : x * gz[k][e];
            }
            T* dst = out + (size_t)t * width + g0 + i;
            if (wide_rows) {
                if (sizeof(T) == 4) {
                    *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                } else {
                    uint2 u;
                    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(o[0], o[1]);
                    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(o[2], o[3]);
                    *reinterpret_cast<uint2*>(dst) = u;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) dst[e] = from_f32<T>(o[e]);
            }
        }
    }
}

TI_API int ti_gated_group_norm(void* out, const float* y, const void* gate, int ld_gate, int gate_off, const float* w,
                               int w_len, int num_tokens, int width, int group, float eps, int gate_first, float out_scale,
                               int gate_sigmoid, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && width > 0 && group > 0 && width % group == 0 && w_len > 0, "gated_group_norm: bad sizes");
    TI_REQUIRE(width / group <= 65535, "gated_group_norm: too many groups");
    if (num_tokens == 0) return 0;
    if (group % 4 == 0 && group <= 512 && (uintptr_t)y % 16 == 0) {          // a warp a group; larger groups: a block
        const long long num_groups = (long long)num_tokens * (width / group);
        const unsigned blocks = (unsigned)((num_groups + 7) / 8);
        const int wide_rows = (uintptr_t)out % 16 == 0;          // width and group are multiples of four: rows of out start on 8 or 16 bytes
        if (dtype == TI_F32)
            ti_launch(gated_group_norm_warp_kernel<float>, blocks, 256, 0, stream, (float*)out, y, (const float*)gate, ld_gate,
                      gate_off, w, w_len, width, group, eps, gate_first, out_scale, num_groups, wide_rows, gate_sigmoid);
        else if (dtype == TI_BF16)
            ti_launch(gated_group_norm_warp_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, y,
                      (const __nv_bfloat16*)gate, ld_gate, gate_off, w, w_len, width, group, eps, gate_first, out_scale, num_groups,
                      wide_rows, gate_sigmoid);
        else TI_REQUIRE(false, "gated_group_norm: unknown dtype %d", dtype);
        TI_CHECK_LAUNCH("gated_group_norm");
        return 0;
    }
    int threads = 32;          // a thread's trips wait for one another's loads: as many threads as a block may have
    while (threads < 1024 && threads < group) threads <<= 1;
    dim3 grid(num_tokens, width / group);
    if (dtype == TI_F32)
        ti_launch(gated_group_norm_kernel<float>, grid, threads, 0, stream, (float*)out, y, (const float*)gate, ld_gate, gate_off,
                  w, w_len, width, group, eps, gate_first, out_scale, gate_sigmoid);
    else if (dtype == TI_BF16)
        ti_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, threads, 0, stream, (__nv_bfloat16*)out, y,
                  (const __nv_bfloat16*)gate, ld_gate, gate_off, w, w_len, width, group, eps, gate_first, out_scale, gate_sigmoid);
    else TI_REQUIRE(false, "gated_group_norm: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("gated_group_norm");
    return 0;
}
