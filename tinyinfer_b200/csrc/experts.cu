// A feed-forward made of many small experts, of which every token runs a few chosen by a router.
//   route    : z = W_router x in float32 from the token's row (the float32 residual, or a sublayer's input in the
//              compute dtype), s = softmax(z) over all experts (or, scoring 1, sigmoid(z) of each expert by itself),
//              the `top` largest s + correction (a learned number per
//              expert that only steers the choice; first index on ties), weights s_k / (sum of the chosen + weight_eps)
//              or, without renormalisation, s_k itself; also counts the tokens of every expert and gives each
//              (token, choice) its rank among them. The last experts of the router may be identity experts, whose
//              output is the token's row itself: they have no weights, the plan gives them no tiles, and `combine`
//              adds weight * row for them
//   plan     : one block: where every expert's rows start in the sorted order, and the list of row tiles
//              [expert, first row, rows] that the grouped product walks
//   place    : slot of every (token, choice) in the sorted order and the token of every slot
//   grouped product : for every tile, rows x W[expert]^T with float32 FMA accumulation in a fixed k order; the up
//              form gathers its rows from the tokens and applies max(v, 0)^2, the down form reads the sorted rows
//   combine_norm_add : y = sum_k weight_k * down[slot_k] (+ the shared expert's output), in choice order, then the
//              residual x32 += w * y * rsqrt(mean(y^2) + eps) and its copy in the compute dtype
//   combine  : the same weighted sum alone, identity experts included, in the compute dtype
//   clamped_glu : an expert's gated activation on the stored product [gate | up]: g = min(gate, limit),
//              u = clamp(up, -limit, limit), g * sigmoid(alpha * g) * (u + 1)
//   silu_glu : silu(gate) * up on the stored product [gate | up]; optionally both halves of a row times the weight of its
//              (token, choice) first: experts that are weighted at their INPUT. The up product is linear, so
//              W (s h) = s (W h) and the weight rides in this kernel; the activation is not, so it cannot move further
// A token's result depends on its own row alone: no capacity, nothing dropped, whatever else is in the batch.
// Nothing here reads back to the host: grids are sized for the worst case and tiles beyond the plan's count return.
#include "common.cuh"
#include "mma_tile.cuh"

constexpr int EX_MAX_TOP = 16;

// ------------------------------------------------------------------ route
// One block per token: its warps share out the experts' logits (16-byte loads of the router's rows where they are
// aligned), then the first warp holds the scores of up to 32 * EX_PER_LANE experts, a lane apiece, and chooses.
constexpr int EX_PER_LANE = 8;
constexpr int EX_ROUTE_THREADS = 512;

template <typename T, typename XT>
__global__ void __launch_bounds__(EX_ROUTE_THREADS) moe_route_kernel(
    int* __restrict__ chosen, float* __restrict__ weight, int* __restrict__ rank, int* __restrict__ counts,
    const XT* __restrict__ x32, const T* __restrict__ w_router, int num_tokens, int hidden, int experts, int top,
    float weight_eps, const float* __restrict__ correction, int renorm, int scoring) {
    __shared__ float logits[32 * EX_PER_LANE];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const XT* x = x32 + (size_t)t * hidden;
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = sizeof(XT) == 4 && hidden % VEC == 0 && ((uintptr_t)w_router & 15) == 0 && ((uintptr_t)x32 & 15) == 0;
    for (int e = warp; e < experts; e += EX_ROUTE_THREADS / 32) {
        const T* w = w_router + (size_t)e * hidden;
        float dot = 0.f;
        if (aligned) {
            const uint4* w4 = reinterpret_cast<const uint4*>(w);
#pragma unroll 4
            for (int v = lane; v < hidden / VEC; v += 32) {
                const uint4 q = w4[v];
                const T* we = reinterpret_cast<const T*>(&q);
                const float4* xp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)v * VEC);
#pragma unroll
                for (int i = 0; i < VEC / 4; ++i) {
                    const float4 f = xp[i];
                    dot = fmaf(f.x, to_f32(we[4 * i]), dot);
                    dot = fmaf(f.y, to_f32(we[4 * i + 1]), dot);
                    dot = fmaf(f.z, to_f32(we[4 * i + 2]), dot);
                    dot = fmaf(f.w, to_f32(we[4 * i + 3]), dot);
                }
            }
        } else {
            for (int i = lane; i < hidden; i += 32) dot = fmaf(to_f32(x[i]), to_f32(w[i]), dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) logits[e] = dot;
    }
    __syncthreads();
    if (warp != 0) return;
    float z[EX_PER_LANE];                              // lane holds experts lane, lane + 32, ...
#pragma unroll
    for (int k = 0; k < EX_PER_LANE; ++k) z[k] = (k * 32 + lane < experts) ? logits[k * 32 + lane] : -INFINITY;
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < EX_PER_LANE; ++k) mx = fmaxf(mx, z[k]);
    mx = warp_max(mx);
    float sum = 0.f;
    float s[EX_PER_LANE];
#pragma unroll
    for (int k = 0; k < EX_PER_LANE; ++k) {
        // -1 marks "no such expert" (scores are >= 0)
        s[k] = (z[k] == -INFINITY) ? -1.f : scoring == 1 ? 1.f / (1.f + expf(-z[k])) : expf(z[k] - mx);
        if (s[k] > 0.f) sum += s[k];
    }
    sum = warp_sum(sum);
    const float inv = scoring == 1 ? 1.f : 1.f / sum;            // a sigmoid score stands by itself
#pragma unroll
    for (int k = 0; k < EX_PER_LANE; ++k) if (s[k] >= 0.f) s[k] *= inv;
    // what the choice goes by: the score plus the expert's correction; -inf: no such expert, or taken already
    float c[EX_PER_LANE];
#pragma unroll
    for (int k = 0; k < EX_PER_LANE; ++k)
        c[k] = s[k] < 0.f ? -INFINITY : (correction ? s[k] + correction[k * 32 + lane] : s[k]);
    float best[EX_MAX_TOP];
    int who[EX_MAX_TOP];
    float total = 0.f;
    for (int ch = 0; ch < top; ++ch) {
        float v = -INFINITY, sv = 0.f;
        int idx = 0x7fffffff;
#pragma unroll
        for (int k = 0; k < EX_PER_LANE; ++k)
            if (c[k] > v) { v = c[k]; sv = s[k]; idx = k * 32 + lane; }     // ascending index within a lane: the first wins
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const float os = __shfl_xor_sync(0xffffffffu, sv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; sv = os; idx = oi; }
        }
        best[ch] = sv;
        who[ch] = idx;
        total += sv;
#pragma unroll
        for (int k = 0; k < EX_PER_LANE; ++k)
            if (idx == k * 32 + lane) c[k] = -INFINITY;
    }
    if (lane == 0) {
        const float norm = renorm ? 1.f / (total + weight_eps) : 1.f;
        for (int ch = 0; ch < top; ++ch) {
            chosen[(size_t)t * top + ch] = who[ch];
            weight[(size_t)t * top + ch] = best[ch] * norm;
            rank[(size_t)t * top + ch] = atomicAdd(counts + who[ch], 1);
        }
    }
}

// ------------------------------------------------------------------ plan
// counts[e] -> starts[e] (exclusive sums, starts[experts] = all rows) and tiles [expert, first row, rows] of the
// first real_experts experts (the others have no weights to multiply by); num_tiles[0] = how many. One block;
// experts and tiles are few.
__global__ void moe_plan_kernel(int* __restrict__ starts, int* __restrict__ tiles, int* __restrict__ num_tiles,
                                const int* __restrict__ counts, int experts, int real_experts, int tile_rows, int max_tiles) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    if (threadIdx.x != 0) return;
    int row = 0, n = 0;
    for (int e = 0; e < experts; ++e) {
        starts[e] = row;
        const int c = counts[e];
        for (int r = 0; r < c && n < max_tiles && e < real_experts; r += tile_rows) {      // identity experts: rows, no tiles
            tiles[3 * n] = e;
            tiles[3 * n + 1] = row + r;
            tiles[3 * n + 2] = min(tile_rows, c - r);
            ++n;
        }
        row += c;
    }
    starts[experts] = row;
    num_tiles[0] = n;
}

__global__ void moe_place_kernel(int* __restrict__ slot_of, int* __restrict__ token_of, const int* __restrict__ chosen,
                                 const int* __restrict__ rank, const int* __restrict__ starts, int n, int top,
                                 float* __restrict__ slot_weight, const float* __restrict__ weight) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int slot = starts[chosen[i]] + rank[i];
    slot_of[i] = slot;
    token_of[slot] = i / top;
    if (slot_weight) slot_weight[slot] = weight[i];        // the weights in expert order, for whoever works on sorted rows
}

// scoring 0: softmax over the experts; 1: the sigmoid of each logit.
// slot_weight (float32 [tokens * top], or null): also receives every (token, choice)'s weight at its row in expert order.
// counts (experts ints) must be zero on entry; the launcher clears them. x_dtype: of the tokens' rows (float32, or
// the compute dtype of a sublayer's input); correction: float32 [experts] or null; renorm: the weights are divided by
// their sum; real_experts: how many of the router's outputs are experts with weights (the rest: identity experts).
TI_API int ti_moe_route(int* chosen, float* weight, int* rank, int* counts, int* starts, int* tiles, int* num_tiles,
                        int* slot_of, int* token_of, const void* x, const void* w_router, int num_tokens, int hidden,
                        int experts, int top, float weight_eps, const float* correction, int renorm, int real_experts,
                        int tile_rows, int max_tiles, int scoring, float* slot_weight, int x_dtype, int dtype,
                        cudaStream_t stream) {
    TI_REQUIRE(scoring == 0 || scoring == 1, "moe_route: scoring %d is neither the softmax (0) nor the sigmoid (1)", scoring);
    TI_REQUIRE(num_tokens >= 0 && hidden > 0 && experts > 0 && top > 0, "moe_route: bad sizes");
    TI_REQUIRE(top <= EX_MAX_TOP && top <= experts, "moe_route: top %d of %d experts (at most %d)", top, experts, EX_MAX_TOP);
    TI_REQUIRE(experts <= 32 * EX_PER_LANE, "moe_route: more than %d experts", 32 * EX_PER_LANE);
    TI_REQUIRE(real_experts >= 0 && real_experts <= experts, "moe_route: %d of %d experts have weights", real_experts, experts);
    TI_REQUIRE(x_dtype == TI_F32 || x_dtype == dtype, "moe_route: the rows are float32 or of the router's dtype");
    if (num_tokens == 0) return 0;
    cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * experts, stream);
    TI_REQUIRE(e == cudaSuccess, "moe_route: %s", cudaGetErrorString(e));
    const int blocks = num_tokens;
    typedef __nv_bfloat16 B;
#define EX_ROUTE(T, XT) ti_launch(moe_route_kernel<T, XT>, blocks, EX_ROUTE_THREADS, 0, stream, chosen, weight, rank, counts, \
                                  (const XT*)x, (const T*)w_router, num_tokens, hidden, experts, top, weight_eps, correction, renorm, scoring)
    if (dtype == TI_F32) EX_ROUTE(float, float);
    else if (dtype == TI_BF16 && x_dtype == TI_F32) EX_ROUTE(B, float);
    else if (dtype == TI_BF16) EX_ROUTE(B, B);
    else TI_REQUIRE(false, "moe_route: unknown dtype %d", dtype);
#undef EX_ROUTE
    TI_CHECK_LAUNCH("moe_route");
    ti_launch(moe_plan_kernel, 1, 32, 0, stream, starts, tiles, num_tiles, (const int*)counts, experts, real_experts, tile_rows,
              max_tiles);
    TI_CHECK_LAUNCH("moe_plan");
    const int n = num_tokens * top;
    ti_launch(moe_place_kernel, (n + 127) / 128, 128, 0, stream, slot_of, token_of, (const int*)chosen, (const int*)rank,
              (const int*)starts, n, top, slot_weight, (const float*)weight);
    TI_CHECK_LAUNCH("moe_place");
    return 0;
}

// ------------------------------------------------------------------ grouped product
constexpr int EG_BM = 32, EG_BN = 64, EG_BK = 16, EG_THREADS = 128;

// out[row][n] = act(sum_k x[src(row)][k] * w[expert][n][k]) for the rows of tile blockIdx.y.
// GATHER: src(row) = token_of[row] (rows of the step's tokens); else src(row) = row (sorted rows).
template <typename T, typename OutT, bool GATHER, bool RELU2>
__global__ void __launch_bounds__(EG_THREADS) moe_gemm_kernel(
    OutT* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w, const int* __restrict__ tiles,
    const int* __restrict__ num_tiles, const int* __restrict__ token_of, int N, int K) {
    __shared__ float As[EG_BK][EG_BM + 4];
    __shared__ float Bs[EG_BK][EG_BN + 4];
    __shared__ int src[EG_BM];
    ti_grid_launch_dependents();
    ti_grid_wait();
    if ((int)blockIdx.y >= num_tiles[0]) return;
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;             // 16 x 8 threads, 4 x 4 outputs each
    const int n0 = blockIdx.x * EG_BN;
    const T* we = w + (size_t)expert * N * K;
    if (tid < EG_BM) src[tid] = tid < rows ? (GATHER ? token_of[row0 + tid] : row0 + tid) : -1;
    __syncthreads();
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += EG_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {                   // 32 x 16 of x
            const int idx = tid + r * EG_THREADS;
            const int row = idx >> 4, col = idx & 15;
            const int k = k0 + col;
            const int s = src[row];
            As[col][row] = (s >= 0 && k < K) ? to_f32(x[(size_t)s * K + k]) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {                   // 64 x 16 of w
            const int idx = tid + r * EG_THREADS;
            const int row = idx >> 4, col = idx & 15;
            const int k = k0 + col, n = n0 + row;
            Bs[col][row] = (n < N && k < K) ? to_f32(we[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < EG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (RELU2) { v = fmaxf(v, 0.f); v *= v; }
            out[(size_t)(row0 + r) * N + n] = from_f32<OutT>(v);
        }
    }
}

// The same tiles on the tensor cores (bfloat16, K a multiple of 8): 32 rows x 128 columns a block, see mma_tile.cuh.
static_assert(mt::BM == EG_BM, "the plan's row tiles serve both kernels");

// MI = 2: row tiles of 32; MI = 4: of 64 (steps that bring an expert many rows: half the trips of its weights).
template <typename OutT, bool GATHER, bool RELU2, int MI>
__global__ void __launch_bounds__(mt::THREADS) moe_gemm_mma_kernel(
    OutT* __restrict__ out, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    const int* __restrict__ tiles, const int* __restrict__ num_tiles, const int* __restrict__ token_of, int N, int K) {
    __shared__ __align__(16) __nv_bfloat16 ring[mt::Ring<MI>::BYTES / 2];
    __shared__ int src[16 * MI];
    ti_grid_launch_dependents();
    ti_grid_wait();
    if ((int)blockIdx.y >= num_tiles[0]) return;
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * mt::BN;
    const __nv_bfloat16* we = w + (size_t)expert * N * K;
    if (threadIdx.x < 16 * MI) src[threadIdx.x] = threadIdx.x < rows ? (GATHER ? token_of[row0 + threadIdx.x] : row0 + threadIdx.x) : -1;
    __syncthreads();
    float acc[MI][4][4];
    mt::tile_product<MI>(acc, ring,
                     [&](int r) { return src[r] >= 0 ? x + (size_t)src[r] * K : nullptr; },
                     [&](int n) { return n0 + n < N ? we + (size_t)(n0 + n) * K : nullptr; }, K, w);
    mt::for_each_pair<MI>(acc, [&](int r, int c, float v0, float v1) {
        if (r >= rows) return;
        if (RELU2) { v0 = fmaxf(v0, 0.f); v0 *= v0; v1 = fmaxf(v1, 0.f); v1 *= v1; }
        OutT* dst = out + (size_t)(row0 + r) * N + n0 + c;
        if (n0 + c < N) dst[0] = from_f32<OutT>(v0);
        if (n0 + c + 1 < N) dst[1] = from_f32<OutT>(v1);
    });
}

TI_API int ti_moe_tile_rows() { return EG_BM; }

// up != 0: x [tokens, K] gathered through token_of, out [slots, N] in the compute dtype after max(v, 0)^2 (up == 1)
// or as it is (up == 2: the activation is a kernel of its own); else x [slots, K], out [slots, N] float32. w [experts, N, K]. max_tiles: the grid's height.
// 1 if row tiles of 64 are taken for these operands (the tensor-core form), else the plan must cut tiles of 32.
TI_API int ti_moe_wide_tiles_ok(int K, int dtype) { return dtype == TI_BF16 && K % 8 == 0 ? 1 : 0; }

TI_API int ti_moe_gemm(void* out, const void* x, const void* w, const int* tiles, const int* num_tiles, const int* token_of,
                       int N, int K, int max_tiles, int tile_rows, int up, int dtype, cudaStream_t stream) {
    TI_REQUIRE(N > 0 && K > 0 && max_tiles >= 0 && max_tiles <= 65535, "moe_gemm: bad sizes");
    const bool tensor_cores = dtype == TI_BF16 && K % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
    TI_REQUIRE(tile_rows == EG_BM || (tile_rows == 64 && tensor_cores), "moe_gemm: row tiles of %d are not taken here", tile_rows);
    if (max_tiles == 0) return 0;
    dim3 grid((N + EG_BN - 1) / EG_BN, max_tiles);
    typedef __nv_bfloat16 B;
    if (dtype == TI_F32) {
        if (up == 2) ti_launch(moe_gemm_kernel<float, float, true, false>, grid, EG_THREADS, 0, stream, (float*)out, (const float*)x, (const float*)w, tiles, num_tiles, token_of, N, K);
        else if (up) ti_launch(moe_gemm_kernel<float, float, true, true>, grid, EG_THREADS, 0, stream, (float*)out, (const float*)x, (const float*)w, tiles, num_tiles, token_of, N, K);
        else ti_launch(moe_gemm_kernel<float, float, false, false>, grid, EG_THREADS, 0, stream, (float*)out, (const float*)x, (const float*)w, tiles, num_tiles, token_of, N, K);
    } else if (tensor_cores) {
        dim3 mgrid((N + mt::BN - 1) / mt::BN, max_tiles);
#define EG_MMA(O, G, R, MI) ti_launch(moe_gemm_mma_kernel<O, G, R, MI>, mgrid, mt::THREADS, 0, stream, (O*)out, (const B*)x, (const B*)w, tiles, num_tiles, token_of, N, K)
        if (tile_rows == 64) { if (up == 2) EG_MMA(B, true, false, 4); else if (up) EG_MMA(B, true, true, 4); else EG_MMA(float, false, false, 4); }
        else { if (up == 2) EG_MMA(B, true, false, 2); else if (up) EG_MMA(B, true, true, 2); else EG_MMA(float, false, false, 2); }
#undef EG_MMA
    } else if (dtype == TI_BF16) {
        if (up == 2) ti_launch(moe_gemm_kernel<B, B, true, false>, grid, EG_THREADS, 0, stream, (B*)out, (const B*)x, (const B*)w, tiles, num_tiles, token_of, N, K);
        else if (up) ti_launch(moe_gemm_kernel<B, B, true, true>, grid, EG_THREADS, 0, stream, (B*)out, (const B*)x, (const B*)w, tiles, num_tiles, token_of, N, K);
        else ti_launch(moe_gemm_kernel<B, float, false, false>, grid, EG_THREADS, 0, stream, (float*)out, (const B*)x, (const B*)w, tiles, num_tiles, token_of, N, K);
    } else TI_REQUIRE(false, "moe_gemm: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("moe_gemm");
    return 0;
}

// ------------------------------------------------------------------ rows into expert order
// out[slot] = x[token_of[slot]]: the sorted copy that a product with tiled operand copies reads (a row a warp).
template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ token_of, int slots, int K) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (slot >= slots) return;
    const T* src = x + (size_t)token_of[slot] * K;
    T* dst = out + (size_t)slot * K;
    constexpr int VEC = 16 / sizeof(T);
    if (K % VEC == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        for (int i = lane; i < K / VEC; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = lane; i < K; i += 32) dst[i] = src[i];
    }
}

TI_API int ti_moe_gather(void* out, const void* x, const int* token_of, int slots, int K, int dtype, cudaStream_t stream) {
    TI_REQUIRE(slots >= 0 && K > 0, "moe_gather: bad sizes");
    if (slots == 0) return 0;
    const int blocks = (slots + 7) / 8;
    if (dtype == TI_F32) ti_launch(moe_gather_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)x, token_of, slots, K);
    else if (dtype == TI_BF16) ti_launch(moe_gather_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, token_of, slots, K);
    else TI_REQUIRE(false, "moe_gather: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("moe_gather");
    return 0;
}

// ------------------------------------------------------------------ combine + norm + residual
template <typename T>
__global__ void moe_combine_norm_add_kernel(float* __restrict__ x32, T* __restrict__ copy, const float* __restrict__ down,
                                            const T* __restrict__ shared_out, const int* __restrict__ slot_of,
                                            const float* __restrict__ weight, const float* __restrict__ norm_w, int size,
                                            int top, float eps) {
    extern __shared__ float row[];
    __shared__ float red[33];
    __shared__ int slots[EX_MAX_TOP];
    __shared__ float wts[EX_MAX_TOP];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        slots[threadIdx.x] = slot_of[(size_t)t * top + threadIdx.x];
        wts[threadIdx.x] = weight[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    const size_t base = (size_t)t * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float v = 0.f;
        for (int c = 0; c < top; ++c) v = fmaf(wts[c], down[(size_t)slots[c] * size + i], v);
        if (shared_out) v += to_f32(shared_out[base + i]);
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = x32[base + i] + norm_w[i] * row[i] * inv;
        x32[base + i] = v;
        if (copy) copy[base + i] = from_f32<T>(v);
    }
}

TI_API int ti_moe_combine_norm_add(float* x32, void* copy, const float* down, const void* shared_out, const int* slot_of,
                                   const float* weight, const float* norm_w, int num_tokens, int size, int top, float eps,
                                   int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && size > 0 && size <= 48 * 1024 / 4 && top > 0 && top <= EX_MAX_TOP, "moe_combine: bad sizes");
    if (num_tokens == 0) return 0;
    int threads = 32;
    while (threads < 512 && threads * 4 < size) threads <<= 1;
    const size_t smem = (size_t)size * 4;
    if (dtype == TI_F32)
        ti_launch(moe_combine_norm_add_kernel<float>, num_tokens, threads, smem, stream, x32, (float*)copy, down,
                  (const float*)shared_out, slot_of, weight, norm_w, size, top, eps);
    else if (dtype == TI_BF16)
        ti_launch(moe_combine_norm_add_kernel<__nv_bfloat16>, num_tokens, threads, smem, stream, x32, (__nv_bfloat16*)copy, down,
                  (const __nv_bfloat16*)shared_out, slot_of, weight, norm_w, size, top, eps);
    else TI_REQUIRE(false, "moe_combine: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("moe_combine_norm_add");
    return 0;
}

// ------------------------------------------------------------------ gated activation of an expert, combine alone
// in [rows][2 * ff] = [gate | up] as the grouped product stored it; out [rows][ff].
template <typename T>
__global__ void moe_clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ in, size_t rows, int ff, float limit, float alpha) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t n = rows * ff, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t r = i / ff;
        const int c = (int)(i % ff);
        const float g = fminf(to_f32(in[r * 2 * ff + c]), limit);
        const float u = fminf(fmaxf(to_f32(in[r * 2 * ff + ff + c]), -limit), limit);
        out[i] = from_f32<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
    }
}

TI_API int ti_moe_clamped_glu(void* out, const void* in, long long rows, int ff, float limit, float alpha, int dtype,
                              cudaStream_t stream) {
    TI_REQUIRE(rows >= 0 && ff > 0, "moe_clamped_glu: bad sizes");
    if (rows == 0) return 0;
    const long long want = (rows * ff + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == TI_F32) ti_launch(moe_clamped_glu_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)in, (size_t)rows, ff, limit, alpha);
    else if (dtype == TI_BF16) ti_launch(moe_clamped_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)in, (size_t)rows, ff, limit, alpha);
    else TI_REQUIRE(false, "moe_clamped_glu: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("moe_clamped_glu");
    return 0;
}

// in [rows][2 * ff] = [gate | up]; out [rows][ff] = silu(s gate) * (s up) with s = row_scale[row] (1 without it), float32
// arithmetic, one rounding.
template <typename T>
__global__ void moe_silu_glu_kernel(T* __restrict__ out, const T* __restrict__ in, size_t rows, int ff,
                                    const float* __restrict__ row_scale) {
    ti_grid_launch_dependents();
    ti_grid_wait();
    const size_t n = rows * ff, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t r = i / ff;
        const int c = (int)(i % ff);
        const float s = row_scale ? row_scale[r] : 1.f;
        const float g = s * to_f32(in[r * 2 * ff + c]);
        const float u = s * to_f32(in[r * 2 * ff + ff + c]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

TI_API int ti_moe_silu_glu(void* out, const void* in, long long rows, int ff, const float* row_scale, int dtype,
                           cudaStream_t stream) {
    TI_REQUIRE(rows >= 0 && ff > 0, "moe_silu_glu: bad sizes");
    if (rows == 0) return 0;
    const long long want = (rows * ff + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == TI_F32) ti_launch(moe_silu_glu_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)in, (size_t)rows, ff, row_scale);
    else if (dtype == TI_BF16) ti_launch(moe_silu_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)in, (size_t)rows, ff, row_scale);
    else TI_REQUIRE(false, "moe_silu_glu: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("moe_silu_glu");
    return 0;
}

// out[t] = sum_c weight[t][c] * (chosen[t][c] < real_experts ? down[slot_of[t][c]] : x[t]), in choice order, float32
// sums, one rounding. A block a token. weight may be null: every weight is one (experts weighted at their input).
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ down, const T* __restrict__ x,
                                   const int* __restrict__ chosen, const int* __restrict__ slot_of,
                                   const float* __restrict__ weight, int size, int top, int real_experts) {
    __shared__ int slots[EX_MAX_TOP];
    __shared__ float wts[EX_MAX_TOP];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        const size_t at = (size_t)t * top + threadIdx.x;
        slots[threadIdx.x] = chosen[at] < real_experts ? slot_of[at] : -1;
        wts[threadIdx.x] = weight ? weight[at] : 1.f;
    }
    __syncthreads();
    const size_t base = (size_t)t * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float v = 0.f;
        for (int c = 0; c < top; ++c)
            v = fmaf(wts[c], slots[c] >= 0 ? down[(size_t)slots[c] * size + i] : to_f32(x[base + i]), v);
        out[base + i] = from_f32<T>(v);
    }
}

TI_API int ti_moe_combine(void* out, const float* down, const void* x, const int* chosen, const int* slot_of,
                          const float* weight, int num_tokens, int size, int top, int real_experts, int dtype,
                          cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && size > 0 && top > 0 && top <= EX_MAX_TOP, "moe_combine: bad sizes");
    if (num_tokens == 0) return 0;
    int threads = 32;
    while (threads < 512 && threads * 4 < size) threads <<= 1;
    if (dtype == TI_F32)
        ti_launch(moe_combine_kernel<float>, num_tokens, threads, 0, stream, (float*)out, down, (const float*)x, chosen, slot_of, weight, size, top, real_experts);
    else if (dtype == TI_BF16)
        ti_launch(moe_combine_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (__nv_bfloat16*)out, down, (const __nv_bfloat16*)x, chosen, slot_of, weight, size, top, real_experts);
    else TI_REQUIRE(false, "moe_combine: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("moe_combine");
    return 0;
}
