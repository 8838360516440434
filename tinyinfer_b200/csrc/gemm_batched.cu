// out[b][m][n] = act(sum_k x[b][m][k] * w[b][n][k] + bias[b][n]) for a batch of small matrix products that share
// their shapes but not their operands: per-head projections of an attention (the head is the batch), the blocks
// of a block-diagonal gate matrix (the block is the batch). Every operand has a row stride and a batch stride, so
// heads or blocks that lie side by side in a row of a [tokens, features] tensor are read and written where they are.
// float32 FMA accumulation in a fixed k order; a row's result does not depend on which other rows share its tile.
// act: 0 none, 1 logistic sigmoid. gate (may be null; the operands' dtype, rows of ldg elements, batch b's columns from
// b * sg on): the result is multiplied by sigmoid(gate[m][b * sg + n]), an output gate that another product made.
#include "common.cuh"
#include "mma_tile.cuh"

constexpr int GB_BM = 64, GB_BN = 64, GB_BK = 16, GB_THREADS = 256;

struct GbShape {
    int M, N, K;
    long long ldx, sx, ldw, sw, ldo, so, sbias;
    const void* gate; long long ldg, sg;
};

template <typename T, typename OutT, int ACT>
__global__ void __launch_bounds__(GB_THREADS) gemm_batched_kernel(
    OutT* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ bias, GbShape s) {
    __shared__ float As[GB_BK][GB_BM + 4];
    __shared__ float Bs[GB_BK][GB_BN + 4];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int b = blockIdx.z;
    const int m0 = blockIdx.y * GB_BM, n0 = blockIdx.x * GB_BN;
    x += (size_t)b * s.sx;
    w += (size_t)b * s.sw;
    out += (size_t)b * s.so;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < s.K; k0 += GB_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * GB_THREADS;
            const int row = idx >> 4, col = idx & 15;
            const int k = k0 + col;
            const int m = m0 + row, n = n0 + row;
            As[col][row] = (m < s.M && k < s.K) ? to_f32(x[(size_t)m * s.ldx + k]) : 0.f;
            Bs[col][row] = (n < s.N && k < s.K) ? to_f32(w[(size_t)n * s.ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GB_BK; ++kk) {
            float a[4], c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) c[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], c[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= s.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= s.N) continue;
            float v = acc[i][j];
            if (bias) v += bias[(size_t)b * s.sbias + n];
            if (ACT == 1) v = 1.f / (1.f + expf(-v));
            if (s.gate) v *= 1.f / (1.f + expf(-to_f32(((const T*)s.gate)[(size_t)m * s.ldg + (size_t)b * s.sg + n])));
            out[(size_t)m * s.ldo + n] = from_f32<OutT>(v);
        }
    }
}

// The same product on the tensor cores (bfloat16; every stride, offset and K a multiple of 8): see mma_tile.cuh.
template <typename OutT, int ACT>
__global__ void __launch_bounds__(mt::THREADS) gemm_batched_mma_kernel(
    OutT* __restrict__ out, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    const float* __restrict__ bias, GbShape s) {
    __shared__ __align__(16) __nv_bfloat16 ring[mt::SMEM_BYTES / 2];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int b = blockIdx.z;
    const int m0 = blockIdx.y * mt::BM, n0 = blockIdx.x * mt::BN;
    const __nv_bfloat16* xb = x + (size_t)b * s.sx;
    const __nv_bfloat16* wb = w + (size_t)b * s.sw;
    out += (size_t)b * s.so;
    float acc[2][4][4];
    mt::tile_product<2>(acc, ring,
                     [&](int r) { return m0 + r < s.M ? xb + (size_t)(m0 + r) * s.ldx : nullptr; },
                     [&](int n) { return n0 + n < s.N ? wb + (size_t)(n0 + n) * s.ldw : nullptr; }, s.K, w);
    mt::for_each_pair<2>(acc, [&](int r, int c, float v0, float v1) {
        const int m = m0 + r, n = n0 + c;
        if (m >= s.M) return;
        float v[2] = {v0, v1};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (n + e >= s.N) continue;
            float u = v[e];
            if (bias) u += bias[(size_t)b * s.sbias + n + e];
            if (ACT == 1) u = 1.f / (1.f + expf(-u));
            if (s.gate) u *= 1.f / (1.f + expf(-__bfloat162float(((const __nv_bfloat16*)s.gate)[(size_t)m * s.ldg + (size_t)b * s.sg + n + e])));
            out[(size_t)m * s.ldo + n + e] = from_f32<OutT>(u);
        }
    });
}

TI_API int ti_gemm_batched(void* out, const void* x, const void* w, const float* bias, int batch, int M, int N, int K,
                           long long ldx, long long sx, long long ldw, long long sw, long long ldo, long long so,
                           long long sbias, int act, int out_f32, const void* gate, long long ldg, long long sg, int dtype,
                           cudaStream_t stream) {
    TI_REQUIRE(batch > 0 && M >= 0 && N > 0 && K > 0, "gemm_batched: bad sizes");
    TI_REQUIRE(act == 0 || act == 1, "gemm_batched: unknown activation %d", act);
    TI_REQUIRE(batch <= 65535, "gemm_batched: too many batches");
    if (M == 0) return 0;
    dim3 grid((N + GB_BN - 1) / GB_BN, (M + GB_BM - 1) / GB_BM, batch);
    TI_REQUIRE(grid.y <= 65535, "gemm_batched: too many rows");
    GbShape s{M, N, K, ldx, sx, ldw, sw, ldo, so, sbias, gate, ldg, sg};
    typedef __nv_bfloat16 B;
#define GB_LAUNCH(T, O, A) ti_launch(gemm_batched_kernel<T, O, A>, grid, GB_THREADS, 0, stream, (O*)out, (const T*)x, (const T*)w, bias, s)
    if (dtype == TI_F32) {
        if (act) GB_LAUNCH(float, float, 1); else GB_LAUNCH(float, float, 0);
    } else if (dtype == TI_BF16 && K % 8 == 0 && ldx % 8 == 0 && sx % 8 == 0 && ldw % 8 == 0 && sw % 8 == 0 &&
               ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0) {
        dim3 mgrid((N + mt::BN - 1) / mt::BN, (M + mt::BM - 1) / mt::BM, batch);
        TI_REQUIRE(mgrid.y <= 65535, "gemm_batched: too many rows");
#define GB_MMA(O, A) ti_launch(gemm_batched_mma_kernel<O, A>, mgrid, mt::THREADS, 0, stream, (O*)out, (const B*)x, (const B*)w, bias, s)
        if (out_f32) { if (act) GB_MMA(float, 1); else GB_MMA(float, 0); }
        else { if (act) GB_MMA(B, 1); else GB_MMA(B, 0); }
#undef GB_MMA
    } else if (dtype == TI_BF16) {
        if (out_f32) { if (act) GB_LAUNCH(B, float, 1); else GB_LAUNCH(B, float, 0); }
        else { if (act) GB_LAUNCH(B, B, 1); else GB_LAUNCH(B, B, 0); }
    } else TI_REQUIRE(false, "gemm_batched: unknown dtype %d", dtype);
#undef GB_LAUNCH
    TI_CHECK_LAUNCH("gemm_batched");
    return 0;
}
