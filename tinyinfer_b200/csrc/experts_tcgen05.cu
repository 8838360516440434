// The grouped products of routed experts for steps that bring an expert many rows, on tcgen05: the plan's row tiles
// hold 128 sorted rows of one expert (experts.cu), a work unit is a row tile x 128 of the expert's output features.
// One CTA an SM walks the units; warp 0 copies operand tiles with TMA (the sorted activations [slots, K] and the
// experts' weights as one matrix [experts * N, K], each through one tensor map, 64 k a stage, 128-byte swizzle),
// warp 1 issues the MMAs (128 x 128 x 16, float32 accumulators in tensor memory, two of them so that the epilogue of
// a unit runs behind the MMAs of the next), warps 2 to 5 read the accumulator (a lane a row), apply max(v, 0)^2 for
// the up form, and store. Rows of a tile beyond the expert's (the next expert's rows, or nothing) and features
// beyond N (the next expert's weights) are computed and not stored. Every wait is bounded and reports through the
// status word; tensor memory is freed on the common exit.
#include "sm100_ptx.cuh"

namespace {
constexpr int GT_BM = 128, GT_BN = 128, GT_BK = 64, GT_UMMA_K = 16, GT_THREADS = 192, GT_STAGES = 5;
constexpr int GT_STAGE_BYTES = (GT_BM + GT_BN) * GT_BK * 2;
constexpr int GT_SMEM = GT_STAGES * GT_STAGE_BYTES + 1024 + 256;

struct GtParams {
    void* out;
    const int* tiles;          // [expert, first row, rows] per row tile
    const int* num_tiles;
    int N, K, col_tiles, up;
    int* status;
};

__global__ void __launch_bounds__(GT_THREADS, 1)
moe_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const GtParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages + GT_STAGES * GT_STAGE_BYTES);
    const uint32_t bar0 = smem_u32(bars);                 // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (GT_STAGES + s); };
    auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * GT_STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * GT_STAGES + 2 + a); };
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;

    ti_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) abort_sh = 0;
    if (threadIdx.x < 2 * GT_STAGES + 4) {
        mbar_init(bar0 + 8u * threadIdx.x, (int)threadIdx.x >= 2 * GT_STAGES + 2 ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_sh, 2 * GT_BN);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_sh;
    ti_grid_wait();                                        // the plan, the sorted rows and `out` belong to earlier kernels until now
    const int num_units = p.num_tiles[0] * p.col_tiles;   // a unit: row tile (unit / col_tiles), column tile (unit % col_tiles)
    const int num_kb = (p.K + GT_BK - 1) / GT_BK;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
                const int tile = unit / p.col_tiles, ct = unit % p.col_tiles;
                const int expert = p.tiles[3 * tile], row0 = p.tiles[3 * tile + 1];
                const int w_row = expert * p.N + ct * GT_BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % GT_STAGES;
                    const uint32_t ph = (it / GT_STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, 31)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), GT_STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(stages + s * GT_STAGE_BYTES);
                    tma_load_2d(a_dst, &map_x, full_bar(s), kb * GT_BK, row0);
                    tma_load_2d(a_dst + GT_BM * GT_BK * 2, &map_w, full_bar(s), kb * GT_BK, w_row);
                }
            }
            if (!ok) {                                     // let the copies in flight land before shared memory is given up
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 1000000ull) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(GT_BM, GT_BN);
            uint32_t it = 0, unit_i = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x, ++unit_i) {
                const uint32_t as = unit_i & 1u, aph = (unit_i >> 1) & 1u;
                if (!mbar_wait(acc_empty_bar(as), aph ^ 1u, abort_flag, p.status, 32)) { ok = false; break; }
                tmem_fence_after();
                const uint32_t d_tmem = tmem_base + as * GT_BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % GT_STAGES;
                    const uint32_t ph = (it / GT_STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, 33)) { ok = false; break; }
                    tmem_fence_after();
                    const uint32_t a_addr = smem_u32(stages + s * GT_STAGE_BYTES);
                    const uint64_t adesc = make_sw128_desc(a_addr);
                    const uint64_t bdesc = make_sw128_desc(a_addr + GT_BM * GT_BK * 2);
#pragma unroll
                    for (int k = 0; k < GT_BK / GT_UMMA_K; ++k)
                        umma_bf16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(acc_full_bar(as));
            }
        }
    } else {
        const int lane_group = warp & 3;                   // the 32 accumulator lanes this warp may read
        const int r = lane_group * 32 + lane;
        uint32_t unit_i = 0;
        bool ok = true;
        for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x, ++unit_i) {
            const int tile = unit / p.col_tiles, ct = unit % p.col_tiles;
            const int row0 = p.tiles[3 * tile + 1], rows = p.tiles[3 * tile + 2];
            const uint32_t as = unit_i & 1u, aph = (unit_i >> 1) & 1u;
            if (!mbar_wait(acc_full_bar(as), aph, abort_flag, p.status, 34)) { ok = false; break; }
            tmem_fence_after();
            const uint32_t t_addr = tmem_base + as * GT_BN + ((uint32_t)(lane_group * 32) << 16);
            const bool live = r < rows;
            const int n0 = ct * GT_BN;
            for (int c = 0; c < GT_BN; c += 32) {
                float v[32];
                tmem_ld32(t_addr + c, v);
                if (!live || n0 + c >= p.N) continue;
                const size_t at = (size_t)(row0 + r) * p.N + n0 + c;
                if (p.up) {
                    if (p.up == 1) {                          // up == 2: stored as it is, the activation is a kernel of its own
#pragma unroll
                        for (int i = 0; i < 32; ++i) { v[i] = fmaxf(v[i], 0.f); v[i] *= v[i]; }
                    }
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + at;
                    if (n0 + c + 32 <= p.N && (p.N & 7) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 q;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                            *reinterpret_cast<uint4*>(dst + i) = q;
                        }
                    } else {
                        for (int i = 0; i < 32 && n0 + c + i < p.N; ++i) dst[i] = __float2bfloat16_rn(v[i]);
                    }
                } else {
                    float* dst = reinterpret_cast<float*>(p.out) + at;
                    if (n0 + c + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    } else {
                        for (int i = 0; i < 32 && n0 + c + i < p.N; ++i) dst[i] = v[i];
                    }
                }
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(as));  // this accumulator may be overwritten
        }
    }
    // ---------------------------------------------------------------- common exit
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        tmem_dealloc(tmem_base, 2 * GT_BN);
    }
}
}  // namespace

// 1 if the tcgen05 form takes these operands: whole k blocks, rows on 16-byte boundaries, operands at least a box tall.
TI_API int ti_moe_gemm_tcgen05_ok(int slots, int experts, int N, int K) {
    return (K % GT_BK == 0 && slots >= GT_BM && (long long)experts * N >= GT_BN && N > 0) ? 1 : 0;
}
TI_API int ti_moe_tcgen05_tile_rows() { return GT_BM; }

// x: sorted rows [slots, K] bfloat16; w [experts, N, K] bfloat16; tiles/num_tiles: the plan with row tiles of 128.
// up == 1: out [slots, N] bfloat16 after max(v, 0)^2; up == 2: bfloat16 as it is; else out [slots, N] float32.
TI_API int ti_moe_gemm_tcgen05(void* out, const void* x, const void* w, const int* tiles, const int* num_tiles, int slots,
                               int experts, int N, int K, int max_tiles, int up, int* status, cudaStream_t stream) {
    TI_REQUIRE(ti_moe_gemm_tcgen05_ok(slots, experts, N, K), "moe_gemm_tcgen05: operands [%d, %d] x [%d, %d, %d] are not taken", slots, K, experts, N, K);
    TI_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0, "moe_gemm_tcgen05: operands must be 16-byte aligned");
    if (max_tiles <= 0) return 0;
    CUtensorMap map_x, map_w;
    if (!ti_get_bf16_map(x, slots, K, GT_BM, &map_x)) return -1;
    if (!ti_get_bf16_map(w, (long long)experts * N, K, GT_BN, &map_w)) return -1;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(moe_gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM);
        TI_REQUIRE(e == cudaSuccess, "moe_gemm_tcgen05: cannot get %d bytes of shared memory: %s", GT_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    GtParams p;
    p.out = out; p.tiles = tiles; p.num_tiles = num_tiles; p.N = N; p.K = K; p.col_tiles = (N + GT_BN - 1) / GT_BN; p.up = up;
    p.status = status;
    const long long units = (long long)max_tiles * p.col_tiles;
    const int grid = (int)(units < ti_sm_count() ? units : ti_sm_count());
    ti_launch(moe_gemm_tcgen05_kernel, grid, GT_THREADS, GT_SMEM, stream, map_x, map_w, p);
    TI_CHECK_LAUNCH("moe_gemm_tcgen05");
    return 0;
}
