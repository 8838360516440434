// Attention over a cached LATENT: a token leaves one row [c | k_rot] in the cache (c: a normed low-rank latent of
// `rank` features from which every head's keys and values are linear maps; k_rot: `rot` rotated key features that
// all heads share). Keys and values are never raised from the latent: a head's query is carried through its key
// map first (q_c = W_uk[h]^T q_plain, a batched product done by the caller), so that
//   score(i, j, h) = (q_c[i,h] . c[j] + q_rot[i,h] . k_rot[j]) * scale
// and the head's output is W_uv[h] (sum_j p_j c[j]): all heads of a token read the same cached rows, and the
// kernel here returns sum_j p_j c[j] per head. Softmax in float32 with a running maximum; optionally the
// denominator also holds exp(sink[h]), a term without key or value that is not scaled and counts once.
//
//   latent_prepare : from the down projections [q latent | kv latent | k_rot] of a token: RMSNorm of the query
//                    latent (-> the up projection's input), RMSNorm of the kv latent and rotation of k_rot
//                    (-> the cache row, through the block table)
//   latent_query   : rotation of the rotated part of every head's query into the query rows [q_c | q_rot]
//   latent_attend  : the attention; a block is one token and up to 8 heads (a warp a head) that share each tile of
//                    32 cached rows in shared memory; with `splits` > 1 the keys are shared out over grid z and a
//                    merge kernel folds the parts in key order
// Float32 arithmetic throughout; the cache and the outputs are in the compute dtype.
#include "common.cuh"

struct LaRotation {                 // as in rope_append.cu: angle p * inv_freq[j], or cos/sin from a table row
    const float* inv_freq;
    const float* table;
    int table_positions, interleaved, rotary_dim;
    float factor;                   // multiplies every cosine and sine (1: a plain rotation)
};

// Feature i of a vector x[0..n) at position pos after the rotation of its first rotary_dim features.
__device__ __forceinline__ float la_rotated(const float* x, int i, int pos, const LaRotation& r) {
    if (i >= r.rotary_dim || (r.inv_freq == nullptr && r.table == nullptr)) return x[i];
    const int half = r.rotary_dim >> 1;
    const int j = r.interleaved ? (i >> 1) : (i < half ? i : i - half);
    const bool first = r.interleaved ? !(i & 1) : i < half;
    const int other = r.interleaved ? (i ^ 1) : (i < half ? i + half : i - half);
    float s, c;
    if (r.table != nullptr) {
        c = r.table[(size_t)pos * r.rotary_dim + j];
        s = r.table[(size_t)pos * r.rotary_dim + half + j];
    } else {
        sincosf((float)pos * r.inv_freq[j], &s, &c);
    }
    c *= r.factor;
    s *= r.factor;
    return first ? x[i] * c - x[other] * s : x[i] * c + x[other] * s;
}

// ------------------------------------------------------------------ prepare
constexpr int LP_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(LP_THREADS) latent_prepare_kernel(
    T* __restrict__ q_latent, T* __restrict__ cache, const float* __restrict__ down, int ld,
    const float* __restrict__ q_w, const float* __restrict__ kv_w, float eps, int q_rank, int rank, int rot,
    LaRotation rotation, const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int page_size, int num_pages, int* __restrict__ status) {
    extern __shared__ float row[];
    __shared__ float red[33];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int width = q_rank + (cache ? rank + rot : 0);
    for (int i = tid; i < width; i += LP_THREADS) row[i] = down[(size_t)t * ld + i];
    __syncthreads();
    float ss = 0.f;
    if (q_rank > 0) {                                  // q_rank 0: the queries have no latent of their own
        for (int i = tid; i < q_rank; i += LP_THREADS) ss += row[i] * row[i];
        ss = block_sum(ss, red);
        const float inv_q = rsqrtf(ss / (float)q_rank + eps);
        for (int i = tid; i < q_rank; i += LP_THREADS)
            q_latent[(size_t)t * q_rank + i] = from_f32<T>(q_w[i] * row[i] * inv_q);
    }
    if (cache == nullptr) return;                      // a layer that reads another layer's cache
    const float* kv = row + q_rank;
    ss = 0.f;
    for (int i = tid; i < rank; i += LP_THREADS) ss += kv[i] * kv[i];
    ss = block_sum(ss, red);
    const float inv_kv = rsqrtf(ss / (float)rank + eps);
    const int pos = positions[t];
    const int logical = pos / page_size;
    const int page = logical < max_blocks ? block_table[(size_t)token_seq[t] * max_blocks + logical] : -1;
    if (page < 0 || page >= num_pages) {
        if (tid == 0 && status) atomicExch(status, 1);     // a token without a page: never write
        return;
    }
    if (rotation.table != nullptr && (pos < 0 || pos >= rotation.table_positions)) {
        if (tid == 0 && status) atomicExch(status, 4);
        return;
    }
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * (rank + rot);
    for (int i = tid; i < rank; i += LP_THREADS) dst[i] = from_f32<T>(kv_w[i] * kv[i] * inv_kv);
    for (int i = tid; i < rot; i += LP_THREADS) dst[rank + i] = from_f32<T>(la_rotated(kv + rank, i, pos, rotation));
}

TI_API int ti_latent_prepare(void* q_latent, void* cache, const float* down, int ld, const float* q_w, const float* kv_w,
                             float eps, int q_rank, int rank, int rot, const float* inv_freq, const float* table,
                             int table_positions, int interleaved, int rotary_dim, float rot_factor, const int* positions,
                             const int* token_seq, const int* block_table, int max_blocks, int num_tokens, int page_size,
                             int num_pages, int* status, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && q_rank >= 0 && rank > 0 && rot >= 0, "latent_prepare: bad sizes");
    TI_REQUIRE(q_rank == 0 || (q_latent && q_w), "latent_prepare: a query latent needs its output and its norm's weight");
    TI_REQUIRE(rotary_dim >= 0 && rotary_dim <= rot && rotary_dim % 2 == 0, "latent_prepare: rotary_dim %d does not fit %d rotated features", rotary_dim, rot);
    const int width = q_rank + rank + rot;
    TI_REQUIRE(width * 4 <= 48 * 1024, "latent_prepare: latents of %d features do not fit shared memory", width);
    if (num_tokens == 0) return 0;
    LaRotation r{inv_freq, table, table_positions, interleaved, rotary_dim, rot_factor};
    const size_t smem = (size_t)width * 4;
    if (dtype == TI_F32)
        ti_launch(latent_prepare_kernel<float>, num_tokens, LP_THREADS, smem, stream, (float*)q_latent, (float*)cache, down, ld,
                  q_w, kv_w, eps, q_rank, rank, rot, r, positions, token_seq, block_table, max_blocks, page_size, num_pages, status);
    else if (dtype == TI_BF16)
        ti_launch(latent_prepare_kernel<__nv_bfloat16>, num_tokens, LP_THREADS, smem, stream, (__nv_bfloat16*)q_latent,
                  (__nv_bfloat16*)cache, down, ld, q_w, kv_w, eps, q_rank, rank, rot, r, positions, token_seq, block_table,
                  max_blocks, page_size, num_pages, status);
    else TI_REQUIRE(false, "latent_prepare: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("latent_prepare");
    return 0;
}

// ------------------------------------------------------------------ query rotation
// q [T, H, plain + rot] (rows of ld_q elements) in the compute dtype -> rows[t][h][rank .. rank + rot) float32 (the first `rank` features
// of a row are written by the batched product with the key maps).
template <typename T>
__global__ void latent_query_kernel(float* __restrict__ rows, const T* __restrict__ q, int ld_q, int heads, int plain, int rot, int rank,
                                    LaRotation rotation, const int* __restrict__ positions) {
    extern __shared__ float part[];
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int n = heads * rot;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int h = i / rot, f = i % rot;
        part[i] = to_f32(q[(size_t)t * ld_q + (size_t)h * (plain + rot) + plain + f]);
    }
    __syncthreads();
    const bool in_table = rotation.table == nullptr || (pos >= 0 && pos < rotation.table_positions);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int h = i / rot, f = i % rot;
        rows[((size_t)t * heads + h) * (rank + rot) + rank + f] = in_table ? la_rotated(part + h * rot, f, pos, rotation) : 0.f;
    }
}

TI_API int ti_latent_query(float* rows, const void* q, int ld_q, int num_tokens, int heads, int plain, int rot, int rank,
                           const float* inv_freq, const float* table, int table_positions, int interleaved, int rotary_dim,
                           float rot_factor, const int* positions, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && heads > 0 && plain >= 0 && rot >= 0 && rank > 0 && ld_q >= heads * (plain + rot), "latent_query: bad sizes");
    TI_REQUIRE(rotary_dim >= 0 && rotary_dim <= rot && rotary_dim % 2 == 0, "latent_query: rotary_dim %d does not fit %d rotated features", rotary_dim, rot);
    TI_REQUIRE(heads * rot * 4 <= 48 * 1024, "latent_query: %d rotated features do not fit shared memory", heads * rot);
    if (num_tokens == 0 || rot == 0) return 0;
    LaRotation r{inv_freq, table, table_positions, interleaved, rotary_dim, rot_factor};
    const size_t smem = (size_t)heads * rot * 4;
    if (dtype == TI_F32)
        ti_launch(latent_query_kernel<float>, num_tokens, 128, smem, stream, rows, (const float*)q, ld_q, heads, plain, rot, rank, r, positions);
    else if (dtype == TI_BF16)
        ti_launch(latent_query_kernel<__nv_bfloat16>, num_tokens, 128, smem, stream, rows, (const __nv_bfloat16*)q, ld_q, heads, plain, rot, rank, r, positions);
    else TI_REQUIRE(false, "latent_query: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("latent_query");
    return 0;
}

// ------------------------------------------------------------------ attention
constexpr int LA_WARPS = 8;
constexpr int LA_KEYS = 32;

// NV: value features a lane accumulates (rank <= 32 * NV).
template <typename T, int NV>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attend_kernel(
    T* __restrict__ out, float* __restrict__ parts, const float* __restrict__ q, const T* __restrict__ cache,
    const float* __restrict__ sink, const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int heads, int rank, int rot, int page_size, int num_pages,
    float scale, int window, int splits, int* __restrict__ status) {
    extern __shared__ float smem[];
    const int dk = rank + rot;
    const int kstride = dk + 1;                         // a lane a key: rows one word apart in the banks
    float* keys = smem;                                 // [LA_KEYS][kstride]
    float* qs = smem + LA_KEYS * kstride;               // [LA_WARPS][dk]
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    const int h = blockIdx.x * LA_WARPS + warp;
    const bool live = h < heads;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    int first = lo, last = pos + 1;                     // this block's keys [first, last)
    if (splits > 1) {
        const int n = pos + 1 - lo;
        const int per = ((n + splits - 1) / splits + LA_KEYS - 1) / LA_KEYS * LA_KEYS;
        first = lo + blockIdx.z * per;
        last = min(pos + 1, first + per);
    }
    const int* table = block_table + (size_t)token_seq[t] * max_blocks;
    if (live) {
        const float* qrow = q + ((size_t)t * heads + h) * dk;
        for (int i = lane; i < dk; i += 32) qs[warp * dk + i] = qrow[i];
    }
    float acc[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[v] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int j0 = first; j0 < last; j0 += LA_KEYS) {
        __syncthreads();                                // the tile before is read; qs is written
        const int n = min(LA_KEYS, last - j0);
        for (int j = warp; j < n; j += LA_WARPS) {      // a warp a cached row
            const int key = j0 + j;
            const int logical = key / page_size;
            const int page = logical < max_blocks ? table[logical] : -1;
            if (page >= 0 && page < num_pages) {
                const T* src = cache + ((size_t)page * page_size + key % page_size) * dk;
                for (int i = lane; i < dk; i += 32) keys[j * kstride + i] = to_f32(src[i]);
            } else {
                if (lane == 0 && status) atomicExch(status, 2);     // a visible key without a page
                for (int i = lane; i < dk; i += 32) keys[j * kstride + i] = 0.f;
            }
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < n) {
            const float* k = keys + lane * kstride;
            const float* qh = qs + warp * dk;
            float dot = 0.f;
            for (int i = 0; i < dk; ++i) dot = fmaf(qh[i], k[i], dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (lane < n) ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] *= corr;
        for (int j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const float* k = keys + j * kstride;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const int i = lane + 32 * v;
                if (i < rank) acc[v] = fmaf(pj, k[i], acc[v]);
            }
        }
    }
    if (!live) return;
    if (splits > 1) {                                   // unnormalised part: [m, l, acc[rank]]
        float* dst = parts + (((size_t)t * heads + h) * splits + blockIdx.z) * (rank + 2);
        if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int i = lane + 32 * v;
            if (i < rank) dst[2 + i] = acc[v];
        }
        return;
    }
    if (sink != nullptr) {                              // one more term of the denominator, without a value
        const float sk = sink[h];
        const float m_new = fmaxf(m, sk);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] *= corr;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* dst = out + ((size_t)t * heads + h) * rank;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = lane + 32 * v;
        if (i < rank) dst[i] = from_f32<T>(acc[v] * inv);
    }
}

// One block per (token, head): folds the parts in key order, then the sink. The parts' weights exp(m_z - m) are
// worked out once into shared memory; the features are then one pass of independent loads.
constexpr int LM_MAX_SPLITS = 64;

template <typename T>
__global__ void latent_merge_kernel(T* __restrict__ out, const float* __restrict__ parts, const float* __restrict__ sink,
                                    int heads, int rank, int splits) {
    __shared__ float wz[LM_MAX_SPLITS];
    __shared__ float inv_l;
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int h = blockIdx.x, t = blockIdx.y;
    const float* src = parts + ((size_t)t * heads + h) * splits * (rank + 2);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float mz[LM_MAX_SPLITS / 32], lz[LM_MAX_SPLITS / 32];
        float m = sink ? sink[h] : -INFINITY;
#pragma unroll
        for (int k = 0; k < LM_MAX_SPLITS / 32; ++k) {
            const int z = lane + 32 * k;
            mz[k] = z < splits ? src[(size_t)z * (rank + 2)] : -INFINITY;
            lz[k] = z < splits ? src[(size_t)z * (rank + 2) + 1] : 0.f;
            m = fmaxf(m, mz[k]);
        }
        m = warp_max(m);
        float l = 0.f;
#pragma unroll
        for (int k = 0; k < LM_MAX_SPLITS / 32; ++k) {
            const int z = lane + 32 * k;
            const float w = (mz[k] == -INFINITY) ? 0.f : expf(mz[k] - m);
            if (z < splits) wz[z] = w;
            l += lz[k] * w;
        }
        l = warp_sum(l);
        if (sink) l += expf(sink[h] - m);
        if (lane == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
    }
    __syncthreads();
    const float inv = inv_l;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        float a = 0.f;
#pragma unroll 8
        for (int z = 0; z < splits; ++z) a = fmaf(src[(size_t)z * (rank + 2) + 2 + i], wz[z], a);
        out[((size_t)t * heads + h) * rank + i] = from_f32<T>(a * inv);
    }
}

// Folds `splits` parts per (token, head) (as the attention kernels leave them) into out [T, heads, rank].
TI_API int ti_latent_merge(void* out, const float* parts, const float* sink, int num_tokens, int heads, int rank, int splits,
                           int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && heads > 0 && rank > 0 && splits >= 1 && splits <= LM_MAX_SPLITS && num_tokens <= 65535,
               "latent_merge: bad sizes (at most %d splits)", LM_MAX_SPLITS);
    if (num_tokens == 0) return 0;
    dim3 mgrid(heads, num_tokens);
    const int threads = rank >= 512 ? 512 : (rank + 31) / 32 * 32;       // a feature a thread
    if (dtype == TI_F32)
        ti_launch(latent_merge_kernel<float>, mgrid, threads, 0, stream, (float*)out, parts, sink, heads, rank, splits);
    else if (dtype == TI_BF16)
        ti_launch(latent_merge_kernel<__nv_bfloat16>, mgrid, threads, 0, stream, (__nv_bfloat16*)out, parts, sink, heads, rank, splits);
    else TI_REQUIRE(false, "latent_merge: unknown dtype %d", dtype);
    TI_CHECK_LAUNCH("latent_merge");
    return 0;
}

template <typename T, int NV>
static cudaError_t la_launch(dim3 grid, size_t smem, cudaStream_t stream, void* out, float* parts, const float* q,
                             const void* cache, const float* sink, const int* positions, const int* token_seq,
                             const int* block_table, int max_blocks, int heads, int rank, int rot, int page_size,
                             int num_pages, float scale, int window, int splits, int* status) {
    auto kernel = latent_attend_kernel<T, NV>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return ti_launch(kernel, grid, LA_WARPS * 32, smem, stream, (T*)out, parts, q, (const T*)cache, sink, positions,
                     token_seq, block_table, max_blocks, heads, rank, rot, page_size, num_pages, scale, window, splits, status);
}

// out [T, heads, rank] (compute dtype); q float32 [T, heads, rank + rot]; cache [pages, page_size, rank + rot];
// parts: float32 scratch of at least T * heads * splits * (rank + 2) floats when splits > 1.
TI_API int ti_latent_attend(void* out, float* parts, long long parts_floats, const float* q, const void* cache,
                            const float* sink, const int* positions, const int* token_seq, const int* block_table,
                            int max_blocks, int num_tokens, int heads, int rank, int rot, int page_size, int num_pages,
                            float scale, int window, int splits, int* status, int dtype, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && heads > 0 && rank > 0 && rot >= 0 && page_size > 0 && window >= 0, "latent_attend: bad sizes");
    TI_REQUIRE(rank <= 512, "latent_attend: a latent of %d features is more than the kernel's 512", rank);
    TI_REQUIRE(num_tokens <= 65535 && splits >= 1 && splits <= LM_MAX_SPLITS, "latent_attend: too many tokens or splits");
    TI_REQUIRE(splits == 1 || (parts != nullptr && parts_floats >= (long long)num_tokens * heads * splits * (rank + 2)),
               "latent_attend: scratch too small for %d splits", splits);
    if (num_tokens == 0) return 0;
    const int dk = rank + rot;
    const size_t smem = ((size_t)LA_KEYS * (dk + 1) + (size_t)LA_WARPS * dk) * 4;
    TI_REQUIRE(smem <= 200 * 1024, "latent_attend: rows of %d features do not fit shared memory", dk);
    dim3 grid((heads + LA_WARPS - 1) / LA_WARPS, num_tokens, splits);
    cudaError_t e;
#define LA_GO(T, NV) e = la_launch<T, NV>(grid, smem, stream, out, parts, q, cache, sink, positions, token_seq, block_table, \
                                          max_blocks, heads, rank, rot, page_size, num_pages, scale, window, splits, status)
    if (dtype == TI_F32) {
        if (rank <= 128) LA_GO(float, 4); else if (rank <= 256) LA_GO(float, 8); else LA_GO(float, 16);
    } else if (dtype == TI_BF16) {
        if (rank <= 128) LA_GO(__nv_bfloat16, 4); else if (rank <= 256) LA_GO(__nv_bfloat16, 8); else LA_GO(__nv_bfloat16, 16);
    } else TI_REQUIRE(false, "latent_attend: unknown dtype %d", dtype);
#undef LA_GO
    TI_REQUIRE(e == cudaSuccess, "latent_attend: %s", cudaGetErrorString(e));
    TI_CHECK_LAUNCH("latent_attend");
    if (splits > 1) return ti_latent_merge(out, parts, sink, num_tokens, heads, rank, splits, dtype, stream);
    return 0;
}
