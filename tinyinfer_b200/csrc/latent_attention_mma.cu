// The attention over a cached latent (see latent_attention.cu for the mechanism) on the warp-level tensor cores,
// bfloat16: the prompt-portion and the decode form of the same kernel.
//
// The rows of a block's query tile are (token, head) pairs: every head of a token reads the same cached rows
// [c | k_rot], so the heads fill the 16-row tiles of mma.sync that a single token's head could not. A block of
// 4 MW warps holds 16 MW rows: MW = 2 for prompt portions (with 16 heads: two consecutive tokens of one request),
// MW = 1 for decoded tokens (one token's heads; the keys may be shared out over grid z, the parts folded by the
// merge kernel of latent_attention.cu). Warp (mw, nw) owns rows [16 mw, +16) and, of the value features, the
// quarter nw. Per tile of 32 cached rows (fetched with cp.async):
//   S  = Q K^T : each warp takes a quarter of the feature range for all 32 keys (its A fragments stay the same for
//                every tile, its B fragments come with ldmatrix from the key tile) and leaves a partial sum in shared
//                memory; after a barrier every warp adds the four partials of its rows,
//   softmax    : float32, running maximum per row, computed alike by the four warps of a row group,
//   O += P V   : P as bfloat16 A fragments from registers, V = the first `rank` features of the same key tile,
//                read with ldmatrix.trans; a warp accumulates 16 rows x its quarter of the features.
// Features beyond the row length are zero in shared memory (the row length is padded to a multiple of 64, and to
// the value features the four warps cover).
#include "common.cuh"
#include "mma_tile.cuh"

namespace lm {
constexpr int KEYS = 32;
constexpr int SPAD = 36;                       // floats per row of a partial score tile

__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const __nv_bfloat16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

struct Args {
    __nv_bfloat16* out;
    float* parts;
    const float* q;
    const __nv_bfloat16* cache;
    const float* sink;
    const int *positions, *token_seq, *cu_seqlens, *block_table;
    int max_blocks, num_seqs, num_tokens, heads, rank, rot, page_size, num_pages;
    float scale;
    int window;                    // 0: every key up to the query's own; n: the last n (itself included)
    int splits, tpb, hpb, dkp;
    int* status;
};

// NT: 8-column tiles of the value features a warp accumulates (the padded rank is 32 NT). KBUF: key-tile buffers
// (2: the next tile is fetched while this one is worked on; 1: two blocks share an SM instead, and one block's
// products run while the other waits for its tile or is in its softmax). PER_SM: blocks meant to share an SM.
template <int MW, int NT, int KBUF, int PER_SM>
__global__ void __launch_bounds__(128 * MW, PER_SM) latent_attend_mma_kernel(Args a) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int dk = a.rank + a.rot;
    const int dkp = a.dkp;                                    // dk padded: a multiple of 64, at least 32 NT
    const int lds = dkp + 8;                                  // halves per row: ldmatrix without bank conflicts
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(raw);                    // [16 MW][lds]
    __nv_bfloat16* Ks = Qs + 16 * MW * lds;                                       // [KBUF][KEYS][lds]
    float* Ss = reinterpret_cast<float*>(Ks + KBUF * KEYS * lds);                    // [MW][4][16][SPAD]
    int* row_tok = reinterpret_cast<int*>(Ss + MW * 4 * 16 * SPAD);               // [16 MW] flat token or -1
    int* row_pos = row_tok + 16 * MW;
    int* row_head = row_pos + 16 * MW;
    __shared__ int blk[3];                                    // request, first flat token, tokens
    ti_grid_launch_dependents();
    ti_grid_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mw = warp >> 2, nw = warp & 3;
    const int g = lane >> 2, t4 = lane & 3;
    constexpr int ROWS = 16 * MW, THREADS = 128 * MW;

    // which tokens this block holds: blocks are dealt request by request, tpb tokens each
    if (tid == 0) {
        int seq = -1, first = 0, n = 0;
        if (a.tpb == 1) {
            if ((int)blockIdx.x < a.num_tokens) { first = blockIdx.x; n = 1; seq = a.token_seq[first]; }
        } else {
            int at = 0;
            for (int s = 0; s < a.num_seqs; ++s) {
                const int r0 = a.cu_seqlens[s], len = a.cu_seqlens[s + 1] - r0;
                const int nb = (len + a.tpb - 1) / a.tpb;
                if ((int)blockIdx.x < at + nb) {
                    seq = s;
                    first = r0 + ((int)blockIdx.x - at) * a.tpb;
                    n = min(a.tpb, r0 + len - first);
                    break;
                }
                at += nb;
            }
        }
        blk[0] = seq; blk[1] = first; blk[2] = n;
    }
    __syncthreads();
    const int seq = blk[0], tok0 = blk[1], ntok = blk[2];
    if (seq < 0) return;
    const int h0 = blockIdx.y * a.hpb;
    if (tid < ROWS) {
        const int tl = tid / a.hpb, hl = tid % a.hpb;
        const bool ok = tl < ntok && h0 + hl < a.heads;
        row_tok[tid] = ok ? tok0 + tl : -1;
        row_pos[tid] = ok ? a.positions[tok0 + tl] : -1;
        row_head[tid] = h0 + hl;
    }
    __syncthreads();
    // the query rows, rounded to bfloat16 (dk is a multiple of 8: four features a load)
    {
        const int quads = dkp / 4;
#pragma unroll 4
        for (int i = tid; i < ROWS * quads; i += THREADS) {
            const int r = i / quads, c = (i % quads) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_tok[r] >= 0 && c < dk)
                v = *reinterpret_cast<const float4*>(a.q + ((size_t)row_tok[r] * a.heads + row_head[r]) * dk + c);
            *reinterpret_cast<uint2*>(Qs + r * lds + c) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
        }
    }
    const int hi = a.positions[tok0 + ntok - 1];              // the block's last token sees the most keys,
    const int lo = a.window > 0 ? max(0, a.positions[tok0] - a.window + 1) : 0;      // its first the oldest
    int first_key = lo, last_key = hi + 1;
    if (a.splits > 1) {
        const int per = ((hi + 1 - lo + a.splits - 1) / a.splits + KEYS - 1) / KEYS * KEYS;
        first_key = lo + blockIdx.z * per;
        last_key = min(hi + 1, first_key + per);
    }
    const int* table = a.block_table + (size_t)seq * a.max_blocks;
    const int chunks = dkp / 8;                                // 16-byte pieces of a row in shared memory
    const int real_chunks = dk / 8;
    // a warp fetches whole rows, their 16-byte pieces a lane apiece; where a row lies is worked out once a tile,
    // lane l for key j0 + l (one division and one look-up in the block table a lane), and handed round by shuffle
    auto load_tile = [&](int j0, int buf) {
        __nv_bfloat16* dst = Ks + buf * KEYS * lds;
        constexpr int PER_WARP = KEYS / (4 * MW);
        const __nv_bfloat16* mine = nullptr;
        {
            const int key = j0 + lane;
            if (key < last_key) {
                const int logical = key / a.page_size;
                const int page = logical < a.max_blocks ? table[logical] : -1;
                if (page >= 0 && page < a.num_pages) mine = a.cache + ((size_t)page * a.page_size + (key - logical * a.page_size)) * dk;
                else if (a.status) atomicExch(a.status, 2);      // a visible key without a page
            }
        }
#pragma unroll
        for (int i = 0; i < PER_WARP; ++i) {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(
                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine), warp * PER_WARP + i));
            __nv_bfloat16* row = dst + (warp * PER_WARP + i) * lds;
            for (int c = lane; c < chunks; c += 32) {
                const bool ok = src != nullptr && c < real_chunks;
                mt::cp16(row + c * 8, ok ? src + c * 8 : a.cache, ok);
            }
        }
    };
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int pos_a = row_pos[mw * 16 + g], pos_b = row_pos[mw * 16 + g + 8];
    // a row sees the keys (old, pos]: old = pos - window, or before the first key without a window
    const int old_a = a.window > 0 ? pos_a - a.window : -1, old_b = a.window > 0 ? pos_b - a.window : -1;
    const int ksteps = dkp / 64;                               // k steps of 16 in this warp's quarter of the features
    const __nv_bfloat16* q_base = Qs + (mw * 16 + (lane & 15)) * lds + nw * (dkp / 4) + (lane >> 4) * 8;
    float* s_mine = Ss + ((mw * 4 + nw) * 16) * SPAD;
    const float* s_all = Ss + (mw * 4 * 16) * SPAD;

    if (KBUF == 2) {
        if (first_key < last_key) load_tile(first_key, 0);
        mt::commit();
    }
    int buf = 0;
    for (int j0 = first_key; j0 < last_key; j0 += KEYS, buf ^= (KBUF - 1)) {
        if (KBUF == 2) {
            if (j0 + KEYS < last_key) load_tile(j0 + KEYS, buf ^ 1);
            mt::commit();
            mt::wait_group<1>();
        } else {
            load_tile(j0, 0);
            mt::commit();
            mt::wait_group<0>();
        }
        __syncthreads();                                       // the tile (and, the first time, Qs) is in shared memory
        const __nv_bfloat16* kt = Ks + buf * KEYS * lds;
        // ---- partial scores: 16 rows x 32 keys over this warp's quarter of the features
        float s[4][4];
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[ni][e] = 0.f;
        const __nv_bfloat16* k_base = kt + ((lane & 7) + ((lane >> 4) << 3)) * lds + nw * (dkp / 4) + ((lane >> 3) & 1) * 8;
#pragma unroll 3
        for (int ks = 0; ks < ksteps; ++ks) {
            unsigned af[4], bf[2][4];
            mt::ldmatrix_x4(af, q_base + ks * 16);
            mt::ldmatrix_x4(bf[0], k_base + ks * 16);
            mt::ldmatrix_x4(bf[1], k_base + 16 * lds + ks * 16);
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) mt::mma16816(s[ni], af, bf[ni >> 1][(ni & 1) * 2], bf[ni >> 1][(ni & 1) * 2 + 1]);
        }
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
            *reinterpret_cast<float2*>(s_mine + g * SPAD + ni * 8 + t4 * 2) = make_float2(s[ni][0], s[ni][1]);
            *reinterpret_cast<float2*>(s_mine + (g + 8) * SPAD + ni * 8 + t4 * 2) = make_float2(s[ni][2], s[ni][3]);
        }
        __syncthreads();
        // ---- the rows' scores: the four partials added, scaled, masked
        float p[4][4];                                         // [key tile of 8][row g: 0,1 | row g+8: 2,3]
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
            float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 xa = *reinterpret_cast<const float2*>(s_all + (w * 16 + g) * SPAD + ni * 8 + t4 * 2);
                const float2 xb = *reinterpret_cast<const float2*>(s_all + (w * 16 + g + 8) * SPAD + ni * 8 + t4 * 2);
                ra.x += xa.x; ra.y += xa.y; rb.x += xb.x; rb.y += xb.y;
            }
            const int key = j0 + ni * 8 + t4 * 2;
            p[ni][0] = (key < last_key && key <= pos_a && key > old_a) ? ra.x * a.scale : -INFINITY;
            p[ni][1] = (key + 1 < last_key && key + 1 <= pos_a && key + 1 > old_a) ? ra.y * a.scale : -INFINITY;
            p[ni][2] = (key < last_key && key <= pos_b && key > old_b) ? rb.x * a.scale : -INFINITY;
            p[ni][3] = (key + 1 < last_key && key + 1 <= pos_b && key + 1 > old_b) ? rb.y * a.scale : -INFINITY;
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) mx = fmaxf(mx, fmaxf(p[ni][2 * r], p[ni][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[r], mx);
            corr[r] = (m_new == -INFINITY || m_run[r] == -INFINITY) ? (m_run[r] == -INFINITY ? 0.f : 1.f) : expf(m_run[r] - m_new);
            float sum = 0.f;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                p[ni][2 * r] = (m_new == -INFINITY) ? 0.f : expf(p[ni][2 * r] - m_new);
                p[ni][2 * r + 1] = (m_new == -INFINITY) ? 0.f : expf(p[ni][2 * r + 1] - m_new);
                sum += p[ni][2 * r] + p[ni][2 * r + 1];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run[r] = l_run[r] * corr[r] + sum;
            m_run[r] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
            o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
        }
        // ---- O += P V over the two halves of the tile's keys
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
            unsigned pf[4];
            pf[0] = pack_bf16(p[2 * kh][0], p[2 * kh][1]);
            pf[1] = pack_bf16(p[2 * kh][2], p[2 * kh][3]);
            pf[2] = pack_bf16(p[2 * kh + 1][0], p[2 * kh + 1][1]);
            pf[3] = pack_bf16(p[2 * kh + 1][2], p[2 * kh + 1][3]);
            const __nv_bfloat16* v_base = kt + (kh * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * lds + nw * (NT * 8) + (lane >> 4) * 8;
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                unsigned vf[4];
                ldmatrix_x4_trans(vf, v_base + np * 16);
                mt::mma16816(o[2 * np], pf, vf[0], vf[1]);
                mt::mma16816(o[2 * np + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();                                       // the tile and the partial scores may be overwritten
    }
    mt::wait_group<0>();
    // ---- results: rows g and g + 8 of this warp's row group, its quarter of the features
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = mw * 16 + g + 8 * r;
        const int tok = row_tok[row];
        if (tok < 0) continue;
        const int h = row_head[row];
        float m = m_run[r], l = l_run[r], c = 1.f;
        if (a.splits > 1) {
            float* dst = a.parts + (((size_t)tok * a.heads + h) * a.splits + blockIdx.z) * (a.rank + 2);
            if (nw == 0 && t4 == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int col = nw * (NT * 8) + nt * 8 + t4 * 2;
                if (col < a.rank) dst[2 + col] = o[nt][2 * r];
                if (col + 1 < a.rank) dst[2 + col + 1] = o[nt][2 * r + 1];
            }
            continue;
        }
        if (a.sink != nullptr) {
            const float sk = a.sink[h];
            const float m_new = fmaxf(m, sk);
            c = (m == -INFINITY) ? 0.f : expf(m - m_new);
            l = l * c + expf(sk - m_new);
        }
        const float inv = l > 0.f ? c / l : 0.f;
        __nv_bfloat16* dst = a.out + ((size_t)tok * a.heads + h) * a.rank;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int col = nw * (NT * 8) + nt * 8 + t4 * 2;
            if (col < a.rank) dst[col] = __float2bfloat16_rn(o[nt][2 * r] * inv);
            if (col + 1 < a.rank) dst[col + 1] = __float2bfloat16_rn(o[nt][2 * r + 1] * inv);
        }
    }
}

template <int MW, int NT, int KBUF, int PER_SM>
static cudaError_t launch(const Args& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kernel = latent_attend_mma_kernel<MW, NT, KBUF, PER_SM>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return ti_launch(kernel, grid, 128 * MW, smem, stream, a);
}
}  // namespace lm

// 1 if the tensor-core form takes these sizes (the caller then need not try): rows of a multiple of 8 features.
TI_API int ti_latent_attend_mma_ok(int rank, int rot) { return (rank + rot) % 8 == 0 && rank <= 512 && rank > 0 ? 1 : 0; }

// decode != 0: every token is a block of its own (its heads are the rows); else blocks of 32 rows are dealt to the
// requests' consecutive tokens, two blocks an SM. q float32 [T, heads, rank + rot]; out bfloat16 [T, heads, rank].
TI_API int ti_latent_attend_mma(void* out, float* parts, long long parts_floats, const float* q, const void* cache,
                                const float* sink, const int* positions, const int* token_seq, const int* cu_seqlens,
                                const int* block_table, int max_blocks, int num_seqs, int num_tokens, int heads, int rank,
                                int rot, int page_size, int num_pages, float scale, int window, int splits, int decode,
                                int* status, cudaStream_t stream) {
    TI_REQUIRE(num_tokens >= 0 && heads > 0 && rank > 0 && rot >= 0 && page_size > 0 && num_seqs > 0 && window >= 0, "latent_attend_mma: bad sizes");
    TI_REQUIRE(ti_latent_attend_mma_ok(rank, rot), "latent_attend_mma: rows of %d + %d features are not taken", rank, rot);
    TI_REQUIRE(splits >= 1 && splits <= 65535, "latent_attend_mma: bad number of splits");
    TI_REQUIRE(splits == 1 || (parts != nullptr && parts_floats >= (long long)num_tokens * heads * splits * (rank + 2)),
               "latent_attend_mma: scratch too small for %d splits", splits);
    if (num_tokens == 0) return 0;
    const int mw = decode ? 1 : 2, kbuf = decode ? 2 : 1;
    const int rows = 16 * mw;
    lm::Args a;
    a.out = (__nv_bfloat16*)out; a.parts = parts; a.q = q; a.cache = (const __nv_bfloat16*)cache; a.sink = sink;
    a.positions = positions; a.token_seq = token_seq; a.cu_seqlens = cu_seqlens; a.block_table = block_table;
    a.max_blocks = max_blocks; a.num_seqs = num_seqs; a.num_tokens = num_tokens; a.heads = heads; a.rank = rank; a.rot = rot;
    a.page_size = page_size; a.num_pages = num_pages; a.scale = scale; a.window = window; a.splits = splits; a.status = status;
    a.hpb = heads < rows ? heads : rows;
    a.tpb = decode ? 1 : (rows / a.hpb > 0 ? rows / a.hpb : 1);
    const int nt = rank <= 128 ? 4 : (rank <= 256 ? 8 : 16);
    const int dkp = ((rank + rot + 63) / 64 * 64) > 32 * nt ? ((rank + rot + 63) / 64 * 64) : 32 * nt, lds = dkp + 8;
    a.dkp = dkp;
    const size_t smem = (size_t)(rows + kbuf * lm::KEYS) * lds * 2 + (size_t)mw * 4 * 16 * lm::SPAD * 4 + (size_t)3 * rows * 4;
    TI_REQUIRE(smem <= 220 * 1024, "latent_attend_mma: rows of %d features do not fit shared memory", rank + rot);
    const int blocks = a.tpb == 1 ? num_tokens : (num_tokens + a.tpb - 1) / a.tpb + num_seqs;
    dim3 grid(blocks, (heads + a.hpb - 1) / a.hpb, splits);
    TI_REQUIRE(grid.y <= 65535, "latent_attend_mma: too many heads");
    cudaError_t e;
    if (decode) e = nt == 4 ? lm::launch<1, 4, 2, 2>(a, grid, smem, stream) : nt == 8 ? lm::launch<1, 8, 2, 2>(a, grid, smem, stream) : lm::launch<1, 16, 2, 2>(a, grid, smem, stream);
    else e = nt == 4 ? lm::launch<2, 4, 1, 2>(a, grid, smem, stream) : nt == 8 ? lm::launch<2, 8, 1, 2>(a, grid, smem, stream) : lm::launch<2, 16, 1, 2>(a, grid, smem, stream);
    TI_REQUIRE(e == cudaSuccess, "latent_attend_mma: %s", cudaGetErrorString(e));
    TI_CHECK_LAUNCH("latent_attend_mma");
    return 0;
}
