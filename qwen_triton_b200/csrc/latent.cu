// Attention through a latent: what stands around the attention kernel of a mixer that caches, per token, one normed
// latent vector c and one rotated key part shared by all heads, and expands keys and values from c per head.
//
// The cache row of a token is [c (rank) | rotated part (rot)], one "kv head" of size rank + rot.  With
// k_h = W_uk_h c and v_h = W_uv_h c the score of head h is q_plain_h . (W_uk_h c) + q_rot_h . k_rot
// = (W_uk_h^T q_plain_h) . c + q_rot_h . k_rot, so the attention kernel runs every head's query
// [W_uk_h^T q_plain_h | q_rot_h] against the cached rows as they are (all heads share the one kv head), its values are
// the first `rank` elements of the same rows, and the head's output is W_uv_h (sum_j p_j c_j).
//
// latent_prepare_kernel   from the first projection's float sums of a token: RMS norm (weight, eps inside the root) of the
//                         query latent -> cq_out; RMS norm of the key/value latent and rotation of the shared key part
//                         by the token's position -> the cache row.
// latent_query_rot_kernel the rotated part of every head's query: rotation by position into the query rows.
// head_product_kernel     Y[t, h, n] = sum_k X[t, h, k] W[h, n, k] for every head with its own matrix (float sums), with
//                         strides for X and Y and optionally times sigmoid(gate[t, h * N + n]).
// head_product_mma_kernel the same on the tensor cores (mma.sync m16n8k16) for bfloat16 matrices and results.
// Rotation: element i of the rotated part turns with element i + rd / 2 by the angle whose cos and sin the table row
// of the position holds (cos | sin, rd columns); elements beyond the first rd pass unchanged.
#include "attention_mma.cuh"

#include <math.h>

using namespace qt;

__device__ __forceinline__ float sum_splits(const float* __restrict__ base, size_t index, int n_splits, size_t split_stride) {
    float acc = base[index];
    for (int s = 1; s < n_splits; ++s) acc += base[index + (size_t)s * split_stride];
    return acc;
}

struct PrepareParams {
    const float* proj; int n_splits; size_t split_stride; int proj_cols;   // columns: query latent | key/value latent | rotated part | ...
    const float* q_norm; const float* kv_norm; float eps;
    const float* cos_sin; int rotary_dim, max_pos;
    void* cq_out;                     // [T, q_rank]
    void* cache;                      // [pages, 1, page_tokens, rank + rot]
    const int* token_seq; const int* token_pos; const int* block_table; int max_blocks;
    int q_rank, rank, rot, page_tokens, ring_tokens, write_kv;
};

// one block per token
template <typename TO>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const PrepareParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const size_t base = (size_t)t * p.proj_cols;
    {
        float sq = 0.f;
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) {
            const float x = sum_splits(p.proj, base + i, p.n_splits, p.split_stride);
            sq += x * x;
        }
        const float inv = rsqrtf(block_sum(sq, scratch) / (float)p.q_rank + p.eps);
        TO* out = (TO*)p.cq_out + (size_t)t * p.q_rank;
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x)
            out[i] = from_float<TO>(sum_splits(p.proj, base + i, p.n_splits, p.split_stride) * inv * p.q_norm[i]);
    }
    if (!p.write_kv) return;
    const int pos = p.token_pos[t];
    const int* table = p.block_table + (size_t)p.token_seq[t] * p.max_blocks;
    TO* row = (TO*)p.cache + cache_offset(table, pos, p.ring_tokens, p.page_tokens, 1, 0, p.rank + p.rot);
    const size_t at = base + p.q_rank;
    float sq = 0.f;
    for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
        const float x = sum_splits(p.proj, at + i, p.n_splits, p.split_stride);
        sq += x * x;
    }
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)p.rank + p.eps);
    for (int i = threadIdx.x; i < p.rank; i += blockDim.x)
        row[i] = from_float<TO>(sum_splits(p.proj, at + i, p.n_splits, p.split_stride) * inv * p.kv_norm[i]);
    const int half = p.rotary_dim / 2;
    const float* cs = p.cos_sin ? p.cos_sin + (size_t)pos * p.rotary_dim : nullptr;
    for (int i = threadIdx.x; i < p.rot; i += blockDim.x) {
        const float x = sum_splits(p.proj, at + p.rank + i, p.n_splits, p.split_stride);
        float y = x;
        if (cs && i < p.rotary_dim) {
            const int pair = i < half ? i : i - half;
            const float other = sum_splits(p.proj, at + p.rank + (i < half ? i + half : i - half), p.n_splits, p.split_stride);
            y = i < half ? x * cs[pair] - other * cs[half + pair] : x * cs[pair] + other * cs[half + pair];
        }
        row[p.rank + i] = from_float<TO>(y);
    }
}

extern "C" int qt_latent_prepare(const float* proj, int n_splits, long long split_stride, int proj_cols, const float* q_norm,
                                 const float* kv_norm, float eps, const float* cos_sin, int rotary_dim, int max_pos, void* cq_out,
                                 void* cache, int out_dtype, const int* token_seq, const int* token_pos, const int* block_table,
                                 int max_blocks, int n_tokens, int q_rank, int rank, int rot, int page_tokens, int ring_tokens,
                                 int write_kv, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && q_rank > 0 && rank > 0 && rot >= 0 && n_splits >= 1 && eps > 0.f, "latent_prepare: bad sizes");
    QT_REQUIRE(q_rank + (write_kv ? rank + rot : 0) <= proj_cols, "latent_prepare: the latents need %d columns of %d",
               q_rank + (write_kv ? rank + rot : 0), proj_cols);
    QT_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= rot && (rotary_dim == 0 || cos_sin),
               "latent_prepare: %d of %d elements rotate", rotary_dim, rot);
    QT_REQUIRE(!write_kv || (cache && block_table && kv_norm), "latent_prepare: no cache to write to");
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    PrepareParams p{proj, n_splits, (size_t)split_stride, proj_cols, q_norm, kv_norm, eps, rotary_dim ? cos_sin : nullptr, rotary_dim, max_pos,
                    cq_out, cache, token_seq, token_pos, block_table, max_blocks, q_rank, rank, rot, page_tokens, ring_tokens, write_kv};
    return QT_DISPATCH_DTYPE(out_dtype, "latent_prepare", {
        launch_kernel(latent_prepare_kernel<T>, dim3(n_tokens), dim3(256), 0, s, p);
        QT_CHECK_LAUNCH("latent_prepare");
        return QT_OK;
    });
}

// ----------------------------------------------------------------------------- the rotated part of the queries
// q [splits, T, heads * (dim + rot)] -> out[t, h, out_offset + i] for i < rot.  One thread per (token, head, element).
template <typename TI, typename TO>
__global__ void latent_query_rot_kernel(const TI* __restrict__ q, int n_splits, size_t split_stride, const float* __restrict__ cos_sin,
                                        int rotary_dim, const int* __restrict__ token_pos, TO* __restrict__ out, long long total,
                                        int heads, int dim, int rot, int out_row, int out_offset) {
    pdl_launch_dependents();
    pdl_wait();
    const int half = rotary_dim / 2;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % rot);
        const long long th = idx / rot;
        const int h = (int)(th % heads);
        const long long t = th / heads;
        const size_t at = ((size_t)t * heads + h) * (dim + rot) + dim;
        const float x = load_sum(q, at + i, n_splits, split_stride);
        float y = x;
        if (i < rotary_dim) {
            const float* cs = cos_sin + (size_t)token_pos[t] * rotary_dim;
            const int pair = i < half ? i : i - half;
            const float other = load_sum(q, at + (i < half ? i + half : i - half), n_splits, split_stride);
            y = i < half ? x * cs[pair] - other * cs[half + pair] : x * cs[pair] + other * cs[half + pair];
        }
        out[((size_t)t * heads + h) * out_row + out_offset + i] = from_float<TO>(y);
    }
}

extern "C" int qt_latent_query_rot(const void* q, int in_dtype, int n_splits, long long split_stride, const float* cos_sin, int rotary_dim,
                                   const int* token_pos, void* out, int out_dtype, int n_tokens, int heads, int dim, int rot, int out_row,
                                   int out_offset, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && heads > 0 && dim >= 0 && rot >= 0 && out_offset >= 0 && out_offset + rot <= out_row, "latent_query_rot: bad sizes");
    QT_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= rot && (rotary_dim == 0 || cos_sin), "latent_query_rot: %d of %d elements rotate",
               rotary_dim, rot);
    if (n_tokens == 0 || rot == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n_tokens * heads * rot;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
#define QT_LAUNCH_ROT(TI, TO)                                                                                                      \
    launch_kernel(latent_query_rot_kernel<TI, TO>, dim3((unsigned)blocks), dim3(256), 0, s, (const TI*)q, n_splits, (size_t)split_stride, \
                  cos_sin, rotary_dim, token_pos, (TO*)out, total, heads, dim, rot, out_row, out_offset)
    if (in_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_ROT(float, float);
    else if (in_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_ROT(float, __nv_bfloat16);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_ROT(__nv_bfloat16, __nv_bfloat16);
    else QT_FAIL(QT_ERR_ARG, "latent_query_rot: element types %d/%d", in_dtype, out_dtype);
#undef QT_LAUNCH_ROT
    QT_CHECK_LAUNCH("latent_query_rot");
    return QT_OK;
}

// ----------------------------------------------------------------------------- a product per head
// grid (n tiles, token tiles, heads); a block of 256 threads forms a tile of HP_TM tokens x HP_TN outputs, K in slices
// of HP_TK through shared memory; a thread owns 2 tokens x 4 outputs.  Float accumulation whatever the element types.
constexpr int HP_TM = 32, HP_TN = 64, HP_TK = 16;

struct HeadProductParams {
    const void* x; int x_splits; size_t x_split_stride; long long x_row, x_head; int x_offset;    // X[t, h, k] at t * x_row + h * x_head + x_offset + k
    const void* w;                                                                                // [heads, N, K]
    void* y; long long y_row, y_head; int y_offset;
    const float* gate; int gate_splits; size_t gate_split_stride; int gate_cols, gate_offset;      // optional: times sigmoid(gate[t, gate_offset + h * N + n])
    int n_tokens, heads, n, k;
};

template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256) head_product_kernel(const HeadProductParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float xs[HP_TK][HP_TM + 1];
    __shared__ float wsm[HP_TK][HP_TN + 1];
    const int h = blockIdx.z, t0 = blockIdx.y * HP_TM, n0 = blockIdx.x * HP_TN;
    const TI* x = (const TI*)p.x;
    const TW* w = (const TW*)p.w + (size_t)h * p.n * p.k;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // outputs n0 + tx + 16 j (j < 4), tokens t0 + ty + 16 i (i < 2)
    float acc[2][4] = {};
    for (int k0 = 0; k0 < p.k; k0 += HP_TK) {
        for (int i = threadIdx.x; i < HP_TM * HP_TK; i += 256) {
            const int kk = i % HP_TK, tt = i / HP_TK;
            const int t = t0 + tt, k = k0 + kk;
            xs[kk][tt] = (t < p.n_tokens && k < p.k)
                ? load_sum(x, (size_t)((long long)t * p.x_row + (long long)h * p.x_head + p.x_offset + k), p.x_splits, p.x_split_stride) : 0.f;
        }
        for (int i = threadIdx.x; i < HP_TN * HP_TK; i += 256) {
            const int kk = i % HP_TK, nn = i / HP_TK;
            const int n = n0 + nn, k = k0 + kk;
            wsm[kk][nn] = (n < p.n && k < p.k) ? to_float(w[(size_t)n * p.k + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HP_TK; ++kk) {
            float a[2], b[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = xs[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = wsm[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
    TO* y = (TO*)p.y;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int t = t0 + ty + 16 * i;
        if (t >= p.n_tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= p.n) continue;
            float v = acc[i][j];
            if (p.gate) {
                const float g = sum_splits(p.gate, (size_t)t * p.gate_cols + p.gate_offset + (size_t)h * p.n + n, p.gate_splits, p.gate_split_stride);
                v = v / (1.f + expf(-g));
            }
            y[(size_t)((long long)t * p.y_row + (long long)h * p.y_head + p.y_offset + n)] = from_float<TO>(v);
        }
    }
}

// The same product on the tensor cores: bfloat16 matrices and results, X bfloat16 (copied by cp.async) or float partial
// sums (added and rounded to bfloat16 on the way into shared memory).  grid (n tiles, token tiles, heads); four warps
// form a tile of 64 tokens x 64 outputs (16 tokens a warp), K in slices of 64 through a two-stage ring.
constexpr int HM_T = 64, HM_N = 64, HM_K = 64, HM_LDS = HM_K + 8;

template <typename TI>
__global__ void __launch_bounds__(128) head_product_mma_kernel(const HeadProductParams p) {
    using namespace qt_mma;
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 tiles[2][2][HM_T * HM_LDS];      // [stage][X | W]
    const int h = blockIdx.z, t0 = blockIdx.y * HM_T, n0 = blockIdx.x * HM_N;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const TI* x = (const TI*)p.x;
    const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (size_t)h * p.n * p.k;
    const int slices = (p.k + HM_K - 1) / HM_K;
    auto issue = [&](int slice) {
        if (slice < slices) {
            const int k0 = slice * HM_K;
            __nv_bfloat16* xs = tiles[slice & 1][0];
            __nv_bfloat16* wt = tiles[slice & 1][1];
            for (int i = tid; i < HM_T * (HM_K / 8); i += 128) {
                const int r = i >> 3, c = (i & 7) * 8;
                const int tok = t0 + r, k = k0 + c;
                __nv_bfloat16* dst = xs + r * HM_LDS + c;
                if constexpr (sizeof(TI) == 2) {
                    if (tok < p.n_tokens && k < p.k) cp_async16(smem_u32(dst), x + (size_t)((long long)tok * p.x_row + (long long)h * p.x_head + p.x_offset + k));
                    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                }
                const int n = n0 + r;
                dst = wt + r * HM_LDS + c;
                if (n < p.n && k < p.k) cp_async16(smem_u32(dst), w + (size_t)n * p.k + k);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
            if constexpr (sizeof(TI) == 4) {
                // float partial sums: every load of the slice is issued before the first value is rounded and stored
                constexpr int PER = HM_T * (HM_K / 8) / 128;
                float4 lo[PER], hi[PER];
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int i = tid + j * 128, tok = t0 + (i >> 3), k = k0 + (i & 7) * 8;
                    lo[j] = hi[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (tok < p.n_tokens && k < p.k) {
                        const float* at = (const float*)p.x + (size_t)((long long)tok * p.x_row + (long long)h * p.x_head + p.x_offset + k);
                        for (int sp = 0; sp < p.x_splits; ++sp) {
                            const float4 a = __ldg(reinterpret_cast<const float4*>(at + (size_t)sp * p.x_split_stride));
                            const float4 b = __ldg(reinterpret_cast<const float4*>(at + (size_t)sp * p.x_split_stride) + 1);
                            lo[j].x += a.x; lo[j].y += a.y; lo[j].z += a.z; lo[j].w += a.w;
                            hi[j].x += b.x; hi[j].y += b.y; hi[j].z += b.z; hi[j].w += b.w;
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int i = tid + j * 128;
                    *reinterpret_cast<uint4*>(xs + (i >> 3) * HM_LDS + (i & 7) * 8) =
                        make_uint4(pack_bf16(lo[j].x, lo[j].y), pack_bf16(lo[j].z, lo[j].w), pack_bf16(hi[j].x, hi[j].y), pack_bf16(hi[j].z, hi[j].w));
                }
            }
        }
        cp_async_commit();
    };
    issue(0);
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    const uint32_t a_off = (uint32_t)((warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * HM_LDS + (lane >> 4) * 8) * 2u;
    const int mi = lane >> 3;
    const uint32_t b_off = (uint32_t)(((mi >> 1) * 8 + (lane & 7)) * HM_LDS + (mi & 1) * 8) * 2u;
    for (int slice = 0; slice < slices; ++slice) {
        issue(slice + 1);
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t xs = smem_u32(tiles[slice & 1][0]), wt = smem_u32(tiles[slice & 1][1]);
#pragma unroll
        for (int ks = 0; ks < HM_K / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, xs + a_off + (uint32_t)ks * 32u);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, wt + b_off + (uint32_t)(np * 16 * HM_LDS + ks * 16) * 2u);
                mma_bf16(acc[2 * np], a, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __nv_bfloat16* y = (__nv_bfloat16*)p.y;
    const bool paired = ((p.y_row | p.y_head | (long long)p.y_offset) & 1) == 0;
    if (p.gate) {
        // the gates of all of this thread's results are summed (split by split, the loads of a split independent of one
        // another) before the first result is stored
        float gates[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) gates[nt][0] = gates[nt][1] = gates[nt][2] = gates[nt][3] = 0.f;
        for (int sp = 0; sp < p.gate_splits; ++sp) {
            const float* gate = p.gate + (size_t)sp * p.gate_split_stride;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int tok = t0 + warp * 16 + g + 8 * r;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    const int n = n0 + nt * 8 + 2 * t;
                    const size_t at = (size_t)tok * p.gate_cols + p.gate_offset + (size_t)h * p.n + n;
                    if (tok < p.n_tokens && n < p.n) gates[nt][2 * r] += __ldg(gate + at);
                    if (tok < p.n_tokens && n + 1 < p.n) gates[nt][2 * r + 1] += __ldg(gate + at + 1);
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = acc[nt][e] / (1.f + expf(-gates[nt][e]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int tok = t0 + warp * 16 + g + 8 * r;
        if (tok >= p.n_tokens) continue;
        __nv_bfloat16* dst = y + (size_t)((long long)tok * p.y_row + (long long)h * p.y_head + p.y_offset);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int n = n0 + nt * 8 + 2 * t;
            if (n >= p.n) continue;
            const float v0 = acc[nt][2 * r], v1 = acc[nt][2 * r + 1];
            if (paired && n + 1 < p.n) {
                *reinterpret_cast<uint32_t*>(dst + n) = pack_bf16(v0, v1);
            } else {
                dst[n] = __float2bfloat16_rn(v0);
                if (n + 1 < p.n) dst[n + 1] = __float2bfloat16_rn(v1);
            }
        }
    }
}

extern "C" int qt_head_product(const void* x, int x_dtype, int x_splits, long long x_split_stride, long long x_row, long long x_head, int x_offset,
                               const void* w, int w_dtype, void* y, int y_dtype, long long y_row, long long y_head, int y_offset,
                               const float* gate, int gate_splits, long long gate_split_stride, int gate_cols, int gate_offset,
                               int n_tokens, int heads, int n, int k, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && heads > 0 && n > 0 && k > 0 && x_splits >= 1 && gate_splits >= 1, "head_product: bad sizes");
    QT_REQUIRE(heads <= 65535 && (n_tokens + HP_TM - 1) / HP_TM <= 65535, "head_product: too many heads or tokens for one launch");
    QT_REQUIRE(!gate || gate_offset + heads * n <= gate_cols, "head_product: the gate needs %d columns at %d of %d", heads * n, gate_offset, gate_cols);
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    HeadProductParams p{x, x_splits, (size_t)x_split_stride, x_row, x_head, x_offset, w, y, y_row, y_head, y_offset,
                        gate, gate_splits, (size_t)gate_split_stride, gate_cols, gate_offset, n_tokens, heads, n, k};
    dim3 grid((n + HP_TN - 1) / HP_TN, (n_tokens + HP_TM - 1) / HP_TM, heads);
    // bfloat16 matrices and results whose rows start on 16 bytes take the tensor cores (QT_B200_HEAD_PRODUCT_MMA=0: never)
    static const bool mma_allowed = [] { const char* env = getenv("QT_B200_HEAD_PRODUCT_MMA"); return !(env && env[0] == '0'); }();
    if (mma_allowed && w_dtype == QT_BF16 && y_dtype == QT_BF16 && k % 8 == 0 && (n_tokens + HM_T - 1) / HM_T <= 65535 &&
        ((x_dtype == QT_F32 && x_row % 4 == 0 && x_head % 4 == 0 && x_offset % 4 == 0 && x_split_stride % 4 == 0 && ((uintptr_t)x & 15) == 0) ||
         (x_dtype == QT_BF16 && x_splits == 1 && x_row % 8 == 0 && x_head % 8 == 0 && x_offset % 8 == 0 && ((uintptr_t)x & 15) == 0)) &&
        ((uintptr_t)w & 15) == 0) {
        dim3 tiles((n + HM_N - 1) / HM_N, (n_tokens + HM_T - 1) / HM_T, heads);
        if (x_dtype == QT_F32) launch_kernel(head_product_mma_kernel<float>, tiles, dim3(128), 0, s, p);
        else launch_kernel(head_product_mma_kernel<__nv_bfloat16>, tiles, dim3(128), 0, s, p);
        QT_CHECK_LAUNCH("head_product_mma");
        return QT_OK;
    }
#define QT_LAUNCH_HP(TI, TW, TO) launch_kernel(head_product_kernel<TI, TW, TO>, grid, dim3(256), 0, s, p)
    if (x_dtype == QT_F32 && w_dtype == QT_F32 && y_dtype == QT_F32) QT_LAUNCH_HP(float, float, float);
    else if (x_dtype == QT_F32 && w_dtype == QT_BF16 && y_dtype == QT_BF16) QT_LAUNCH_HP(float, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == QT_BF16 && w_dtype == QT_BF16 && y_dtype == QT_BF16) QT_LAUNCH_HP(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else QT_FAIL(QT_ERR_ARG, "head_product: element types %d/%d/%d", x_dtype, w_dtype, y_dtype);
#undef QT_LAUNCH_HP
    QT_CHECK_LAUNCH("head_product");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(latent)
