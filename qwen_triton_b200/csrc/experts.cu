// Feed-forward experts chosen per token by a table: each token runs the `top` experts that the table's row of its
// token id names, out[t] = sum_k weight_k * W_down[e_k] act(W_up[e_k] x[t]).  The routing is read on the device
// (token ids and table are device arrays), so a step with these kernels has the same launches whatever the tokens
// are and can be captured in a CUDA graph.
//
// Two forms.  Few tokens (a decode step): one pass of matrix-vector products per (token, expert) pair, the expert's
// rows streamed once per pair.  Many tokens: the pairs are ordered by expert on the device (count, offsets, scatter;
// every expert's run padded to whole tiles of rows), and the two products run tile by tile, a tile's rows all of one
// expert, so that an expert's weights are read once per tile instead of once per pair.
//
// The same kernels serve experts chosen by a learned router: without token ids the "table" is read by token (row t
// holds the experts that a router kernel chose for token t), every pair has a weight of its own (`pair_weights`),
// an expert may be gated (its first matrix holds [gate; up] rows, mid = gate(g, u)), and a further term
// row_scale[t] * base[t] (a shared expert behind a gate of one number per token) may be added to the sum.
#include "common.cuh"

#include <math.h>

using namespace qt;

// ----------------------------------------------------------------------------- few tokens: per pair
constexpr int EV_WARPS = 8;
constexpr int EV_FEATS = 4;        // output features per warp and pass

struct ExpertParams {
    const void* x;            // [T, width] normed rows
    const int* token_ids;     // [T]
    const int* table;         // [vocab, top]
    const void* up;           // [E, ff, width]
    const void* down;         // [E, width, ff]
    void* mid;                // [T * top, ff] activations
    float* out;               // [T, width] float
    int n_tokens, vocab, top, experts, width, ff, act;
    float pair_weight;        // weight of every chosen expert (1 / top for an unweighted mean)
    const float* pair_weights;  // [T, top] a weight per pair instead, or null
    int gated; float limit;     // up holds [E, 2 ff, width]: ff gate rows, then ff up rows; mid = gated_value(g, u, act, limit)
    const float* base; int base_splits; size_t base_stride;   // [splits, T, width] float added to out, times row_scale[t]; or null
    const float* row_scale;     // [T] or null (1)
    const float* in_weights;    // [T, top] or null: a pair's expert reads its token's row times this (a weight on the input, not the output)
};

__device__ __forceinline__ int expert_of(const ExpertParams& p, int t, int k) {
    int id = p.token_ids ? p.token_ids[t] : t;            // no ids: the table's row t is token t's
    id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
    int e = p.table[(size_t)id * p.top + k];
    return e < 0 ? 0 : (e >= p.experts ? p.experts - 1 : e);          // never read outside the weights
}

// Eight consecutive elements of a weight row as floats, by 16-byte loads (rows that start on 16-byte boundaries).
__device__ __forceinline__ void load8(const float* src, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* src, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[2 * j] = __low2float(h[j]); v[2 * j + 1] = __high2float(h[j]); }
}

// EV_FEATS dot products of consecutive weight rows (`stride` apart, `n` elements each) with a vector in shared memory,
// summed over the warp.  VEC: n is a multiple of 8 and the rows start on 16-byte boundaries; every lane then loads 16
// bytes of each row per turn, all rows' loads of a turn ahead of its arithmetic.
template <typename T, bool VEC>
__device__ __forceinline__ void warp_dots(const T* __restrict__ w, size_t stride, int rows, int n, const float* __restrict__ xs, int lane,
                                          float (&acc)[EV_FEATS]) {
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) acc[j] = 0.f;
    if (VEC) {
        for (int i = lane * 8; i < n; i += 256) {
            float wv[EV_FEATS][8];
#pragma unroll
            for (int j = 0; j < EV_FEATS; ++j) load8(w + (size_t)(j < rows ? j : 0) * stride + i, wv[j]);
            const float4 xa = *reinterpret_cast<const float4*>(xs + i), xb = *reinterpret_cast<const float4*>(xs + i + 4);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int j = 0; j < EV_FEATS; ++j)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[j] += wv[j][e] * xv[e];
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            const float xv = xs[i];
#pragma unroll
            for (int j = 0; j < EV_FEATS; ++j)
                if (j < rows) acc[j] += to_float(w[(size_t)j * stride + i]) * xv;
        }
    }
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) acc[j] = warp_sum(acc[j]);
}

// mid[pair, f] = act(W_up[e][f, :] . x[t, :]).  grid (pairs, feature blocks); x[t] in shared memory as float.
template <typename T, bool VEC>
__global__ void __launch_bounds__(EV_WARPS * 32) expert_up_kernel(const ExpertParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];
    const int pair = blockIdx.x, t = pair / p.top, k = pair % p.top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* x = (const T*)p.x + (size_t)t * p.width;
    const float in_weight = p.in_weights ? p.in_weights[pair] : 1.f;
    for (int i = threadIdx.x; i < p.width; i += blockDim.x) xs[i] = to_float(x[i]) * in_weight;
    __syncthreads();
    const int e = expert_of(p, t, k);
    const T* w = (const T*)p.up + (size_t)e * (p.gated ? 2 : 1) * p.ff * p.width;
    T* mid = (T*)p.mid + (size_t)pair * p.ff;
    const int f0 = (blockIdx.y * EV_WARPS + warp) * EV_FEATS;
    if (f0 >= p.ff) return;
    float acc[EV_FEATS];
    warp_dots<T, VEC>(w + (size_t)f0 * p.width, (size_t)p.width, p.ff - f0, p.width, xs, lane, acc);
    if (p.gated) {
        float up[EV_FEATS];
        warp_dots<T, VEC>(w + (size_t)(p.ff + f0) * p.width, (size_t)p.width, p.ff - f0, p.width, xs, lane, up);
#pragma unroll
        for (int j = 0; j < EV_FEATS; ++j)
            if (lane == 0 && f0 + j < p.ff) mid[f0 + j] = from_float<T>(gated_value<false>(acc[j], up[j], p.act, p.limit));
        return;
    }
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j)
        if (lane == 0 && f0 + j < p.ff) mid[f0 + j] = from_float<T>(gate_activation<false>(acc[j], p.act));
}

// out[t, c] = pair_weight * sum_k W_down[e_k][c, :] . mid[t * top + k, :].  grid (tokens, column blocks).
template <typename T, bool VEC>
__global__ void __launch_bounds__(EV_WARPS * 32) expert_down_kernel(const ExpertParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float ms[];                 // [top, ff]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* mid = (const T*)p.mid + (size_t)t * p.top * p.ff;
    for (int i = threadIdx.x; i < p.top * p.ff; i += blockDim.x) ms[i] = to_float(mid[i]);
    __syncthreads();
    const int c0 = (blockIdx.y * EV_WARPS + warp) * EV_FEATS;
    if (c0 >= p.width) return;
    float total[EV_FEATS];
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j) total[j] = 0.f;
    for (int k = 0; k < p.top; ++k) {                      // in the order of the table's row
        const int e = expert_of(p, t, k);
        const T* w = (const T*)p.down + (size_t)e * p.width * p.ff;
        float acc[EV_FEATS];
        warp_dots<T, VEC>(w + (size_t)c0 * p.ff, (size_t)p.ff, p.width - c0, p.ff, ms + k * p.ff, lane, acc);
        const float weight = p.pair_weights ? p.pair_weights[(size_t)t * p.top + k] : 1.f;
#pragma unroll
        for (int j = 0; j < EV_FEATS; ++j) total[j] += acc[j] * weight;
    }
#pragma unroll
    for (int j = 0; j < EV_FEATS; ++j)
        if (lane == 0 && c0 + j < p.width) {
            const size_t at = (size_t)t * p.width + c0 + j;
            float y = p.pair_weights ? total[j] : total[j] * p.pair_weight;
            if (p.base) y += (p.row_scale ? p.row_scale[t] : 1.f) * load_sum(p.base, at, p.base_splits, p.base_stride);
            p.out[at] = y;
        }
}

static int check_experts(const char* name, int n_tokens, int vocab, int top, int experts, int width, int ff, int act) {
    QT_REQUIRE(n_tokens >= 0 && vocab > 0 && top > 0 && experts > 0 && top <= experts, "%s: bad routing sizes T=%d V=%d top=%d E=%d", name, n_tokens, vocab, top, experts);
    QT_REQUIRE(width > 0 && ff > 0, "%s: bad sizes width=%d ff=%d", name, width, ff);
    QT_REQUIRE(act >= 0 && act <= QT_ACT_CAPPED, "%s: unknown activation code %d", name, act);
    return QT_OK;
}

extern "C" int qt_experts_by_pair(const void* x, const int* token_ids, const int* table, const void* up, const void* down, void* mid,
                                  float* out, int dtype, int n_tokens, int vocab, int top, int experts, int width, int ff, int act,
                                  float pair_weight, const float* pair_weights, int gated, float limit, const float* base,
                                  int base_splits, long long base_stride, const float* row_scale, const float* in_weights, void* stream) {
    QT_REQUIRE(gated || act < QT_ACT_COUNT, "experts_by_pair: activation %d needs gated experts", act);
    int rc = check_experts("experts_by_pair", n_tokens, vocab, top, experts, width, ff, act);
    if (rc) return rc;
    if (n_tokens == 0) return QT_OK;
    QT_REQUIRE((size_t)width * 4 <= 200 * 1024 && (size_t)top * ff * 4 <= 200 * 1024, "experts_by_pair: a row of %d or %d x %d floats does not fit shared memory", width, top, ff);
    ExpertParams p{x, token_ids, table, up, down, mid, out, n_tokens, vocab, top, experts, width, ff, act, pair_weight,
                   pair_weights, gated, limit, base, base_splits, (size_t)base_stride, row_scale, in_weights};
    cudaStream_t s = (cudaStream_t)stream;
    const int per_block = EV_WARPS * EV_FEATS;
    return QT_DISPATCH_DTYPE(dtype, "experts_by_pair", {
        const size_t smem_up = (size_t)width * sizeof(float), smem_down = (size_t)top * ff * sizeof(float);
        const dim3 grid_up(n_tokens * top, (ff + per_block - 1) / per_block), grid_down(n_tokens, (width + per_block - 1) / per_block);
        // 16-byte loads: rows of both weights, and the experts' matrices, start on 16-byte boundaries
        const bool vec = width % 8 == 0 && ff % 8 == 0 && (uintptr_t)up % 16 == 0 && (uintptr_t)down % 16 == 0;
        if (vec) {
            if (smem_up > 48 * 1024) cudaFuncSetAttribute(expert_up_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
            if (smem_down > 48 * 1024) cudaFuncSetAttribute(expert_down_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
            launch_kernel(expert_up_kernel<T, true>, grid_up, dim3(EV_WARPS * 32), smem_up, s, p);
            QT_CHECK_LAUNCH("expert_up");
            launch_kernel(expert_down_kernel<T, true>, grid_down, dim3(EV_WARPS * 32), smem_down, s, p);
        } else {
            if (smem_up > 48 * 1024) cudaFuncSetAttribute(expert_up_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
            if (smem_down > 48 * 1024) cudaFuncSetAttribute(expert_down_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
            launch_kernel(expert_up_kernel<T, false>, grid_up, dim3(EV_WARPS * 32), smem_up, s, p);
            QT_CHECK_LAUNCH("expert_up");
            launch_kernel(expert_down_kernel<T, false>, grid_down, dim3(EV_WARPS * 32), smem_down, s, p);
        }
        QT_CHECK_LAUNCH("expert_down");
        return QT_OK;
    });
}

// ----------------------------------------------------------------------------- many tokens: pairs ordered by expert
// Routing for the tiled products (experts_tc.cu).  One block: count the pairs of every expert, give every expert a
// run of rows padded to whole tiles of `tile_rows`, and give every pair a row in its expert's run.
//   pair_row[pair]     the pair's row in the ordered buffers
//   row_token[row]     the pair whose token's (normed) input the row holds (the token is pair / top), -1 for padding
//   tile_expert[tile]  the expert of the tile's rows, -1 for tiles beyond the last run
// Which row of its run a pair gets depends on the order the threads arrive in; a row's results do not depend on where
// it lies, so the output does not either.
__global__ void __launch_bounds__(1024) expert_route_kernel(const ExpertParams p, int* __restrict__ pair_row, int* __restrict__ row_token,
                                                            int* __restrict__ tile_expert, int tile_rows, int max_tiles) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int route_smem[];
    int* counts = route_smem;                 // [E]
    int* starts = counts + p.experts;         // [E + 1], in rows
    int* cursor = starts + p.experts + 1;     // [E]
    const int pairs = p.n_tokens * p.top;
    for (int e = threadIdx.x; e < p.experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) atomicAdd(&counts[expert_of(p, pair / p.top, pair % p.top)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < p.experts; ++e) {
            starts[e] = at;
            at += (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
        }
        starts[p.experts] = at;
    }
    __syncthreads();
    const int used_tiles = starts[p.experts] / tile_rows;
    for (int e = threadIdx.x; e < p.experts; e += blockDim.x)
        for (int tile = starts[e] / tile_rows; tile < starts[e + 1] / tile_rows; ++tile) tile_expert[tile] = e;
    for (int tile = used_tiles + threadIdx.x; tile < max_tiles; tile += blockDim.x) tile_expert[tile] = -1;
    for (int row = threadIdx.x; row < max_tiles * tile_rows; row += blockDim.x) row_token[row] = -1;
    __syncthreads();
    for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
        const int e = expert_of(p, pair / p.top, pair % p.top);
        const int row = starts[e] + atomicAdd(&cursor[e], 1);
        pair_row[pair] = row;
        row_token[row] = pair;
    }
}

// ordered[row, :] = x[row_token[row] / top, :] (zeros for padding rows), times the pair's input weight where there is one
// (the product in float, rounded once).  One block per row, 16 bytes per thread and turn.
__global__ void expert_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ row_token, uint4* __restrict__ ordered, int chunks, int top,
                                     const float* __restrict__ in_weights) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, pair = row_token[row], token = pair >= 0 ? pair / top : -1;
    const float w = (in_weights && pair >= 0) ? in_weights[pair] : 1.f;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        uint4 v = token >= 0 ? x[(size_t)token * chunks + c] : make_uint4(0u, 0u, 0u, 0u);
        if (in_weights) {
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(__low2float(h[j]) * w, __high2float(h[j]) * w);
        }
        ordered[(size_t)row * chunks + c] = v;
    }
}

// out[t, :] = pair_weight * sum_k y[pair_row[t * top + k], :], in float, in the order of k.
template <typename T>
__global__ void expert_combine_kernel(const T* __restrict__ y, const int* __restrict__ pair_row, float* __restrict__ out, int top, int width,
                                      float pair_weight, const float* __restrict__ pair_weights, const float* __restrict__ base,
                                      int base_splits, size_t base_stride, const float* __restrict__ row_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k)
            acc += to_float(y[(size_t)pair_row[t * top + k] * width + c]) * (pair_weights ? pair_weights[(size_t)t * top + k] : 1.f);
        if (!pair_weights) acc *= pair_weight;
        const size_t at = (size_t)t * width + c;
        if (base) acc += (row_scale ? row_scale[t] : 1.f) * load_sum(base, at, base_splits, base_stride);
        out[at] = acc;
    }
}

// A learned router's choice.  logits [splits, T, cols] float (column e < experts: expert e; column `experts`, if
// shared_gate, the logit of a shared expert's gate).  Scores are sigmoid(logit); the `top` largest are chosen (by their
// logits; of equal ones the lower expert first), their weights are the scores over their sum (+ 1e-20) times `scale`, or, without `normalize`, the scores themselves times `scale`.
// One warp per token; chosen [T, top], weights [T, top], gate [T] = sigmoid of the extra column.
__global__ void __launch_bounds__(128) route_top_kernel(const float* __restrict__ logits, int n_splits, size_t split_stride, int cols,
                                                        int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ gate,
                                                        int n_tokens, int experts, int top, float scale, int normalize) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float route_scores[];                      // [warps][experts]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* score = route_scores + (size_t)warp * experts;        // the logits: their order is the scores' order, and two logits
    // that differ stay apart where their sigmoids round to the same float
    for (int e = lane; e < experts; e += 32) score[e] = load_sum(logits, (size_t)t * cols + e, n_splits, split_stride);
    if (gate && lane == 0) gate[t] = 1.f / (1.f + expf(-load_sum(logits, (size_t)t * cols + experts, n_splits, split_stride)));
    __syncwarp();
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = experts;
        for (int e = lane; e < experts; e += 32)
            if (score[e] > best || at == experts) { best = score[e]; at = e; }
        for (int off = 16; off > 0; off >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, off);
            const int where = __shfl_xor_sync(0xffffffffu, at, off);
            if (where < experts && (at == experts || other > best || (other == best && where < at))) { best = other; at = where; }
        }
        const float chosen_score = 1.f / (1.f + expf(-best));
        sum += chosen_score;
        if (lane == 0) { chosen[(size_t)t * top + k] = at; weights[(size_t)t * top + k] = chosen_score; score[at] = -INFINITY; }
        __syncwarp();
    }
    if (lane < top) {
        for (int k = lane; k < top; k += 32)
            weights[(size_t)t * top + k] = normalize ? weights[(size_t)t * top + k] / (sum + 1e-20f) * scale : weights[(size_t)t * top + k] * scale;
    }
}

extern "C" int qt_route_top(const float* logits, int n_splits, long long split_stride, int cols, int* chosen, float* weights, float* gate,
                            int n_tokens, int experts, int top, float scale, int normalize, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && experts > 0 && top > 0 && top <= experts && cols >= experts + (gate ? 1 : 0) && n_splits >= 1,
               "route_top: bad sizes T=%d E=%d top=%d cols=%d", n_tokens, experts, top, cols);
    QT_REQUIRE((size_t)4 * experts * sizeof(float) <= 48 * 1024, "route_top: %d experts are too many for a warp's scores in shared memory", experts);
    if (n_tokens == 0) return QT_OK;
    launch_kernel(route_top_kernel, dim3((n_tokens + 3) / 4), dim3(128), (size_t)4 * experts * sizeof(float), (cudaStream_t)stream, logits, n_splits,
                  (size_t)split_stride, cols, chosen, weights, gate, n_tokens, experts, top, scale, normalize);
    QT_CHECK_LAUNCH("route_top");
    return QT_OK;
}

extern "C" int qt_experts_route(const void* x, const int* token_ids, const int* table, void* ordered, int* pair_row, int* row_token,
                                int* tile_expert, int n_tokens, int vocab, int top, int experts, int width, int tile_rows, int max_tiles,
                                const float* in_weights, void* stream) {
    int rc = check_experts("experts_route", n_tokens, vocab, top, experts, width, 1, 0);
    if (rc) return rc;
    if (n_tokens == 0) return QT_OK;
    QT_REQUIRE(width % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)ordered % 16 == 0, "experts_route: rows of 16-byte pieces are needed (width=%d)", width);
    QT_REQUIRE(tile_rows > 0 && (long long)max_tiles * tile_rows >= (long long)n_tokens * top, "experts_route: %d tiles of %d rows do not hold the pairs", max_tiles, tile_rows);
    QT_REQUIRE((3 * (size_t)experts + 1) * sizeof(int) <= 48 * 1024, "experts_route: %d experts are too many for one block's counters", experts);
    ExpertParams p{x, token_ids, table, nullptr, nullptr, nullptr, nullptr, n_tokens, vocab, top, experts, width, 1, 0, 0.f,
                   nullptr, 0, 0.f, nullptr, 1, 0, nullptr, nullptr};
    cudaStream_t s = (cudaStream_t)stream;
    launch_kernel(expert_route_kernel, dim3(1), dim3(1024), (3 * (size_t)experts + 1) * sizeof(int), s, p, pair_row, row_token, tile_expert, tile_rows, max_tiles);
    QT_CHECK_LAUNCH("expert_route");
    launch_kernel(expert_gather_kernel, dim3(max_tiles * tile_rows), dim3(128), 0, s, (const uint4*)x, (const int*)row_token, (uint4*)ordered, width / 8, top, in_weights);
    QT_CHECK_LAUNCH("expert_gather");
    return QT_OK;
}

extern "C" int qt_experts_combine(const void* y, int dtype, const int* pair_row, float* out, int n_tokens, int top, int width, float pair_weight,
                                  const float* pair_weights, const float* base, int base_splits, long long base_stride,
                                  const float* row_scale, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && top > 0 && width > 0, "experts_combine: bad sizes T=%d top=%d width=%d", n_tokens, top, width);
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    return QT_DISPATCH_DTYPE(dtype, "experts_combine", {
        // few tokens: the columns of a row over several blocks, so that the launch fills the machine
        const unsigned column_blocks = n_tokens >= 1024 ? 1u : (unsigned)((width + 255) / 256);
        launch_kernel(expert_combine_kernel<T>, dim3(n_tokens, column_blocks), dim3(256), 0, s, (const T*)y, pair_row, out, top, width, pair_weight, pair_weights, base,
                      base_splits, (size_t)base_stride, row_scale);
        QT_CHECK_LAUNCH("expert_combine");
        return QT_OK;
    });
}

QT_DEFINE_LAST_ERROR(experts)
