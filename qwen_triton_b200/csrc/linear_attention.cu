// Linear attention with a constant decay per head, and the norm and gate behind it.
//
// Per head a float state S [dim, vdim] is carried from token to token of a sequence:
//     S <- decay_h * S + k_t v_t^T;      o_t = S^T q_t        (o_t is read after token t has been written)
// q, k [heads, dim] and v [heads, vdim] are columns of one projection's float sums (split-K partial sums are added in
// their order); with `act` they pass SiLU on the way in.  The recurrence, the state and the output are float.
//
// linear_attention_scan_kernel   grid (column blocks, heads, sequences), 256 threads: a block owns 32 columns of a
//   head's state, a column belongs to 8 neighbouring lanes, each holding RPL consecutive rows of it in registers, so a
//   token costs a thread 2 RPL fused multiply-adds and the column's sum over rows three shuffles.  The state is kept
//   transposed, [slots, heads, vdim, dim], so that the 8 lanes of a column read and write 8 RPL consecutive floats.
//   A sequence's tokens are walked in order, 16 at a time through shared memory; a one-token step is the same kernel
//   with one token, whose cost is the state's bytes.
// linear_attention_gate_norm_kernel   one block per token: out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g) * scale,
//   the mean over all heads' outputs of the token at once, g the projection's gate columns, rounded once to the
//   output type.
#include "common.cuh"

#include <math.h>

using namespace qt;

constexpr int LA_LANES = 8;        // lanes per state column
constexpr int LA_COLS = 32;        // columns per block
constexpr int LA_CHUNK = 16;       // tokens staged in shared memory at a time

struct LinAttnParams {
    const float* proj; int n_splits; size_t split_stride; int proj_cols;   // [splits, T, proj_cols]
    int at_q, at_k, at_v;              // first columns of q, k and v
    const float* decay;                // [heads]
    float* state;                      // [slots + 1, heads, vdim, dim]
    float* out;                        // [T, heads, vdim]
    const int* seq_start; const int* slots;
    int heads, dim, vdim, act;
};

__device__ __forceinline__ float la_in(const LinAttnParams& p, size_t index) {
    float x = p.proj[index];
    for (int s = 1; s < p.n_splits; ++s) x += p.proj[index + (size_t)s * p.split_stride];
    return p.act ? x / (1.f + expf(-x)) : x;
}

template <int RPL>
__global__ void __launch_bounds__(LA_COLS * LA_LANES) linear_attention_scan_kernel(const LinAttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int STRIDE = LA_LANES * (RPL + 4);          // a token's q (or k) row in shared memory: 4 floats of padding per lane's
    __shared__ __align__(16) float qs[LA_CHUNK * STRIDE];  // piece, so that the 8 lanes' 16-byte reads fall on different banks
    __shared__ __align__(16) float ks[LA_CHUNK * STRIDE];
    __shared__ float vs[LA_CHUNK * LA_COLS];
    const int head = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x % LA_LANES, col_in_block = threadIdx.x / LA_LANES;
    const int col = blockIdx.x * LA_COLS + col_in_block;
    const int begin = p.seq_start[seq], end = p.seq_start[seq + 1];
    if (begin >= end) return;
    const float decay = p.decay[head];
    const bool live = col < p.vdim;
    float* state = p.state + (((size_t)p.slots[seq] * p.heads + head) * p.vdim + (live ? col : 0)) * p.dim;
    const int row0 = lane * RPL;
    const bool vec = p.dim % 4 == 0 && ((uintptr_t)p.state & 15) == 0;
    float S[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) S[i] = 0.f;
    if (live) {
        if (vec) {
#pragma unroll
            for (int i = 0; i < RPL; i += 4)
                if (row0 + i < p.dim) {
                    const float4 v = *reinterpret_cast<const float4*>(state + row0 + i);
                    S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w;
                }
        } else {
#pragma unroll
            for (int i = 0; i < RPL; ++i)
                if (row0 + i < p.dim) S[i] = state[row0 + i];
        }
    }
    for (int t0 = begin; t0 < end; t0 += LA_CHUNK) {
        const int count = min(LA_CHUNK, end - t0);
        __syncthreads();                                   // the chunk before has been read
        for (int i = threadIdx.x; i < count * LA_LANES * RPL; i += blockDim.x) {
            const int tok = i / (LA_LANES * RPL), r = i % (LA_LANES * RPL);
            const size_t row = (size_t)(t0 + tok) * p.proj_cols;
            const int at = tok * STRIDE + (r / RPL) * (RPL + 4) + r % RPL;
            qs[at] = r < p.dim ? la_in(p, row + p.at_q + (size_t)head * p.dim + r) : 0.f;
            ks[at] = r < p.dim ? la_in(p, row + p.at_k + (size_t)head * p.dim + r) : 0.f;
        }
        for (int i = threadIdx.x; i < count * LA_COLS; i += blockDim.x) {
            const int tok = i / LA_COLS, c = blockIdx.x * LA_COLS + i % LA_COLS;
            vs[i] = c < p.vdim ? la_in(p, (size_t)(t0 + tok) * p.proj_cols + p.at_v + (size_t)head * p.vdim + c) : 0.f;
        }
        __syncthreads();
        for (int tok = 0; tok < count; ++tok) {
            const float v = vs[tok * LA_COLS + col_in_block];
            const float* qrow = qs + tok * STRIDE + lane * (RPL + 4);
            const float* krow = ks + tok * STRIDE + lane * (RPL + 4);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(krow + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qrow + i);
                S[i] = fmaf(decay, S[i], k4.x * v);         acc = fmaf(S[i], q4.x, acc);
                S[i + 1] = fmaf(decay, S[i + 1], k4.y * v); acc = fmaf(S[i + 1], q4.y, acc);
                S[i + 2] = fmaf(decay, S[i + 2], k4.z * v); acc = fmaf(S[i + 2], q4.z, acc);
                S[i + 3] = fmaf(decay, S[i + 3], k4.w * v); acc = fmaf(S[i + 3], q4.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (lane == 0 && live) p.out[((size_t)(t0 + tok) * p.heads + head) * p.vdim + col] = acc;
        }
    }
    if (live) {
        if (vec) {
#pragma unroll
            for (int i = 0; i < RPL; i += 4)
                if (row0 + i < p.dim) *reinterpret_cast<float4*>(state + row0 + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < RPL; ++i)
                if (row0 + i < p.dim) state[row0 + i] = S[i];
        }
    }
}

extern "C" int qt_linear_attention_scan(const float* proj, int n_splits, long long split_stride, int proj_cols, int at_q, int at_k, int at_v,
                                        const float* decay, float* state, float* out, const int* seq_start, const int* slots, int n_seqs,
                                        int heads, int dim, int vdim, int act, void* stream) {
    QT_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0 && n_splits >= 1, "linear_attention_scan: bad sizes B=%d H=%d dim=%d vdim=%d", n_seqs, heads, dim, vdim);
    QT_REQUIRE(dim <= LA_LANES * 32, "linear_attention_scan: %d key channels per head are beyond what a column's lanes hold (%d)", dim, LA_LANES * 32);
    QT_REQUIRE(at_q >= 0 && at_k >= 0 && at_v >= 0 && at_q + heads * dim <= proj_cols && at_k + heads * dim <= proj_cols && at_v + heads * vdim <= proj_cols,
               "linear_attention_scan: q, k or v columns outside the projection's %d", proj_cols);
    if (n_seqs == 0) return QT_OK;
    LinAttnParams p{proj, n_splits, (size_t)split_stride, proj_cols, at_q, at_k, at_v, decay, state, out, seq_start, slots, heads, dim, vdim, act};
    const dim3 grid((vdim + LA_COLS - 1) / LA_COLS, heads, n_seqs), block(LA_COLS * LA_LANES);
    cudaStream_t s = (cudaStream_t)stream;
    if (dim <= LA_LANES * 8) launch_kernel(linear_attention_scan_kernel<8>, grid, block, 0, s, p);
    else if (dim <= LA_LANES * 16) launch_kernel(linear_attention_scan_kernel<16>, grid, block, 0, s, p);
    else launch_kernel(linear_attention_scan_kernel<32>, grid, block, 0, s, p);
    QT_CHECK_LAUNCH("linear_attention_scan");
    return QT_OK;
}

// ----------------------------------------------------------------------------- norm over all heads, gate, scale
template <typename TO>
__global__ void linear_attention_gate_norm_kernel(const float* __restrict__ o, const float* __restrict__ proj, int n_splits, size_t split_stride,
                                                  int proj_cols, int at_gate, const float* __restrict__ weight, float eps, float scale,
                                                  TO* __restrict__ out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    const float* row = o + t * width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) sq += row[i] * row[i];
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)width + eps) * scale;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float y = row[i] * inv * weight[i];
        if (proj) {
            const size_t at = t * proj_cols + at_gate + i;
            float g = proj[at];
            for (int s = 1; s < n_splits; ++s) g += proj[at + (size_t)s * split_stride];
            y = y / (1.f + expf(-g));
        }
        out[t * width + i] = from_float<TO>(y);
    }
}

extern "C" int qt_linear_attention_gate_norm(const float* o, const float* proj, int n_splits, long long split_stride, int proj_cols, int at_gate,
                                             const float* weight, float eps, float scale, void* out, int out_dtype, int n_tokens, int width,
                                             void* stream) {
    QT_REQUIRE(n_tokens >= 0 && width > 0 && eps > 0.f, "linear_attention_gate_norm: bad sizes T=%d width=%d", n_tokens, width);
    QT_REQUIRE(!proj || (at_gate >= 0 && at_gate + width <= proj_cols && n_splits >= 1), "linear_attention_gate_norm: gate columns outside the projection");
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    return QT_DISPATCH_DTYPE(out_dtype, "linear_attention_gate_norm", {
        launch_kernel(linear_attention_gate_norm_kernel<T>, dim3(n_tokens), dim3(threads), 0, s, o, proj, n_splits, (size_t)split_stride, proj_cols,
                      at_gate, weight, eps, scale, (T*)out, width);
        QT_CHECK_LAUNCH("linear_attention_gate_norm");
        return QT_OK;
    });
}

QT_DEFINE_LAST_ERROR(linear_attention)
