// Linear attention with a constant decay per head, and the norm and gate behind it.
//
// Per head a float state S [dim, vdim] is carried from token to token of a sequence:
//     S <- decay_h * S + k_t v_t^T;      o_t = S^T q_t        (o_t is read after token t has been written)
// q, k [heads, dim] and v [heads, vdim] are columns of one projection's float sums (split-K partial sums are added in
// their order); with `act` they pass SiLU on the way in.  The recurrence, the state and the output are float.
//
// linear_attention_scan_kernel   grid (column blocks, heads, sequences): a block owns 32 (or 16) columns of a
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
#include <stdlib.h>

using namespace qt;

constexpr int LA_LANES = 8;        // lanes per state column
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

__device__ __forceinline__ float la_raw(const LinAttnParams& p, size_t index) {
    float x = __ldg(p.proj + index);
    for (int s = 1; s < p.n_splits; ++s) x += __ldg(p.proj + index + (size_t)s * p.split_stride);
    return x;
}
__device__ __forceinline__ float la_act(const LinAttnParams& p, float x) { return p.act ? x / (1.f + expf(-x)) : x; }

// out[t, c] = SiLU(sum_s proj[s][t, c]) (or the sum itself) for the first `cols` columns of every row: q, k and v of a
// step, summed and activated once where every block of the recurrence would otherwise activate its head's q and k again.
__global__ void linear_attention_prepare_kernel(const float* __restrict__ proj, int n_splits, size_t split_stride, int proj_cols, int cols,
                                                float* __restrict__ out, long long total, int act) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const size_t at = (size_t)(i / cols) * proj_cols + (size_t)(i % cols);
        float x = proj[at];
        for (int s = 1; s < n_splits; ++s) x += proj[at + (size_t)s * split_stride];
        out[i] = act ? x / (1.f + expf(-x)) : x;
    }
}

extern "C" int qt_linear_attention_prepare(const float* proj, int n_splits, long long split_stride, int proj_cols, int cols, float* out, int n_tokens,
                                           int act, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && cols > 0 && cols <= proj_cols && n_splits >= 1, "linear_attention_prepare: %d of %d columns", cols, proj_cols);
    if (n_tokens == 0) return QT_OK;
    const long long total = (long long)n_tokens * cols;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    launch_kernel(linear_attention_prepare_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, proj, n_splits, (size_t)split_stride, proj_cols,
                  cols, out, total, act);
    QT_CHECK_LAUNCH("linear_attention_prepare");
    return QT_OK;
}

// COLS columns of a head's state per block (COLS * 8 threads).  A chunk's q, k and v are fetched into registers while the
// chunk before is worked on (every load of a chunk is issued before the first is used), pass SiLU where asked and go to
// shared memory behind a barrier.
template <int RPL, int COLS>
__global__ void __launch_bounds__(COLS * LA_LANES) linear_attention_scan_kernel(const LinAttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int THREADS = COLS * LA_LANES;
    constexpr int STRIDE = LA_LANES * (RPL + 4);          // a token's q (or k) row in shared memory: 4 floats of padding per lane's
    constexpr int ROW = LA_LANES * RPL;                   // piece, so that the 8 lanes' 16-byte reads fall on different banks
    constexpr int QK_PER = LA_CHUNK * ROW / THREADS;      // q (and k) elements of a chunk per thread
    constexpr int V_PER = LA_CHUNK * COLS / THREADS;      // v elements of a chunk per thread (2)
    __shared__ __align__(16) float qs[LA_CHUNK * STRIDE];
    __shared__ __align__(16) float ks[LA_CHUNK * STRIDE];
    __shared__ float vs[LA_CHUNK * COLS];
    const int head = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x % LA_LANES, col_in_block = threadIdx.x / LA_LANES;
    const int col = blockIdx.x * COLS + col_in_block;
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
    float qr[QK_PER], kr[QK_PER], vr[V_PER];
    auto fetch = [&](int t0) {                             // the chunk from token t0 on, into registers
        const int count = min(LA_CHUNK, end - t0);
#pragma unroll
        for (int j = 0; j < QK_PER; ++j) {
            const int i = threadIdx.x + j * THREADS, tok = i / ROW, r = i % ROW;
            const bool has = tok < count && r < p.dim;
            const size_t row = (size_t)(t0 + tok) * p.proj_cols + (size_t)head * p.dim + r;
            qr[j] = has ? la_raw(p, row + p.at_q) : 0.f;
            kr[j] = has ? la_raw(p, row + p.at_k) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < V_PER; ++j) {
            const int i = threadIdx.x + j * THREADS, tok = i / COLS, c = blockIdx.x * COLS + i % COLS;
            vr[j] = (tok < count && c < p.vdim) ? la_raw(p, (size_t)(t0 + tok) * p.proj_cols + p.at_v + (size_t)head * p.vdim + c) : 0.f;
        }
    };
    fetch(begin);
    for (int t0 = begin; t0 < end; t0 += LA_CHUNK) {
        const int count = min(LA_CHUNK, end - t0);
        __syncthreads();                                   // the chunk before has been read
#pragma unroll
        for (int j = 0; j < QK_PER; ++j) {
            const int i = threadIdx.x + j * THREADS, tok = i / ROW, r = i % ROW;
            const int at = tok * STRIDE + (r / RPL) * (RPL + 4) + r % RPL;
            qs[at] = la_act(p, qr[j]);
            ks[at] = la_act(p, kr[j]);
        }
#pragma unroll
        for (int j = 0; j < V_PER; ++j) vs[threadIdx.x + j * THREADS] = la_act(p, vr[j]);
        __syncthreads();
        if (t0 + LA_CHUNK < end) fetch(t0 + LA_CHUNK);     // in flight while this chunk is worked on
#pragma unroll 2
        for (int tok = 0; tok < count; ++tok) {
            const float v = vs[tok * COLS + col_in_block];
            const float* qrow = qs + tok * STRIDE + lane * (RPL + 4);
            const float* krow = ks + tok * STRIDE + lane * (RPL + 4);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(krow + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qrow + i);
                S[i] = fmaf(decay, S[i], k4.x * v);         a0 = fmaf(S[i], q4.x, a0);
                S[i + 1] = fmaf(decay, S[i + 1], k4.y * v); a1 = fmaf(S[i + 1], q4.y, a1);
                S[i + 2] = fmaf(decay, S[i + 2], k4.z * v); a2 = fmaf(S[i + 2], q4.z, a2);
                S[i + 3] = fmaf(decay, S[i + 3], k4.w * v); a3 = fmaf(S[i + 3], q4.w, a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
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

// Steps in which no sequence brings more than a few tokens (one-token steps above all): nothing is staged or fetched
// ahead, a thread reads its rows' q and k from the projection itself (the 32 columns of a block read the same ones, from
// L1), so the kernel is short and light in registers and many blocks share an SM; its cost is the state's bytes.
template <int RPL>
__global__ void __launch_bounds__(32 * LA_LANES) linear_attention_step_kernel(const LinAttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x % LA_LANES, col = blockIdx.x * 32 + threadIdx.x / LA_LANES;
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
    const bool quads = p.n_splits == 1 && p.dim % 4 == 0 && p.at_q % 4 == 0 && p.at_k % 4 == 0 && p.proj_cols % 4 == 0 && ((uintptr_t)p.proj & 15) == 0;
    for (int t = begin; t < end; ++t) {
        const size_t row = (size_t)t * p.proj_cols;
        const float v = live ? la_act(p, la_raw(p, row + p.at_v + (size_t)head * p.vdim + col)) : 0.f;
        float q[RPL], k[RPL];
        const size_t q_at = row + p.at_q + (size_t)head * p.dim + row0, k_at = row + p.at_k + (size_t)head * p.dim + row0;
        if (quads) {                                        // 16-byte loads of a row that is finished and aligned
#pragma unroll
            for (int i = 0; i < RPL; i += 4) {
                const bool has = row0 + i < p.dim;
                const float4 q4 = has ? __ldg(reinterpret_cast<const float4*>(p.proj + q_at + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 k4 = has ? __ldg(reinterpret_cast<const float4*>(p.proj + k_at + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
                q[i] = q4.x; q[i + 1] = q4.y; q[i + 2] = q4.z; q[i + 3] = q4.w;
                k[i] = k4.x; k[i + 1] = k4.y; k[i + 2] = k4.z; k[i + 3] = k4.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < RPL; ++i) {                 // every load of the token ahead of its arithmetic
                const bool has = row0 + i < p.dim;
                q[i] = has ? la_raw(p, q_at + i) : 0.f;
                k[i] = has ? la_raw(p, k_at + i) : 0.f;
            }
        }
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPL; i += 2) {
            S[i] = fmaf(decay, S[i], la_act(p, k[i]) * v);             a0 = fmaf(S[i], la_act(p, q[i]), a0);
            S[i + 1] = fmaf(decay, S[i + 1], la_act(p, k[i + 1]) * v); a1 = fmaf(S[i + 1], la_act(p, q[i + 1]), a1);
        }
        float acc = a0 + a1;
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (lane == 0 && live) p.out[((size_t)t * p.heads + head) * p.vdim + col] = acc;
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

// The same recurrence with a whole warp per column, for a step that brings one long portion or few of them: lane l holds the
// column's rows i * 128 + 4 l + e (i < NV, e < 4), so a token is a shorter chain of instructions per warp and an SM holds
// four times the warps, which is what hides a chain's latencies when there are few columns to go round.  Every warp
// reads the whole q and k of a token from shared memory, so this form moves four times the shared-memory bytes of the
// one above: it loses where the blocks of the other form fill the machine.
constexpr int LW_COLS = 8;         // state columns per block, one warp each
constexpr int LW_THREADS = LW_COLS * 32;

template <int NV>
__global__ void __launch_bounds__(LW_THREADS) linear_attention_scan_warp_kernel(const LinAttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int ROW = NV * 128;                         // a token's q (or k) row in shared memory, zeros beyond dim
    constexpr int QK_PER = LA_CHUNK * ROW / LW_THREADS;   // q (and k) elements of a chunk per thread
    __shared__ __align__(16) float qs[LA_CHUNK * ROW];
    __shared__ __align__(16) float ks[LA_CHUNK * ROW];
    __shared__ float vs[LA_CHUNK * LW_COLS];
    const int head = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * LW_COLS + warp;
    const int begin = p.seq_start[seq], end = p.seq_start[seq + 1];
    if (begin >= end) return;
    const float decay = p.decay[head];
    const bool live = col < p.vdim;
    float* state = p.state + (((size_t)p.slots[seq] * p.heads + head) * p.vdim + (live ? col : 0)) * p.dim;
    const bool vec = p.dim % 4 == 0 && ((uintptr_t)p.state & 15) == 0;
    float S[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int r = i * 128 + 4 * lane;
        S[i][0] = S[i][1] = S[i][2] = S[i][3] = 0.f;
        if (!live) continue;
        if (vec) {
            if (r < p.dim) { const float4 v = *reinterpret_cast<const float4*>(state + r); S[i][0] = v.x; S[i][1] = v.y; S[i][2] = v.z; S[i][3] = v.w; }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (r + e < p.dim) S[i][e] = state[r + e];
        }
    }
    float qr[QK_PER], kr[QK_PER], vr = 0.f;
    auto fetch = [&](int t0) {                             // the chunk from token t0 on, into registers
        const int count = min(LA_CHUNK, end - t0);
#pragma unroll
        for (int j = 0; j < QK_PER; ++j) {
            const int i = threadIdx.x + j * LW_THREADS, tok = i / ROW, r = i % ROW;
            const bool has = tok < count && r < p.dim;
            const size_t row = (size_t)(t0 + tok) * p.proj_cols + (size_t)head * p.dim + r;
            qr[j] = has ? la_raw(p, row + p.at_q) : 0.f;
            kr[j] = has ? la_raw(p, row + p.at_k) : 0.f;
        }
        if (threadIdx.x < LA_CHUNK * LW_COLS) {
            const int tok = threadIdx.x / LW_COLS, c = blockIdx.x * LW_COLS + threadIdx.x % LW_COLS;
            vr = (tok < count && c < p.vdim) ? la_raw(p, (size_t)(t0 + tok) * p.proj_cols + p.at_v + (size_t)head * p.vdim + c) : 0.f;
        }
    };
    fetch(begin);
    for (int t0 = begin; t0 < end; t0 += LA_CHUNK) {
        const int count = min(LA_CHUNK, end - t0);
        __syncthreads();                                   // the chunk before has been read
#pragma unroll
        for (int j = 0; j < QK_PER; ++j) {
            qs[threadIdx.x + j * LW_THREADS] = la_act(p, qr[j]);
            ks[threadIdx.x + j * LW_THREADS] = la_act(p, kr[j]);
        }
        if (threadIdx.x < LA_CHUNK * LW_COLS) vs[threadIdx.x] = la_act(p, vr);
        __syncthreads();
        if (t0 + LA_CHUNK < end) fetch(t0 + LA_CHUNK);     // in flight while this chunk is worked on
#pragma unroll 4
        for (int tok = 0; tok < count; ++tok) {
            const float v = vs[tok * LW_COLS + warp];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + tok * ROW + i * 128 + 4 * lane);
                const float4 q4 = *reinterpret_cast<const float4*>(qs + tok * ROW + i * 128 + 4 * lane);
                S[i][0] = fmaf(decay, S[i][0], k4.x * v); a0 = fmaf(S[i][0], q4.x, a0);
                S[i][1] = fmaf(decay, S[i][1], k4.y * v); a1 = fmaf(S[i][1], q4.y, a1);
                S[i][2] = fmaf(decay, S[i][2], k4.z * v); a2 = fmaf(S[i][2], q4.z, a2);
                S[i][3] = fmaf(decay, S[i][3], k4.w * v); a3 = fmaf(S[i][3], q4.w, a3);
            }
            const float acc = warp_sum((a0 + a1) + (a2 + a3));
            if (lane == 0 && live) p.out[((size_t)(t0 + tok) * p.heads + head) * p.vdim + col] = acc;
        }
    }
    if (!live) return;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int r = i * 128 + 4 * lane;
        if (vec) {
            if (r < p.dim) *reinterpret_cast<float4*>(state + r) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (r + e < p.dim) state[r + e] = S[i][e];
        }
    }
}

extern "C" int qt_linear_attention_scan(const float* proj, int n_splits, long long split_stride, int proj_cols, int at_q, int at_k, int at_v,
                                        const float* decay, float* state, float* out, const int* seq_start, const int* slots, int n_seqs,
                                        int heads, int dim, int vdim, int act, int max_q_len, void* stream) {
    QT_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0 && n_splits >= 1, "linear_attention_scan: bad sizes B=%d H=%d dim=%d vdim=%d", n_seqs, heads, dim, vdim);
    QT_REQUIRE(dim <= LA_LANES * 32, "linear_attention_scan: %d key channels per head are beyond what a column's lanes hold (%d)", dim, LA_LANES * 32);
    QT_REQUIRE(at_q >= 0 && at_k >= 0 && at_v >= 0 && at_q + heads * dim <= proj_cols && at_k + heads * dim <= proj_cols && at_v + heads * vdim <= proj_cols,
               "linear_attention_scan: q, k or v columns outside the projection's %d", proj_cols);
    if (n_seqs == 0) return QT_OK;
    LinAttnParams p{proj, n_splits, (size_t)split_stride, proj_cols, at_q, at_k, at_v, decay, state, out, seq_start, slots, heads, dim, vdim, act};
    cudaStream_t s = (cudaStream_t)stream;
    // blocks of 32 columns where they fill the machine twice over (many sequences: every block stages its head's q and k
    // itself), else of 16, so that one prompt still gives most SMs a block
    const bool wide = (long long)((vdim + 31) / 32) * heads * n_seqs >= 2LL * sm_count();
    if (max_q_len <= 4) {                                  // few tokens a sequence: the short kernel
        const dim3 grid((vdim + 31) / 32, heads, n_seqs), block(32 * LA_LANES);
        if (dim <= LA_LANES * 8) launch_kernel(linear_attention_step_kernel<8>, grid, block, 0, s, p);
        else if (dim <= LA_LANES * 16) launch_kernel(linear_attention_step_kernel<16>, grid, block, 0, s, p);
        else launch_kernel(linear_attention_step_kernel<32>, grid, block, 0, s, p);
        QT_CHECK_LAUNCH("linear_attention_scan");
        return QT_OK;
    }
    // long portions of few sequences, with a head's rows within what 32 lanes hold four at a time: a warp per column
    static const bool warp_form = [] { const char* env = getenv("QT_B200_LINEAR_WARP"); return !(env && env[0] == '0'); }();
    if (warp_form && max_q_len >= 64 && dim > 64 && (long long)((vdim + 15) / 16) * heads * n_seqs < 2LL * sm_count()) {
        const dim3 grid((vdim + LW_COLS - 1) / LW_COLS, heads, n_seqs), block(LW_THREADS);
        if (dim <= 128) launch_kernel(linear_attention_scan_warp_kernel<1>, grid, block, 0, s, p);
        else launch_kernel(linear_attention_scan_warp_kernel<2>, grid, block, 0, s, p);
        QT_CHECK_LAUNCH("linear_attention_scan");
        return QT_OK;
    }
#define QT_LAUNCH_LA(RPL)                                                                                                              \
    do {                                                                                                                               \
        if (wide) launch_kernel(linear_attention_scan_kernel<RPL, 32>, dim3((vdim + 31) / 32, heads, n_seqs), dim3(32 * LA_LANES), 0, s, p); \
        else launch_kernel(linear_attention_scan_kernel<RPL, 16>, dim3((vdim + 15) / 16, heads, n_seqs), dim3(16 * LA_LANES), 0, s, p);      \
    } while (0)
    if (dim <= LA_LANES * 8) QT_LAUNCH_LA(8);
    else if (dim <= LA_LANES * 16) QT_LAUNCH_LA(16);
    else QT_LAUNCH_LA(32);
#undef QT_LAUNCH_LA
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
