// What stands between the first projection of an attention mixer whose queries and keys pass a short causal
// convolution over time, and its attention kernel; and the sigmoid gate on the heads' outputs behind it.
//
// conv_qk_write_kernel   y_t[c] = sum_j taps[c][j] * u_(t - n + 1 + j)[c] over the n taps of channel c, in float, where u
//                        are the projection's float sums (bias included) of this step's rows and, for positions before
//                        the step's first token, the sequence's kept inputs (zeros before the sequence's start).  The
//                        first nq * d channels are the queries (written to q_out), the next nkv * d the keys (written
//                        into the paged cache at the token's position).  Values are the keys, so nothing else is stored.
// conv_keep_kernel       kept[slot] <- the raw inputs of the sequence's last n - 1 positions after this step.
// gate_mul_kernel        x[t][c] *= sigmoid(sum_s gate[s][t][offset + c]): a gate computed from the mixer's input by one
//                        more block of rows of the first projection.  With `group` > 1 every `group` consecutive
//                        columns share one gate column (one number per head).
#include "common.cuh"

#include <math.h>

using namespace qt;

constexpr int MAX_TAPS = 16;

struct ConvParams {
    const float* proj; int n_splits; size_t split_stride; int proj_cols;   // [splits, T, proj_cols]; columns: q | k | ...
    const float* taps;                // [channels, n_taps], the last column is the current token's
    const float* kept;                // [slots + 1, n_taps - 1, channels]
    const int* token_seq; const int* token_pos; const int* seq_start; const int* slots;
    void* q_out;                      // [T, nq, d]
    void* k_cache;                    // [pages, nkv, page_tokens, d]
    const int* block_table; int max_blocks;
    int n_tokens, nq, nkv, d, n_taps, page_tokens, ring_tokens, write_kv;
};

__device__ __forceinline__ float sum_splits(const float* __restrict__ base, size_t index, int n_splits, size_t split_stride) {
    float acc = base[index];
    for (int s = 1; s < n_splits; ++s) acc += base[index + (size_t)s * split_stride];
    return acc;
}

// grid (channel blocks, tokens)
template <typename TO>
__global__ void __launch_bounds__(128) conv_qk_write_kernel(const ConvParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int q_channels = p.nq * p.d, channels = (p.nq + p.nkv) * p.d;
    if (c >= channels) return;
    const int seq = p.token_seq[t], pos = p.token_pos[t];
    const int row0 = p.seq_start[seq];
    const int local = t - row0;                                   // index among the step's tokens of this sequence
    const int rows = p.n_taps - 1;
    const float* mine = p.kept + (size_t)p.slots[seq] * rows * channels + c;
    float y = 0.f;
    for (int j = 0; j < p.n_taps; ++j) {
        const int from = local - rows + j;                        // negative: a position before this step
        const float u = from >= 0 ? sum_splits(p.proj, (size_t)(row0 + from) * p.proj_cols + c, p.n_splits, p.split_stride)
                                  : mine[(size_t)(rows + from) * channels];
        y += p.taps[(size_t)c * p.n_taps + j] * u;
    }
    if (c < q_channels) {
        ((TO*)p.q_out)[(size_t)t * q_channels + c] = from_float<TO>(y);
    } else if (p.write_kv) {
        const int kc = c - q_channels;
        const int* table = p.block_table + (size_t)seq * p.max_blocks;
        ((TO*)p.k_cache)[cache_offset(table, pos, p.ring_tokens, p.page_tokens, p.nkv, kc / p.d, p.d) + kc % p.d] = from_float<TO>(y);
    }
}

// One thread per (sequence, channel): it reads what it needs of the old rows before it writes.
__global__ void conv_keep_kernel(const float* __restrict__ proj, int n_splits, size_t split_stride, int proj_cols,
                                 float* __restrict__ kept, const int* __restrict__ seq_start, const int* __restrict__ slots,
                                 int channels, int n_taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int row0 = seq_start[seq], count = seq_start[seq + 1] - row0;
    const int rows = n_taps - 1;
    float* mine = kept + (size_t)slots[seq] * rows * channels + c;
    float value[MAX_TAPS];
    for (int j = 0; j < rows; ++j) {
        const int from = count - rows + j;
        value[j] = from >= 0 ? sum_splits(proj, (size_t)(row0 + from) * proj_cols + c, n_splits, split_stride)
                             : mine[(size_t)(rows + from) * channels];
    }
    for (int j = 0; j < rows; ++j) mine[(size_t)j * channels] = value[j];
}

extern "C" int qt_conv_qk_write(const float* proj, int n_splits, long long split_stride, int proj_cols, const float* taps, float* kept,
                                const int* token_seq, const int* token_pos, const int* seq_start, const int* slots, void* q_out,
                                void* k_cache, int out_dtype, const int* block_table, int max_blocks, int n_tokens, int n_seqs, int nq,
                                int nkv, int d, int n_taps, int page_tokens, int ring_tokens, int write_kv, void* stream) {
    QT_REQUIRE(n_tokens >= 0 && n_seqs >= 0 && nq > 0 && nkv > 0 && d > 0 && n_splits >= 1, "conv_qk_write: bad sizes");
    QT_REQUIRE(n_taps >= 1 && n_taps <= MAX_TAPS, "conv_qk_write: %d taps (1..%d)", n_taps, MAX_TAPS);
    QT_REQUIRE((nq + nkv) * d <= proj_cols, "conv_qk_write: %d channels in a projection of %d columns", (nq + nkv) * d, proj_cols);
    QT_REQUIRE(!write_kv || (k_cache && block_table), "conv_qk_write: no cache to write the keys to");
    QT_REQUIRE(n_tokens <= 65535 && n_seqs <= 65535, "conv_qk_write: too many tokens or sequences for one launch");
    if (n_tokens == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int channels = (nq + nkv) * d;
    ConvParams p{proj, n_splits, (size_t)split_stride, proj_cols, taps, kept, token_seq, token_pos, seq_start, slots, q_out, k_cache,
                 block_table, max_blocks, n_tokens, nq, nkv, d, n_taps, page_tokens, ring_tokens, write_kv};
    int rc = QT_DISPATCH_DTYPE(out_dtype, "conv_qk_write", {
        launch_kernel(conv_qk_write_kernel<T>, dim3((channels + 127) / 128, n_tokens), dim3(128), 0, s, p);
        QT_CHECK_LAUNCH("conv_qk_write");
        return QT_OK;
    });
    if (rc) return rc;
    if (n_taps > 1) {
        launch_kernel(conv_keep_kernel, dim3((channels + 127) / 128, n_seqs), dim3(128), 0, s, proj, n_splits, (size_t)split_stride, proj_cols,
                      kept, seq_start, slots, channels, n_taps);
        QT_CHECK_LAUNCH("conv_keep");
    }
    return QT_OK;
}

// ----------------------------------------------------------------------------- sigmoid gate on the heads' outputs
template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ x, const float* __restrict__ gate, int n_splits, size_t split_stride, int gate_cols,
                                int gate_offset, long long total, int cols, int group) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols;
        const int c = (int)(i % cols);
        const float g = sum_splits(gate, (size_t)t * gate_cols + gate_offset + c / group, n_splits, split_stride);
        x[i] = from_float<T>(to_float(x[i]) / (1.f + expf(-g)));
    }
}

extern "C" int qt_gate_mul(void* x, int dtype, const float* gate, int n_splits, long long split_stride, int gate_cols, int gate_offset,
                           int n_rows, int cols, int group, void* stream) {
    if (group <= 0) group = 1;
    QT_REQUIRE(n_rows >= 0 && cols > 0 && gate_offset >= 0 && gate_offset + (cols + group - 1) / group <= gate_cols && n_splits >= 1,
               "gate_mul: %d columns at %d of %d", cols, gate_offset, gate_cols);
    if (n_rows == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n_rows * cols;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    return QT_DISPATCH_DTYPE(dtype, "gate_mul", {
        launch_kernel(gate_mul_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, s, (T*)x, gate, n_splits, (size_t)split_stride, gate_cols,
                      gate_offset, total, cols, group);
        QT_CHECK_LAUNCH("gate_mul");
        return QT_OK;
    });
}

QT_DEFINE_LAST_ERROR(short_conv)
