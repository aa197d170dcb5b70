// Layer norm (with or without bias) around the float residual stream, and an activation on a product's sums.
//
// add_layernorm_kernel: one block per output row r, src = rows ? rows[r] : r.
//   d = sum_s delta[s][src]                                   (float; split-K partial sums added in their order)
//   if (post_weight) d = (d - mean(d)) / sqrt(var(d) + eps) * post_weight (+ post_bias)   (a norm on the sublayer's output)
//   x = residual[src] + d;  if (!rows) residual[src] = x      (the stream is updated in place)
//   out[r] = (x - mean(x)) / sqrt(var(x) + eps) * weight (+ bias)     (rounded once to the output type)
//   without `weight`: out[r] = x                              (a sublayer that reads the stream itself)
// The variance is the mean of the squared deviations from the mean, taken in a second pass over the row, which the
// block keeps in shared memory.  A layer that norms what a sublayer returns before adding it, and norms the stream
// again for the next sublayer, is one launch per sublayer.
//
// activation_kernel: out = act(sum_s in[s]) elementwise, for a feed-forward of two matrices with no gate.
#include "common.cuh"

#include <math.h>

using namespace qt;

template <typename TD, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_splits, size_t split_stride,
                                     const float* __restrict__ post_weight, const float* __restrict__ post_bias,
                                     const float* __restrict__ weight, const float* __restrict__ bias, float eps,
                                     TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row[];            // [hidden]
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * hidden;
    const float inv_n = 1.f / (float)hidden;
    if (delta) {
        float sum = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float d = load_sum(delta, (size_t)src * hidden + i, n_splits, split_stride);
            row[i] = d;
            sum += d;
        }
        if (post_weight) {
            const float mean = block_sum(sum, scratch) * inv_n;
            float sq = 0.f;
            for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
                const float c = row[i] - mean;
                sq += c * c;
            }
            const float inv = rsqrtf(block_sum(sq, scratch) * inv_n + eps);
            for (int i = threadIdx.x; i < hidden; i += blockDim.x) row[i] = (row[i] - mean) * inv * post_weight[i] + (post_bias ? post_bias[i] : 0.f);
        }
    }
    float sum = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float x = res[i] + (delta ? row[i] : 0.f);
        row[i] = x;
        if (!rows) res[i] = x;
        sum += x;
    }
    TO* o = out + (size_t)r * hidden;
    if (!weight) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TO>(row[i]);      // each thread reads what it wrote
        return;
    }
    const float mean = block_sum(sum, scratch) * inv_n;
    float sq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float c = row[i] - mean;
        sq += c * c;
    }
    const float inv = rsqrtf(block_sum(sq, scratch) * inv_n + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TO>((row[i] - mean) * inv * weight[i] + (bias ? bias[i] : 0.f));
}

// The same for rows of up to 4,096 elements whose length and strides are multiples of four: a thread holds four elements
// of the row in registers (16-byte loads of the sums and the stream, all issued before the first sum is needed; 8- or
// 16-byte stores), and the row never passes through shared memory.  Every element is summed over the splits in the same
// order as above.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TD, typename TO>
__global__ void add_layernorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_splits, size_t split_stride,
                                         const float* __restrict__ post_weight, const float* __restrict__ post_bias,
                                         const float* __restrict__ weight, const float* __restrict__ bias, float eps,
                                         TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * hidden;
    const float inv_n = 1.f / (float)hidden;
    const int i = threadIdx.x;
    const bool has = i < (hidden >> 2);              // a thread holds one quad of the row in registers (blockDim.x >= hidden / 4)
    // everything the thread reads is asked for at once: the sums, the stream and both weights
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f), d = x, w = x, pw = x, b = x, pb = x;
    if (has) {
        x = load4(res + 4 * i);
        if (weight) w = load4(weight + 4 * i);
        if (bias) b = load4(bias + 4 * i);
        if (post_weight) pw = load4(post_weight + 4 * i);
        if (post_bias) pb = load4(post_bias + 4 * i);
        if (delta) {
            const TD* at = delta + (size_t)src * hidden + 4 * i;
            d = load4(at);
            for (int s = 1; s < n_splits; ++s) {
                const float4 e = load4(at + (size_t)s * split_stride);
                d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
            }
        }
    }
    if (delta && post_weight) {
        const float mean = block_sum((d.x + d.y) + (d.z + d.w), scratch) * inv_n;
        const float a = d.x - mean, g = d.y - mean, c = d.z - mean, e = d.w - mean;
        const float inv = rsqrtf(block_sum(has ? (a * a + g * g) + (c * c + e * e) : 0.f, scratch) * inv_n + eps);
        d = make_float4(a * inv * pw.x + pb.x, g * inv * pw.y + pb.y, c * inv * pw.z + pb.z, e * inv * pw.w + pb.w);
    }
    if (delta) { x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w; }
    if (!rows && has) store4(res + 4 * i, x);
    if (!weight) {
        if (has) store4(out + (size_t)r * hidden + 4 * i, x);
        return;
    }
    const float mean = block_sum((x.x + x.y) + (x.z + x.w), scratch) * inv_n;
    const float a = x.x - mean, g = x.y - mean, c = x.z - mean, e = x.w - mean;
    const float inv = rsqrtf(block_sum(has ? (a * a + g * g) + (c * c + e * e) : 0.f, scratch) * inv_n + eps);
    if (has) store4(out + (size_t)r * hidden + 4 * i, make_float4(a * inv * w.x + b.x, g * inv * w.y + b.y, c * inv * w.z + b.z, e * inv * w.w + b.w));
}

extern "C" int qt_add_layernorm(float* residual, const void* delta, int delta_dtype, int n_splits, long long split_stride,
                                const float* post_weight, const float* post_bias, const float* weight, const float* bias, float eps,
                                void* out, int out_dtype, const int* rows, int n_rows, int hidden, void* stream) {
    QT_REQUIRE(n_rows >= 0 && hidden > 0 && n_splits >= 1, "add_layernorm: bad sizes rows=%d H=%d splits=%d", n_rows, hidden, n_splits);
    QT_REQUIRE(eps > 0.f, "add_layernorm: eps must be positive");
    QT_REQUIRE(delta || !post_weight, "add_layernorm: a norm on an addition that is not there");
    QT_REQUIRE((post_weight || !post_bias) && (weight || !bias), "add_layernorm: a bias without its weight");
    if (n_rows == 0) return QT_OK;
    const size_t smem = (size_t)hidden * sizeof(float);
    QT_REQUIRE(smem <= 200 * 1024, "add_layernorm: a row of %d elements does not fit shared memory", hidden);
    cudaStream_t s = (cudaStream_t)stream;
    int threads = ((hidden + 3) / 4 + 31) / 32 * 32;
    threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
    // rows of at most 1,024 whole quads whose every pointer and stride keeps 16-byte alignment go four elements a thread
    const auto misaligned = [](const void* ptr) { return ((uintptr_t)ptr & 15) != 0; };
    const bool vec = hidden % 4 == 0 && hidden <= 4 * threads && split_stride % 4 == 0 && !misaligned(residual) && !misaligned(delta) && !misaligned(post_weight) &&
                     !misaligned(weight) && !misaligned(out) && !misaligned(bias) && !misaligned(post_bias);
#define QT_LAUNCH_LN(TD, TO)                                                                                                        \
    do {                                                                                                                            \
        if (smem > 48 * 1024) {                                                                                                     \
            cudaError_t err = cudaFuncSetAttribute(add_layernorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "add_layernorm: cannot raise shared memory: %s", cudaGetErrorString(err)); \
        }                                                                                                                           \
        if (vec)                                                                                                                    \
            launch_kernel(add_layernorm_vec_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, s, residual, (const TD*)delta, n_splits, \
                          (size_t)split_stride, post_weight, post_bias, weight, bias, eps, (TO*)out, rows, hidden);                                  \
        else                                                                                                                        \
            launch_kernel(add_layernorm_kernel<TD, TO>, dim3(n_rows), dim3(threads), smem, s, residual, (const TD*)delta, n_splits, \
                          (size_t)split_stride, post_weight, post_bias, weight, bias, eps, (TO*)out, rows, hidden);                                  \
    } while (0)
    if (delta_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_LN(float, float);
    else if (delta_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_LN(float, __nv_bfloat16);
    else if (delta_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_LN(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == QT_BF16 && out_dtype == QT_F32) QT_LAUNCH_LN(__nv_bfloat16, float);
    else QT_FAIL(QT_ERR_ARG, "add_layernorm: unknown element types %d/%d", delta_dtype, out_dtype);
#undef QT_LAUNCH_LN
    QT_CHECK_LAUNCH("add_layernorm");
    return QT_OK;
}

// ----------------------------------------------------------------------------- activation on a product's sums
template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ in, int n_splits, size_t split_stride, TO* __restrict__ out, long long total, int act) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_float<TO>(gate_activation<false>(load_sum(in, (size_t)i, n_splits, split_stride), act));
}

// Four elements a thread, for totals, strides and pointers that keep the alignment of a quad.
template <typename TI, typename TO>
__global__ void activation_vec_kernel(const TI* __restrict__ in, int n_splits, size_t split_stride, TO* __restrict__ out, long long quads, int act) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (long long)gridDim.x * blockDim.x) {
        float4 v = load4(in + 4 * i);
        for (int s = 1; s < n_splits; ++s) {
            const float4 e = load4(in + 4 * i + (size_t)s * split_stride);
            v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
        }
        store4(out + 4 * i, make_float4(gate_activation<false>(v.x, act), gate_activation<false>(v.y, act), gate_activation<false>(v.z, act),
                                        gate_activation<false>(v.w, act)));
    }
}

extern "C" int qt_activation(const void* in, int in_dtype, int n_splits, long long split_stride, void* out, int out_dtype, int n_rows,
                             int cols, int act, void* stream) {
    QT_REQUIRE(n_rows >= 0 && cols > 0 && n_splits >= 1, "activation: bad sizes rows=%d cols=%d splits=%d", n_rows, cols, n_splits);
    QT_REQUIRE(act >= 0 && act < QT_ACT_COUNT, "activation: unknown activation code %d", act);
    if (n_rows == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n_rows * cols;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    const bool vec = total % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0;
    if (vec) blocks = (total / 4 + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
#define QT_LAUNCH_ACT(TI, TO)                                                                                                        \
    do {                                                                                                                             \
        if (vec) launch_kernel(activation_vec_kernel<TI, TO>, dim3((unsigned)blocks), dim3(256), 0, s, (const TI*)in, n_splits,       \
                               (size_t)split_stride, (TO*)out, total / 4, act);                                                      \
        else launch_kernel(activation_kernel<TI, TO>, dim3((unsigned)blocks), dim3(256), 0, s, (const TI*)in, n_splits,              \
                           (size_t)split_stride, (TO*)out, total, act);                                                              \
    } while (0)
    if (in_dtype == QT_F32 && out_dtype == QT_F32) QT_LAUNCH_ACT(float, float);
    else if (in_dtype == QT_F32 && out_dtype == QT_BF16) QT_LAUNCH_ACT(float, __nv_bfloat16);
    else if (in_dtype == QT_BF16 && out_dtype == QT_BF16) QT_LAUNCH_ACT(__nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == QT_BF16 && out_dtype == QT_F32) QT_LAUNCH_ACT(__nv_bfloat16, float);
    else QT_FAIL(QT_ERR_ARG, "activation: unknown element types %d/%d", in_dtype, out_dtype);
#undef QT_LAUNCH_ACT
    QT_CHECK_LAUNCH("activation");
    return QT_OK;
}

// ----------------------------------------------------------------------------- a weighted sum of two products' sums
// out = wa * sum_s a[s] + wb * sum_s b[s], in float: two sublayers that run side by side on the same input and are
// mixed with two constants before anything else happens to them.
template <typename TA, typename TB>
__global__ void weighted_sum_kernel(const TA* __restrict__ a, int a_splits, size_t a_stride, float wa, const TB* __restrict__ b, int b_splits,
                                    size_t b_stride, float wb, float* __restrict__ out, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        out[i] = wa * load_sum(a, (size_t)i, a_splits, a_stride) + wb * load_sum(b, (size_t)i, b_splits, b_stride);
}

extern "C" int qt_weighted_sum(const void* a, int a_dtype, int a_splits, long long a_stride, float wa, const void* b, int b_dtype, int b_splits,
                               long long b_stride, float wb, float* out, long long total, void* stream) {
    QT_REQUIRE(total >= 0 && a_splits >= 1 && b_splits >= 1, "weighted_sum: bad sizes");
    if (total == 0) return QT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    long long blocks = (total + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
#define QT_LAUNCH_WS(TA, TB) launch_kernel(weighted_sum_kernel<TA, TB>, dim3((unsigned)blocks), dim3(256), 0, s, (const TA*)a, a_splits, (size_t)a_stride, wa, \
                                           (const TB*)b, b_splits, (size_t)b_stride, wb, out, total)
    if (a_dtype == QT_F32 && b_dtype == QT_F32) QT_LAUNCH_WS(float, float);
    else if (a_dtype == QT_F32 && b_dtype == QT_BF16) QT_LAUNCH_WS(float, __nv_bfloat16);
    else if (a_dtype == QT_BF16 && b_dtype == QT_F32) QT_LAUNCH_WS(__nv_bfloat16, float);
    else if (a_dtype == QT_BF16 && b_dtype == QT_BF16) QT_LAUNCH_WS(__nv_bfloat16, __nv_bfloat16);
    else QT_FAIL(QT_ERR_ARG, "weighted_sum: unknown element types %d/%d", a_dtype, b_dtype);
#undef QT_LAUNCH_WS
    QT_CHECK_LAUNCH("weighted_sum");
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(layernorm)
