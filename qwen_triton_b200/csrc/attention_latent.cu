// bfloat16 attention over cached latent rows on the tensor cores (mma.sync m16n8k16, float accumulation).
//
// The cache holds one row of `row` elements per token and all heads read it: a head's query is as long as the row
// (its first `rank` elements meet the latent, the rest the shared rotated key part) and the values are the row's first
// `rank` elements.  Because every head reads the same keys, the rows of a query tile are (token, head) pairs: a block takes
// 64 consecutive pairs of one sequence (64 / heads tokens of a prompt, or the heads of a one-token step) and walks the
// pages of 64 tokens its rows can see through a two-stage cp.async ring, so a page is read once for all heads.
//
// Eight warps: warp w owns rows 16 (w / 2) .. + 15 and the value columns of half (w % 2).  The two warps of a row group
// form the scores of 32 keys of the page each (the query fragments come from shared memory by ldmatrix at every step of
// the sum, a row being too long for registers), hand each other the row maxima and then the weights through shared
// memory (two barriers of 64 threads a page), keep the same online softmax, in float in the base-2 domain, and each
// multiplies all 64 weights with its half of the value columns.  With `n_splits` > 1 the pages of a sequence are cut into
// that many ranges, one block each, whose partial results go to float scratch and are merged by the combine kernel that
// the other decode kernels use.  (Where a page's keys are cut among the row groups, see the kernel, both warps of a row
// group still form the same scores.)
//
// Causal: the key at position j is visible to the query at position i iff j <= i.  Takes rows and ranks that are
// multiples of 8 (shared-memory rows are padded with zeros to the next multiple of 16), ranks up to 512, a positive
// scale and pages of 64 tokens; the generic kernels of attention.cu take everything else.
#include "attention_mma.cuh"

using namespace qt;
using namespace qt_mma;

namespace {

struct LatentParams {
    const __nv_bfloat16* q;        // [T, heads, row]
    const __nv_bfloat16* cache;    // [pages, 1, 64, row]
    __nv_bfloat16* out;            // [T, heads, rank]
    const int* block_table; int max_blocks;
    const int* seq_start; const int* seq_past;   // prompts: packed sequences with a past (seq_len null)
    const int* seq_len;                          // one-token steps: keys each sequence sees, its own included
    int heads, row, rank;
    float scale;
    int n_splits; float* part_acc; float* part_ml;
};

constexpr int LT_ROWS = 64;
constexpr int LT_THREADS = 256;

// Copy of a [64, row] page into shared-memory rows of lds elements by the whole block, 16 bytes per cp.async.
__device__ __forceinline__ void copy_page(uint32_t dst, const __nv_bfloat16* src, int row, int lds, int tid) {
    const int chunks = row >> 3, pieces = PAGE * chunks;
    int r = tid / chunks, c = tid % chunks;
    const int dr = LT_THREADS / chunks, dc = LT_THREADS % chunks;
    for (int i = tid; i < pieces; i += LT_THREADS) {
        cp_async16(dst + (uint32_t)(r * lds + c * 8) * 2u, src + (size_t)r * row + c * 8);
        r += dr; c += dc;
        if (c >= chunks) { c -= chunks; ++r; }
    }
}

// NT_MAX: n8 tiles of value columns a warp may hold.  KP: parts into which the keys of a page are cut among the row
// groups (1, 2 or 4).  With KP > 1 a block has 4 / KP row groups (16 or 32 rows, the heads of a one-token step) and row
// group r of part k walks keys 64 k / KP .. of every page with a softmax of its own; a part's result is one more
// partial result for the combine kernel: n_splits * KP per row, this block's at split * KP + k.
template <int NT_MAX, int KP>
__global__ void __launch_bounds__(LT_THREADS, 1) latent_attention_kernel(const LatentParams p) {
    constexpr int GROUPS = 4 / KP, BLOCK_ROWS = 16 * GROUPS, SNT = 8 / KP, KEYS = PAGE / KP;
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int row = p.row, rank = p.rank, heads = p.heads;
    const int ksteps = (row + 15) >> 4, lds = ksteps * 16 + PAD;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rg = (warp >> 1) % GROUPS, kpart = (warp >> 1) / GROUPS, cg = warp & 1, kb = kpart * KEYS;
    const int seq = blockIdx.z, split = blockIdx.y;
    const bool one_token = p.seq_len != nullptr;
    const int q_begin = one_token ? seq : p.seq_start[seq];
    const int q_len = one_token ? 1 : p.seq_start[seq + 1] - q_begin;
    const int past = one_token ? p.seq_len[seq] - 1 : p.seq_past[seq];
    const int total = q_len * heads;                       // (token, head) pairs of this sequence
    // a prompt's tiles in descending order: the last rows see the most keys, and the blocks that walk the most pages start first
    const int q0 = (one_token ? (int)blockIdx.x : (int)(gridDim.x - 1 - blockIdx.x)) * BLOCK_ROWS;
    if (q0 >= total) return;
    const int rows = min(BLOCK_ROWS, total - q0);
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    const int p_last = past + (q0 + rows - 1) / heads;     // below 0: a padded row of a captured step, which sees nothing

    const uint32_t tile_bytes = (uint32_t)PAGE * lds * 2u;
    const uint32_t q_s = smem_u32(smem_raw), kv0 = q_s + tile_bytes;
    if (row & 15) {                                        // the padding of the rows' sums must hold zeros
        for (int i = tid; i < (int)(3u * tile_bytes / 16u); i += LT_THREADS) reinterpret_cast<uint4*>(smem_raw)[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
    }
    const int n_tiles = p_last >= 0 ? p_last / PAGE + 1 : 0;
    const int per = (n_tiles + p.n_splits - 1) / p.n_splits;
    const int tile_begin = min(n_tiles, split * per), tile_end = min(n_tiles, tile_begin + per);

    {
        const int chunks = row >> 3;
        __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
        for (int i = tid; i < LT_ROWS * chunks; i += LT_THREADS) {
            const int r = i / chunks, c = i % chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)q_begin * heads + q0 + r) * row + c * 8);
            *reinterpret_cast<uint4*>(q_tile + r * lds + c * 8) = v;
        }
    }
    auto issue = [&](int tile) {
        if (tile < tile_end) copy_page(kv0 + (uint32_t)((tile - tile_begin) & 1) * tile_bytes, p.cache + (size_t)table[tile] * PAGE * row, row, lds, tid);
        cp_async_commit();
    };
    issue(tile_begin);

    // value columns of this warp: pairs of n8 tiles [pair0, pair0 + npairs)
    const int pairs = (rank + 15) >> 4, half = (pairs + 1) >> 1;
    const int pair0 = cg * half, npairs = max(0, min(half, pairs - pair0));
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[NT_MAX][4];
#pragma unroll
    for (int i = 0; i < NT_MAX; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const float scale2 = p.scale * LOG2E;
    const bool active = rg * 16 < rows;
    // absolute positions of this thread's two rows; rows beyond the tile's last act as its last row
    const int last_row = q0 + rows - 1;
    const int qpos[2] = {past + min(q0 + rg * 16 + g, last_row) / heads, past + min(q0 + rg * 16 + g + 8, last_row) / heads};
    const int warp_pos_min = past + min(q0 + rg * 16, last_row) / heads, warp_pos_max = past + min(q0 + rg * 16 + 15, last_row) / heads;
    const uint32_t q_frag = q_s + (uint32_t)((rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * lds + (lane >> 4) * 8) * 2u;
    const int mi = lane >> 3;
    const uint32_t k_frag = (uint32_t)((kb + (mi >> 1) * 8 + (lane & 7)) * lds + (mi & 1) * 8) * 2u;
    const uint32_t v_frag = (uint32_t)((kb + (mi & 1) * 8 + (lane & 7)) * lds + pair0 * 16 + (mi >> 1) * 8) * 2u;

    // KP == 1: what the two warps of a row group exchange.  xw[r]: the four floats of padding behind the query tile's row
    // of this thread's row r (maxima of the two warps, then their sums); p_rows: the row group's 16 x 64 weights, bfloat16.
    float* xw[2] = {reinterpret_cast<float*>(smem_raw + ((size_t)(rg * 16 + g) * lds + ksteps * 16) * 2),
                    reinterpret_cast<float*>(smem_raw + ((size_t)(rg * 16 + g + 8) * lds + ksteps * 16) * 2)};
    uint8_t* p_rows = smem_raw + 3 * (size_t)tile_bytes + (size_t)rg * 16 * PAGE * 2;
    const uint32_t p_frag = smem_u32(p_rows) + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * PAGE + (lane >> 4) * 8) * 2u;
    auto pair_sync = [](int group) { asm volatile("bar.sync %0, 64;" ::"r"(group + 1) : "memory"); };

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        issue(tile + 1);
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t k_s = kv0 + (uint32_t)((tile - tile_begin) & 1) * tile_bytes;
        const int pos0 = tile * PAGE + kb;                         // position of this warp's first key of the page
        if constexpr (KP == 1) {
            // The two warps of a row group form the scores of 32 keys each and hand each other the row maxima (through
            // the padding behind the rows of the query tile) and the weights (through p_s), so no score is formed twice.
            if (active && pos0 <= warp_pos_max) {
                const int kc = cg * 32;
                float s[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll 2
                for (int ks = 0; ks < ksteps; ++ks) {
                    uint32_t a[4];
                    ldmatrix_x4(a, q_frag + (uint32_t)ks * 32u);
#pragma unroll
                    for (int np = 0; np < 2; ++np) {
                        uint32_t b[4];
                        ldmatrix_x4(b, k_s + k_frag + (uint32_t)((kc + np * 16) * lds + ks * 16) * 2u);
                        mma_bf16(s[2 * np], a, b[0], b[1]);
                        mma_bf16(s[2 * np + 1], a, b[2], b[3]);
                    }
                }
                if (pos0 + PAGE - 1 > warp_pos_min) {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (pos0 + kc + nt * 8 + 2 * t + (e & 1) > qpos[e >> 1]) s[nt][e] = -INFINITY;
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    if (t == 0) xw[r][cg] = mx[r];
                }
                pair_sync(rg);
                float alpha[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], xw[r][cg ^ 1]);
                    const float m_new = fmaxf(m[r], mx[r] * scale2);
                    const float m_use = m_new == -INFINITY ? 0.f : m_new;
                    alpha[r] = fast_exp2(m[r] - m_use);
                    m[r] = m_new;
                    float sum = 0.f;
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        s[nt][2 * r] = fast_exp2(fmaf(s[nt][2 * r], scale2, -m_use));
                        s[nt][2 * r + 1] = fast_exp2(fmaf(s[nt][2 * r + 1], scale2, -m_use));
                        sum += s[nt][2 * r] + s[nt][2 * r + 1];
                        *reinterpret_cast<uint32_t*>(p_rows + ((g + 8 * r) * PAGE + kc + nt * 8 + 2 * t) * 2) = pack_bf16(s[nt][2 * r], s[nt][2 * r + 1]);
                    }
                    l[r] = l[r] * alpha[r] + sum;              // this warp's keys only; the halves meet after the last page
                }
                pair_sync(rg);
#pragma unroll
                for (int nt = 0; nt < NT_MAX; ++nt) { o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1]; }
#pragma unroll
                for (int j = 0; j < 4; ++j) {                        // 16 keys at a time: two steps of its own, two of the other warp's
                    uint32_t pa[4];
                    if ((j >> 1) == cg) {
                        const int jj = j & 1;
                        pa[0] = pack_bf16(s[2 * jj][0], s[2 * jj][1]); pa[1] = pack_bf16(s[2 * jj][2], s[2 * jj][3]);
                        pa[2] = pack_bf16(s[2 * jj + 1][0], s[2 * jj + 1][1]); pa[3] = pack_bf16(s[2 * jj + 1][2], s[2 * jj + 1][3]);
                    } else {
                        ldmatrix_x4(pa, p_frag + (uint32_t)j * 32u);
                    }
#pragma unroll
                    for (int nt2 = 0; nt2 < NT_MAX / 2; ++nt2) {
                        if (nt2 < npairs) {
                            uint32_t b[4];
                            ldmatrix_x4_trans(b, k_s + v_frag + (uint32_t)(j * 16 * lds + nt2 * 16) * 2u);
                            mma_bf16(o[2 * nt2], pa, b[0], b[1]);
                            mma_bf16(o[2 * nt2 + 1], pa, b[2], b[3]);
                        }
                    }
                }
            }
        } else if (active && pos0 <= warp_pos_max) {
            float s[SNT][4];
#pragma unroll
            for (int i = 0; i < SNT; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll 2
            for (int ks = 0; ks < ksteps; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, q_frag + (uint32_t)ks * 32u);
#pragma unroll
                for (int np = 0; np < SNT / 2; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, k_s + k_frag + (uint32_t)(np * 16 * lds + ks * 16) * 2u);
                    mma_bf16(s[2 * np], a, b[0], b[1]);
                    mma_bf16(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            if (pos0 + KEYS - 1 > warp_pos_min) {
#pragma unroll
                for (int nt = 0; nt < SNT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (pos0 + nt * 8 + 2 * t + (e & 1) > qpos[e >> 1]) s[nt][e] = -INFINITY;
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < SNT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r] * scale2);       // scale2 > 0: the max of the scaled scores
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                alpha[r] = fast_exp2(m[r] - m_use);
                m[r] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int nt = 0; nt < SNT; ++nt) {
                    s[nt][2 * r] = fast_exp2(fmaf(s[nt][2 * r], scale2, -m_use));
                    s[nt][2 * r + 1] = fast_exp2(fmaf(s[nt][2 * r + 1], scale2, -m_use));
                    sum += s[nt][2 * r] + s[nt][2 * r + 1];
                }
                l[r] = l[r] * alpha[r] + sum;
            }
#pragma unroll
            for (int nt = 0; nt < NT_MAX; ++nt) { o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1]; }
#pragma unroll
            for (int j = 0; j < SNT / 2; ++j) {                      // 16 keys at a time
                const uint32_t pa[4] = {pack_bf16(s[2 * j][0], s[2 * j][1]), pack_bf16(s[2 * j][2], s[2 * j][3]),
                                        pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]), pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3])};
#pragma unroll
                for (int nt2 = 0; nt2 < NT_MAX / 2; ++nt2) {
                    if (nt2 < npairs) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, k_s + v_frag + (uint32_t)(j * 16 * lds + nt2 * 16) * 2u);
                        mma_bf16(o[2 * nt2], pa, b[0], b[1]);
                        mma_bf16(o[2 * nt2 + 1], pa, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (!active) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    if constexpr (KP == 1) {                                    // the two warps' sums over their halves of the keys meet
        if (t == 0) { xw[0][2 + cg] = l[0]; xw[1][2 + cg] = l[1]; }
        pair_sync(rg);
        l[0] += xw[0][2 + (cg ^ 1)];
        l[1] += xw[1][2 + (cg ^ 1)];
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int local = rg * 16 + g + 8 * r;
        if (local >= rows) continue;
        const size_t pair = (size_t)q_begin * heads + q0 + local;      // (token, head) pair of the step
        if (p.n_splits * KP == 1) {
            const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
            __nv_bfloat16* dst = p.out + pair * rank;
#pragma unroll
            for (int nt = 0; nt < NT_MAX; ++nt) {
                const int col = pair0 * 16 + nt * 8 + 2 * t;
                if (nt < 2 * npairs && col < rank) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
            }
        } else {
            const size_t slot = pair * (p.n_splits * KP) + split * KP + kpart;
            float* dst = p.part_acc + slot * rank;
#pragma unroll
            for (int nt = 0; nt < NT_MAX; ++nt) {
                const int col = pair0 * 16 + nt * 8 + 2 * t;
                if (nt < 2 * npairs && col < rank) *reinterpret_cast<float2*>(dst + col) = make_float2(o[nt][2 * r], o[nt][2 * r + 1]);
            }
            if (cg == 0 && t == 0) { p.part_ml[slot * 2] = m[r] * LN2; p.part_ml[slot * 2 + 1] = l[r]; }   // natural-log domain for the combine kernel
        }
    }
}

template <typename K>
int raise_smem(K kernel, size_t bytes, const char* name) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err != cudaSuccess) QT_FAIL(QT_ERR_LAUNCH, "%s: cannot raise shared memory to %zu: %s", name, bytes, cudaGetErrorString(err));
    return QT_OK;
}

}  // namespace

// Prompts (seq_len null: packed sequences from seq_start and seq_past, max_q_len tokens at most) or one-token steps
// (seq_len given: one query token per sequence).
extern "C" int qt_attention_latent(const void* q, const void* cache, void* out, const int* block_table, int max_blocks,
                                   const int* seq_start, const int* seq_past, const int* seq_len, int n_seqs, int max_q_len,
                                   int heads, int row, int rank, int page_tokens, float scale, int n_splits, float* part_acc,
                                   float* part_ml, void* stream) {
    if (n_seqs == 0 || max_q_len == 0) return QT_OK;
    QT_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && heads > 0, "attention_latent: %d sequences, %d heads", n_seqs, heads);
    QT_REQUIRE(row >= 8 && row % 8 == 0 && rank >= 8 && rank % 8 == 0 && rank <= row && rank <= 512,
               "attention_latent: rows of %d with %d value elements (multiples of 8, values up to 512; use the generic kernel)", row, rank);
    QT_REQUIRE(page_tokens == PAGE, "attention_latent: pages of %d tokens (this kernel walks pages of %d)", page_tokens, PAGE);
    QT_REQUIRE(scale > 0.f, "attention_latent: the score scale must be positive (the row maximum is taken before scaling)");
    QT_REQUIRE((seq_len != nullptr) != (seq_start != nullptr && seq_past != nullptr), "attention_latent: either seq_len or seq_start and seq_past");
    QT_REQUIRE(n_splits >= 1 && n_splits <= 65535 && (n_splits == 1 || (part_acc && part_ml)), "attention_latent: %d key ranges need scratch memory", n_splits);
    // A one-token step of few heads leaves most row groups of a block without rows: there the keys of a page are cut
    // among the row groups, and a block delivers 4 (up to 16 heads) or 2 (up to 32) of the n_splits partial results.
    const int kp = !seq_len ? 1 : (heads <= 16 && n_splits % 4 == 0) ? 4 : (heads <= 32 && n_splits % 2 == 0) ? 2 : 1;
    const int block_rows = 64 / kp;
    const int lds = (row + 15) / 16 * 16 + PAD;
    const size_t smem = (size_t)3 * PAGE * lds * 2 + (size_t)4 * 16 * PAGE * 2;      // three tiles and the row groups' weights
    QT_REQUIRE(smem <= 227 * 1024, "attention_latent: rows of %d elements do not fit shared memory (use the generic kernel)", row);
    LatentParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, block_table, max_blocks, seq_start, seq_past,
                   seq_len, heads, row, rank, scale, n_splits / kp, part_acc, part_ml};
    const long long most_rows = (long long)(seq_len ? 1 : max_q_len) * heads;
    dim3 grid((unsigned)((most_rows + block_rows - 1) / block_rows), n_splits / kp, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
#define QT_LAUNCH_LATENT_KP(NT, KP)                                                                                       \
    do {                                                                                                                 \
        static bool ok = false;                                                                                          \
        if (!ok) { rc = raise_smem(latent_attention_kernel<NT, KP>, 227 * 1024, "attention_latent"); if (rc) return rc; ok = true; } \
        launch_kernel(latent_attention_kernel<NT, KP>, grid, dim3(LT_THREADS), smem, s, p);                               \
    } while (0)
#define QT_LAUNCH_LATENT(NT)                                                                                              \
    do {                                                                                                                 \
        if (kp == 4) QT_LAUNCH_LATENT_KP(NT, 4);                                                                         \
        else if (kp == 2) QT_LAUNCH_LATENT_KP(NT, 2);                                                                    \
        else QT_LAUNCH_LATENT_KP(NT, 1);                                                                                 \
    } while (0)
    if (rank <= 128) QT_LAUNCH_LATENT(8);
    else if (rank <= 256) QT_LAUNCH_LATENT(16);
    else QT_LAUNCH_LATENT(32);
#undef QT_LAUNCH_LATENT
#undef QT_LAUNCH_LATENT_KP
    QT_CHECK_LAUNCH("attention_latent");
    if (n_splits > 1) {
        launch_kernel(attention_combine_mma_kernel, dim3(n_seqs * heads), dim3(128), 0, s, part_acc, part_ml, (__nv_bfloat16*)out, n_splits, rank, 0, (const float*)nullptr, 1);
        QT_CHECK_LAUNCH("attention_combine_mma");
    }
    return QT_OK;
}

QT_DEFINE_LAST_ERROR(attention_latent)
