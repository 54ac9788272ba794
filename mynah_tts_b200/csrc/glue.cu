// Layer glue of the Magpie decoder step: LayerNorm (+ fused int8 activation
// quantization), stand-alone activation quantization, GELU, residual add,
// per-codebook embedding mean, position add, constrained argmax and the small
// element-wise helpers of the backend seam.
//
// "strict" variants reproduce the reference's scalar summation order
// (src/kernels.c:186-244 portable branch, src/graph.c:760-804) so that a row
// normalized here equals the row normalized on the CPU bit for bit; the fast
// variants use fixed-order tree reductions and agree to rounding error.
#include "common.cuh"
#include "launch.h"

#include <float.h>
#include <stdlib.h>

namespace {

// ---------------------------------------------------------------- LayerNorm
// One CTA per row.  Dynamic shared memory: the row, then the squares and the gain (strict
// form) or the gain and the bias (fast form).
template <bool STRICT>
__global__ void __launch_bounds__(256)
k_layernorm(const float *__restrict__ in, float *__restrict__ out, const float *__restrict__ gain,
            const float *__restrict__ bias, int width, float eps, int8_t *__restrict__ qx,
            float *__restrict__ sx, const int *__restrict__ n_active) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[96];
    __shared__ float stat[2];
    // gain and bias are constants: they are staged while the preceding launch still runs
    float *gs = row + width, *bs = gs + width;
    if (!STRICT) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            gs[i] = __ldg(gain + i);
            if (bias != nullptr) bs[i] = __ldg(bias + i);
        }
    } else {
        // strict: gs holds the squares, the gain sits behind them
        for (int i = threadIdx.x; i < width; i += blockDim.x) bs[i] = __ldg(gain + i);
    }
    const int live = mb_lane_count(n_active);
    mb_pdl_wait();
    mb_pdl_trigger();
    const int r = blockIdx.x;
    if (r >= live) return;
    const float *x = in + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = x[i];
    __syncthreads();
    float *y_out = out == nullptr ? nullptr : out + (size_t)r * width;
    int8_t *q = qx == nullptr ? nullptr : qx + (size_t)r * width;
    float sxv;
    if (STRICT) {
        // the reference's two sequential chains (mean, variance); the squares sit behind the row
        sxv = mb_ln_block_strict(row, width, bs, bias, eps, gs, stat, red, y_out, qx != nullptr, q);
    } else {
        // the routine shared with the products' fused prologue
        sxv = mb_ln_block<1>(row, width, gs, bias == nullptr ? nullptr : bs, eps, red, y_out, qx != nullptr, q);
    }
    if (qx != nullptr && threadIdx.x == 0) sx[r] = sxv;
}

// Per-row int8 activation quantization (src/qmat.c:93-113).
__global__ void __launch_bounds__(256)
k_quant_rows(const float *__restrict__ in, int width, int8_t *__restrict__ qx,
             float *__restrict__ sx, const int *__restrict__ n_active) {
    const int live = mb_lane_count(n_active);
    mb_pdl_wait();
    mb_pdl_trigger();
    __shared__ float red[33];
    const int r = blockIdx.x;
    if (r >= live) return;
    const float *x = in + (size_t)r * width;
    constexpr int VMAX = 4;                            // float4s a thread keeps in registers
    if ((width & 3) == 0 && width <= 4 * VMAX * (int)blockDim.x && (reinterpret_cast<uintptr_t>(in) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(qx) & 3u) == 0) {
        // the row is read once, four values per thread and load, and stays in registers
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        const int n4 = width >> 2;
        float4 v[VMAX];
        float vmax = 0.0f;
#pragma unroll
        for (int j = 0; j < VMAX; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            v[j] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < VMAX; ++j)
            vmax = fmaxf(fmaxf(vmax, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
        vmax = block_max1(vmax, red);
        const float inv4 = vmax > 0.0f ? __fdiv_rn(127.0f, vmax) : 0.0f;
        char4 *q4 = reinterpret_cast<char4 *>(qx + (size_t)r * width);
#pragma unroll
        for (int j = 0; j < VMAX; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n4) {
                char4 c;
                c.x = (signed char)min(127, max(-127, round_half_away(__fmul_rn(v[j].x, inv4))));
                c.y = (signed char)min(127, max(-127, round_half_away(__fmul_rn(v[j].y, inv4))));
                c.z = (signed char)min(127, max(-127, round_half_away(__fmul_rn(v[j].z, inv4))));
                c.w = (signed char)min(127, max(-127, round_half_away(__fmul_rn(v[j].w, inv4))));
                q4[i] = c;
            }
        }
        if (threadIdx.x == 0) sx[r] = vmax > 0.0f ? __fdiv_rn(vmax, 127.0f) : 0.0f;
        return;
    }
    float amax = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) amax = fmaxf(amax, fabsf(x[i]));
    amax = block_max(amax, red);
    int8_t *q = qx + (size_t)r * width;
    if (amax == 0.0f) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) q[i] = 0;
        if (threadIdx.x == 0) sx[r] = 0.0f;
        return;
    }
    const float inv = __fdiv_rn(127.0f, amax);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        int v = round_half_away(__fmul_rn(x[i], inv));
        v = min(127, max(-127, v));
        q[i] = (int8_t)v;
    }
    if (threadIdx.x == 0) sx[r] = __fdiv_rn(amax, 127.0f);
}

template <bool STRICT>
__global__ void k_gelu(float *data, size_t n, const uint32_t *tanh_tab) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) data[i] = gelu_tanh<STRICT>(data[i], tanh_tab);
}

__global__ void k_residual_add(float *out, const float *in, size_t n) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(out[i], in[i]);
}

__global__ void k_scale(float *data, size_t n, float scale) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) data[i] = __fmul_rn(data[i], scale);
}

// Non-finite -> 0, else clamp to [-1, 1] (src/backend.c:815-820).
__global__ void k_clip(float *data, size_t n) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = data[i];
    data[i] = !isfinite(v) ? 0.0f : (v > 1.0f ? 1.0f : (v < -1.0f ? -1.0f : v));
}

__global__ void k_bias_add(float *out, const float *bias, size_t total, size_t cols) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = __fadd_rn(out[i], bias[i % cols]);
}

// ---------------------------------------------------------------- argmax
// Candidates: ids below codebook_size, plus eos_id when allowed; strict `>`
// against a running best that starts at -FLT_MAX keeps the first of equal
// values and yields 0 when nothing exceeds -FLT_MAX (src/backend.c:825-847).
__global__ void __launch_bounds__(256)
k_argmax_rows(const float *__restrict__ logits, int vocab, int codebook_size, int eos_id,
              const int *__restrict__ allow_eos, int allow_eos_scalar,
              unsigned *__restrict__ tokens, unsigned *__restrict__ codes,
              int *__restrict__ eos_flag, int tables_per_stream,
              const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    __shared__ float bv[256];
    __shared__ unsigned bi[256];
    const int r = blockIdx.x;
    const int stream = r / tables_per_stream;
    if (n_active != nullptr && stream >= *n_active) return;
    const int allow = allow_eos != nullptr ? allow_eos[stream] : allow_eos_scalar;
    const float *row = logits + (size_t)r * vocab;
    float best = -FLT_MAX;
    unsigned idx = 0xffffffffu;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        if (!(i < codebook_size || (allow && i == eos_id))) continue;
        const float v = row[i];
        if (v > best) { best = v; idx = (unsigned)i; }
    }
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) {
            const float ov = bv[threadIdx.x + s];
            const unsigned oi = bi[threadIdx.x + s];
            if (ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi < bi[threadIdx.x])) {
                bv[threadIdx.x] = ov;
                bi[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const unsigned tok = bi[0] == 0xffffffffu ? 0u : bi[0];
        tokens[r] = tok;
        if (codes != nullptr) codes[r] = tok < (unsigned)codebook_size ? tok : 0u;
        if (eos_flag != nullptr && tok == (unsigned)eos_id) atomicOr(&eos_flag[stream], 1);
    }
}

// ---------------------------------------------------------------- embedding
// row = sum_t table_t[code_t] (in table order), row /= tables, x = row + pe
// (src/graph.c:771-803 then src/graph.c:3156-3157).
__global__ void __launch_bounds__(256)
k_embed_frames(const float *const *__restrict__ tables, int n_tables, int vocab, int width,
               const unsigned *__restrict__ codes, const float *__restrict__ position,
               const int *__restrict__ lens, float *__restrict__ x,
               const int *__restrict__ n_active, int *__restrict__ status) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b = blockIdx.x;
    if (n_active != nullptr && b >= *n_active) return;
    const float *pe = position + (size_t)lens[b] * width;
    // codes and table bases of up to ET tables at a time, all fetched before any row: the
    // three loads behind each table row (code, base, row) otherwise run one after another
    constexpr int ET = 8;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};          // this thread's elements d, d + 256, ...
    const int per_thread = (width + (int)blockDim.x - 1) / (int)blockDim.x;
    if (per_thread > 4) {                             // wide rows: the plain loop
        for (int d = threadIdx.x; d < width; d += blockDim.x) {
            float row = 0.0f;
            for (int t = 0; t < n_tables; ++t) {
                unsigned code = codes[(size_t)b * n_tables + t];
                if (code >= (unsigned)vocab) {
                    if (status != nullptr) atomicOr(status, 1);
                    code = 0;
                }
                row = __fadd_rn(row, tables[t][(size_t)code * width + d]);
            }
            row = __fdiv_rn(row, (float)n_tables);
            x[(size_t)b * width + d] = __fadd_rn(row, pe[d]);
        }
        return;
    }
    bool bad = false;
    for (int t0 = 0; t0 < n_tables; t0 += ET) {
        const float *base[ET];
#pragma unroll
        for (int u = 0; u < ET; ++u) {
            const int t = t0 + u;
            unsigned code = t < n_tables ? codes[(size_t)b * n_tables + t] : 0u;
            if (code >= (unsigned)vocab) { bad = true; code = 0u; }
            base[u] = t < n_tables ? tables[t] + (size_t)code * width : nullptr;
        }
        float v[ET][4];
#pragma unroll
        for (int u = 0; u < ET; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int d = threadIdx.x + j * blockDim.x;
                v[u][j] = (t0 + u < n_tables && d < width) ? base[u][d] : 0.0f;
            }
#pragma unroll
        for (int u = 0; u < ET; ++u)
            if (t0 + u < n_tables)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = __fadd_rn(acc[j], v[u][j]);   // table order
    }
    if (bad && threadIdx.x == 0 && status != nullptr) atomicOr(status, 1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int d = threadIdx.x + j * blockDim.x;
        if (d < width) x[(size_t)b * width + d] = __fadd_rn(__fdiv_rn(acc[j], (float)n_tables), pe[d]);
    }
}

__global__ void __launch_bounds__(256)
k_add_position(const float *__restrict__ rows, const float *__restrict__ position,
               const int *__restrict__ lens, float *__restrict__ x, int width,
               const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b = blockIdx.x;
    if (n_active != nullptr && b >= *n_active) return;
    const float *pe = position + (size_t)lens[b] * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x)
        x[(size_t)b * width + d] = __fadd_rn(rows[(size_t)b * width + d], pe[d]);
}

// x[b] = rows[b] + row: the local transformer's input at one position
// (src/graph.c:1262-1264; every lane is at the same position of its frame).
__global__ void __launch_bounds__(256)
k_add_row(const float *__restrict__ rows, const float *__restrict__ row, float *__restrict__ x, int width,
          const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b = blockIdx.x;
    if (n_active != nullptr && b >= *n_active) return;
    for (int d = threadIdx.x; d < width; d += blockDim.x)
        x[(size_t)b * width + d] = __fadd_rn(rows[(size_t)b * width + d], row[d]);
}

// One table of one stacked frame, one CTA per lane: the tail of the per-stream loop of
// sample_local_frame_batch (src/graph.c:1538-1652).
//   * candidates below codebook_size, and EOS when allowed, compete; the rest count as
//     -FLT_MAX;
//   * greedy pick: largest logit, first index on ties;
//   * when temperature > 0 and topk > 1: the top-k in the reference's insertion order
//     (higher logit first, earlier index first among equals) is produced by sorting
//     (logit, index) keys: for k <= 128 and 1024..4096 keys each warp sorts its share in
//     registers and three rounds of pairwise merges keep the 128 largest (block_top128);
//     otherwise a bitonic sort of all keys in shared memory; weights exp((l - max) / T) are summed in that order by one
//     thread, the lane's xorshift64 state advances once, and the drawn token is the first
//     whose running sum reaches draw = (top 24 bits / 2^24) * total (the last one if none);
//   * EOS is reported if the greedy or the drawn token is EOS; the stored code collapses
//     specials to 0; the embedding row of the fed-back token becomes the next input.
// Dynamic shared memory: n2 keys of 8 bytes + n2 floats, n2 = vocab rounded up to a power
// of two.
__device__ __forceinline__ unsigned ordered_bits(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(unsigned o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

// ---- top 128 of the sampler's keys without block-wide sorting steps
// Bitonic sort of 32 * R keys held by one warp, largest first: element e = r * 32 + lane is
// register r of lane `lane`.  Strides of 32 and more exchange registers of one lane, smaller
// strides exchange lanes by shuffle; no shared memory, no barrier.
template <int R>
__device__ __forceinline__ void warp_sort_desc(unsigned long long (&v)[R], int lane) {
#pragma unroll
    for (int size = 2; size <= 32 * R; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= 32) {
                const int rs = stride >> 5;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if ((r & rs) == 0) {
                        const bool desc = (((r * 32 + lane) & size) == 0);
                        const unsigned long long a = v[r], c = v[r | rs];
                        if ((a < c) == desc) { v[r] = c; v[r | rs] = a; }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const unsigned long long other = __shfl_xor_sync(MB_FULL, v[r], stride);
                    const bool desc = (((r * 32 + lane) & size) == 0);
                    const bool keep_max = (((lane & stride) == 0) == desc);
                    v[r] = keep_max ? (v[r] > other ? v[r] : other) : (v[r] < other ? v[r] : other);
                }
            }
        }
    }
}

// Two lists of 128 keys sorted largest first -> the 128 largest of both, sorted, by one warp:
// max(A[e], B[127 - e]) is a bitonic sequence holding them; seven merge steps sort it.
__device__ __forceinline__ void warp_merge_top128(const unsigned long long *A, const unsigned long long *B,
                                                  unsigned long long *out, int lane) {
    unsigned long long v[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int e = r * 32 + lane;
        const unsigned long long a = A[e], c = B[127 - e];
        v[r] = a > c ? a : c;
    }
    __syncwarp();                                            // `out` may be A: all reads are done
#pragma unroll
    for (int rs = 2; rs >= 1; rs >>= 1)
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if ((r & rs) == 0) {
                const unsigned long long a = v[r], c = v[r | rs];
                if (a < c) { v[r] = c; v[r | rs] = a; }
            }
#pragma unroll
    for (int stride = 16; stride > 0; stride >>= 1)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const unsigned long long other = __shfl_xor_sync(MB_FULL, v[r], stride);
            v[r] = ((lane & stride) == 0) ? (v[r] > other ? v[r] : other) : (v[r] < other ? v[r] : other);
        }
#pragma unroll
    for (int r = 0; r < 4; ++r) out[r * 32 + lane] = v[r];
}

// keys[0 .. 256 * R) (256 threads, R keys each) -> keys[0 .. 128) = the 128 largest, sorted.
// Each of the eight warps sorts its 32 * R keys in registers and keeps 128; three rounds of
// pairwise merges (four, two, one warp) leave the result in place.
template <int R>
__device__ __forceinline__ void block_top128(unsigned long long *keys) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long v[R];
#pragma unroll
    for (int r = 0; r < R; ++r) v[r] = keys[r * 256 + threadIdx.x];
    __syncthreads();
    warp_sort_desc<R>(v, lane);
#pragma unroll
    for (int r = 0; r < 4; ++r) keys[warp * 128 + r * 32 + lane] = v[r];
    __syncthreads();
    if (warp < 4) warp_merge_top128(keys + 256 * warp, keys + 256 * warp + 128, keys + 256 * warp, lane);
    __syncthreads();
    if (warp < 2) warp_merge_top128(keys + 512 * warp, keys + 512 * warp + 256, keys + 512 * warp, lane);
    __syncthreads();
    if (warp == 0) warp_merge_top128(keys, keys + 512, keys, lane);
    __syncthreads();
}

template <bool STRICT>
__global__ void __launch_bounds__(256)
k_local_sample(const float *__restrict__ logits, int ld, int vocab, int n2, int codebook_size, int eos_id,
               const int *__restrict__ allow_eos, const float *__restrict__ temperature,
               const unsigned *__restrict__ topk, unsigned long long *__restrict__ rng, int table, int tables,
               int codebooks, unsigned *__restrict__ tokens, unsigned *__restrict__ codes,
               int *__restrict__ eos_flag, int *__restrict__ eos_sub, const float *__restrict__ emb_table,
               float *__restrict__ row_in, const float *__restrict__ next_row, float *__restrict__ x_out, int width,
               const uint32_t *__restrict__ exp_tab,
               const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    extern __shared__ __align__(8) unsigned char sample_smem[];
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(sample_smem);
    float *weights = reinterpret_cast<float *>(keys + n2);
    __shared__ float s_best[8];
    __shared__ int s_idx[8];
    __shared__ unsigned s_emit;
    const int b = blockIdx.x;
    if (n_active != nullptr && b >= *n_active) return;
    const float *lg = logits + (size_t)b * ld;
    const bool eos_ok = allow_eos == nullptr || allow_eos[b] != 0;
    const float temp = temperature != nullptr ? temperature[b] : 0.0f;
    const unsigned k = topk != nullptr ? topk[b] : 0u;
    const bool sampling = temp > 0.0f && k > 1u && rng != nullptr;
    float best = -FLT_MAX;
    int best_i = 0x7fffffff;
    for (int c = threadIdx.x; c < n2; c += blockDim.x) {
        unsigned long long key = 0ull;                       // padding sorts after every candidate
        if (c < vocab) {
            const bool ok = c < codebook_size || (c == eos_id && eos_ok);
            float v = ok ? lg[c] : -FLT_MAX;
            if (ok && v > best) { best = v; best_i = c; }
            if (v == 0.0f) v = 0.0f;                         // -0 and +0 compare equal: one key for both
            key = ((unsigned long long)ordered_bits(v) << 32) | (unsigned)(0xffffffffu - (unsigned)c);
        }
        if (sampling) keys[c] = key;
    }
    // first-on-ties argmax over the block
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(MB_FULL, best, o);
        const int oi = __shfl_xor_sync(MB_FULL, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_best[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (sampling && k <= 128u && blockDim.x == 256 && (n2 == 1024 || n2 == 2048 || n2 == 4096)) {
        // only the first k keys are read below: the 128 largest, sorted, are enough
        if (n2 == 1024) block_top128<4>(keys);
        else if (n2 == 2048) block_top128<8>(keys);
        else block_top128<16>(keys);
    } else if (sampling) {
        for (int size = 2; size <= n2; size <<= 1)
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int i = threadIdx.x; i < (n2 >> 1); i += blockDim.x) {
                    const int lo = ((i / stride) * stride * 2) + (i % stride), hi = lo + stride;
                    const bool descending = ((lo & size) == 0);
                    const unsigned long long a = keys[lo], c = keys[hi];
                    if ((a < c) == descending) { keys[lo] = c; keys[hi] = a; }
                }
                __syncthreads();
            }
    }
    if (sampling) {
        const int used = (int)min(k, (unsigned)vocab);
        const float maximum = from_ordered_bits((unsigned)(keys[0] >> 32));
        for (int q = threadIdx.x; q < used; q += blockDim.x) {
            const float l = from_ordered_bits((unsigned)(keys[q] >> 32));
            weights[q] = exp_ref<STRICT>(__fdiv_rn(__fsub_rn(l, maximum), temp), exp_tab);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float gb = s_best[0];
        int gi = s_idx[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (s_best[w] > gb || (s_best[w] == gb && s_idx[w] < gi)) { gb = s_best[w]; gi = s_idx[w]; }
        const unsigned argmax = gi == 0x7fffffff ? 0u : (unsigned)gi;
        unsigned value = argmax;
        if (sampling) {
            const int used = (int)min(k, (unsigned)vocab);
            // sequential sums in list order (the reference's), sixteen weights fetched at a
            // time so that the chain is the additions, not a shared-memory load per step
            float total = 0.0f;
            for (int q0 = 0; q0 < used; q0 += 16) {
                float w[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) w[u] = q0 + u < used ? weights[q0 + u] : 0.0f;
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (q0 + u < used) total = __fadd_rn(total, w[u]);
            }
            unsigned long long state = rng[b];
            state ^= state << 13;
            state ^= state >> 7;
            state ^= state << 17;
            if (state == 0ull) state = 0x9e3779b97f4a7c15ull;
            rng[b] = state;
            const float draw = __fmul_rn(__fdiv_rn((float)((state >> 40) & 0xffffffull), 16777216.0f), total);
            float cumulative = 0.0f;
            int pick = used - 1;                             // the last one if no running sum reaches the draw
            for (int q0 = 0; q0 < used && pick == used - 1; q0 += 16) {
                float w[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) w[u] = q0 + u < used ? weights[q0 + u] : 0.0f;
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    if (q0 + u < used && pick == used - 1) {
                        cumulative = __fadd_rn(cumulative, w[u]);
                        if (draw <= cumulative) pick = q0 + u;
                    }
                }
            }
            value = 0xffffffffu - (unsigned)(keys[pick] & 0xffffffffull);
        }
        const bool eos = argmax == (unsigned)eos_id || value == (unsigned)eos_id;
        if (eos) {
            if (eos_flag != nullptr) eos_flag[b] = 1;
            if (eos_sub != nullptr) eos_sub[b] = min(eos_sub[b], table / codebooks);
        }
        tokens[(size_t)b * tables + table] = value;
        codes[(size_t)b * tables + table] = value < (unsigned)codebook_size ? value : 0u;
        s_emit = value < (unsigned)vocab ? value : 0u;
    }
    __syncthreads();
    const float *e = emb_table + (size_t)s_emit * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        const float v = e[d];
        row_in[(size_t)b * width + d] = v;
        if (x_out != nullptr) x_out[(size_t)b * width + d] = __fadd_rn(v, next_row[d]);
    }
}

// out[t] = table[ids[t]] + position[t]   (encode_text, src/graph.c:728-733 and 651-653)
__global__ void __launch_bounds__(256)
k_gather_rows(const float *__restrict__ table, const int *__restrict__ ids, const float *__restrict__ position,
              float *__restrict__ out, int width) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int t = blockIdx.x;
    const float *row = table + (size_t)ids[t] * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[(size_t)t * width + i] = __fadd_rn(row[i], position[(size_t)t * width + i]);
}

// Causal unfold of `length` rows over a convolution window (unfold_causal,
// src/graph.c:267-286): col[t][i * kernel + k] = in[t - (kernel - 1) + k][i], zero before
// the first row.
__global__ void __launch_bounds__(256)
k_unfold_causal(const float *__restrict__ in, float *__restrict__ col, int channels, int kernel) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int t = blockIdx.x;
    const int total = channels * kernel;
    for (int j = threadIdx.x; j < total; j += blockDim.x) {
        const int i = j / kernel, k = j - i * kernel;
        const int src = t - (kernel - 1) + k;
        col[(size_t)t * total + j] = src < 0 ? 0.0f : in[(size_t)src * channels + i];
    }
}

__global__ void k_advance_lens(int *lens, int batch, const int *n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch && (n_active == nullptr || b < *n_active)) lens[b] += 1;
}

// One CTA; thread b serves lane b.  frame_idx is read by every thread before the
// barrier and bumped by thread 0 after it.
__global__ void __launch_bounds__(1024)
k_frame_advance(int *lens, const unsigned *__restrict__ tokens_cur, unsigned *__restrict__ history,
                int *frame_idx, const int *__restrict__ eos_flag, int *eos_frame, int *allow_eos,
                int batch, int lane_stride, int tables, const int *__restrict__ min_frames, int history_frames,
                const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const int frame = *frame_idx;
    const int nb = n_active != nullptr ? min(batch, *n_active) : batch;
    __syncthreads();
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
        if (b < nb) {
            lens[b] += 1;
            if (history != nullptr && frame < history_frames)
                for (int t = 0; t < tables; ++t)
                    history[((size_t)frame * lane_stride + b) * tables + t] = tokens_cur[(size_t)b * tables + t];
            if (eos_frame != nullptr && eos_flag[b] != 0 && eos_frame[b] < 0) eos_frame[b] = frame;
        }
        if (allow_eos != nullptr && min_frames != nullptr) allow_eos[b] = (frame + 1 >= *min_frames) ? 1 : 0;
    }
    if (threadIdx.x == 0) *frame_idx = frame + 1;
}

int g_pdl = -1;

inline unsigned blocks_for(size_t n) { return (unsigned)((n + 255) / 256); }

}  // namespace

extern "C" int mb_layernorm(const float *in, float *out, const float *gain, const float *bias,
                            size_t rows, size_t width, float eps, int8_t *qx, float *sx,
                            const int *n_active, int strict, mb_stream stream) {
    /* strict: the row, its squares and the gain; else the row, the gain and the bias slot */
    const size_t smem = width * sizeof(float) * 3u;
    if (rows == 0 || width == 0 || smem > 48u * 1024u) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (strict)
        mb_launch(k_layernorm<true>, dim3((unsigned)rows), dim3(256), smem, s, in, out, gain, bias, (int)width, eps,
                                                            qx, sx, n_active);
    else
        mb_launch(k_layernorm<false>, dim3((unsigned)rows), dim3(256), smem, s, in, out, gain, bias, (int)width, eps,
                                                             qx, sx, n_active);
    return mb_check_launch();
}

#ifdef MB_PHASE_TICKS
// Profiling builds only (make TICKS=1): SM cycles per term of mb_seq_sum over `n` floats in
// shared memory, one thread, `reps` sums in a row (n a multiple of 16, at most 4096).
namespace {
__global__ void k_seq_sum_cycles(int n, int reps, long long *cycles, float *sink) {
    extern __shared__ __align__(16) float row[];
    for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = (float)((i * 2654435761u) % 1000u) / 977.0f - 0.5f;
    __syncthreads();
    if (threadIdx.x != 0) return;
    float acc = 0.0f;
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
        const float s = mb_seq_sum(row, n);
        acc += s;
        row[0] = row[0] + (s > 1e30f ? 1.0f : 0.0f);       // keeps the sums apart
    }
    *cycles = clock64() - t0;
    *sink = acc;
}
}  // namespace
extern "C" __attribute__((visibility("default")))
int mynah_b200_debug_seq_sum_cycles(size_t n, size_t reps, double *cycles_per_term) {
    if (n == 0 || (n % 16u) != 0 || n > 4096u || reps == 0 || cycles_per_term == nullptr) return -1;
    long long *dc = nullptr;
    float *ds = nullptr;
    if (cudaMalloc((void **)&dc, sizeof(long long)) != cudaSuccess || cudaMalloc((void **)&ds, sizeof(float)) != cudaSuccess) return -1;
    for (int pass = 0; pass < 2; ++pass) k_seq_sum_cycles<<<1, 256, n * sizeof(float)>>>((int)n, (int)reps, dc, ds);
    long long c = 0;
    const int rc = (int)cudaMemcpy(&c, dc, sizeof(c), cudaMemcpyDeviceToHost);
    cudaFree(dc); cudaFree(ds);
    *cycles_per_term = (double)c / (double)reps / (double)n;
    return rc;
}
#endif

extern "C" int mb_quant_rows(const float *in, size_t rows, size_t width, int8_t *qx, float *sx,
                             const int *n_active, mb_stream stream) {
    if (rows == 0 || width == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_quant_rows, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, in, (int)width, qx, sx, n_active);
    return mb_check_launch();
}

extern "C" int mb_gelu(float *data, size_t n, int strict, const uint32_t *tanh_tab, mb_stream stream) {
    if (n == 0) return 0;
    if (strict) mb_launch(k_gelu<true>, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, data, n, tanh_tab);
    else mb_launch(k_gelu<false>, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, data, n, nullptr);
    return mb_check_launch();
}

extern "C" int mb_residual_add(float *out, const float *in, size_t n, mb_stream stream) {
    if (n == 0) return 0;
    mb_launch(k_residual_add, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, out, in, n);
    return mb_check_launch();
}

extern "C" int mb_scale(float *data, size_t n, float scale, mb_stream stream) {
    if (n == 0) return 0;
    mb_launch(k_scale, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, data, n, scale);
    return mb_check_launch();
}

extern "C" int mb_clip(float *data, size_t n, mb_stream stream) {
    if (n == 0) return 0;
    mb_launch(k_clip, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, data, n);
    return mb_check_launch();
}

extern "C" int mb_bias_add(float *out, const float *bias, size_t rows, size_t cols,
                           mb_stream stream) {
    if (rows * cols == 0) return 0;
    mb_launch(k_bias_add, dim3(blocks_for(rows * cols)), dim3(256), 0, (cudaStream_t)stream, out, bias, rows * cols,
                                                                         cols);
    return mb_check_launch();
}

extern "C" int mb_argmax_rows(const float *logits, size_t rows, size_t vocab, size_t codebook_size,
                              size_t eos_id, const int *allow_eos, int allow_eos_scalar,
                              unsigned *tokens, unsigned *codes, int *eos_flag,
                              size_t tables_per_stream, const int *n_active, mb_stream stream) {
    if (rows == 0 || vocab == 0 || tables_per_stream == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_argmax_rows, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, 
        logits, (int)vocab, (int)codebook_size, (int)eos_id, allow_eos, allow_eos_scalar, tokens,
        codes, eos_flag, (int)tables_per_stream, n_active);
    return mb_check_launch();
}

extern "C" int mb_embed_frames(const float *const *tables, size_t n_tables, size_t vocab,
                               size_t width, const unsigned *codes, const float *position,
                               const int *lens, float *x, size_t batch, const int *n_active,
                               int *status, mb_stream stream) {
    if (batch == 0 || n_tables == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_embed_frames, dim3((unsigned)batch), dim3(256), 0, (cudaStream_t)stream, 
        tables, (int)n_tables, (int)vocab, (int)width, codes, position, lens, x, n_active, status);
    return mb_check_launch();
}

extern "C" int mb_add_position(const float *rows, const float *position, const int *lens, float *x,
                               size_t batch, size_t width, const int *n_active, mb_stream stream) {
    if (batch == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_add_position, dim3((unsigned)batch), dim3(256), 0, (cudaStream_t)stream, rows, position, lens, x,
                                                                      (int)width, n_active);
    return mb_check_launch();
}

extern "C" int mb_add_row(const float *rows, const float *row, float *x, size_t batch, size_t width,
                          const int *n_active, mb_stream stream) {
    if (batch == 0 || width == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_add_row, dim3((unsigned)batch), dim3(256), 0, (cudaStream_t)stream, rows, row, x, (int)width, n_active);
    return mb_check_launch();
}

extern "C" size_t mb_local_sample_smem(size_t vocab) {
    size_t n2 = 2;
    while (n2 < vocab) n2 <<= 1;
    return n2 * (sizeof(unsigned long long) + sizeof(float));
}

extern "C" int mb_local_sample(const mb_sample_args *a, mb_stream stream) {
    if (a == nullptr || a->logits == nullptr || a->batch == 0 || a->vocab == 0 || a->tables == 0 ||
        a->codebooks == 0 || a->tokens == nullptr || a->codes == nullptr || a->emb_table == nullptr ||
        a->row_in == nullptr)
        return (int)cudaErrorInvalidValue;
    size_t n2 = 2;
    while (n2 < a->vocab) n2 <<= 1;
    const size_t smem = mb_local_sample_smem(a->vocab);
    if (smem > 200u * 1024u) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(k_local_sample<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(k_local_sample<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (a->strict)
        mb_launch(k_local_sample<true>, dim3((unsigned)a->batch), dim3(256), smem, s, a->logits, (int)a->logits_stride,
                  (int)a->vocab, (int)n2, (int)a->codebook_size, (int)a->eos_id, a->allow_eos, a->temperature, a->topk,
                  a->rng, (int)a->table, (int)a->tables, (int)a->codebooks, a->tokens, a->codes, a->eos_flag,
                  a->eos_sub, a->emb_table, a->row_in, a->next_row, a->next_row == nullptr ? nullptr : a->x_out, (int)a->width,
                  a->exp_tab, a->n_active);
    else
        mb_launch(k_local_sample<false>, dim3((unsigned)a->batch), dim3(256), smem, s, a->logits, (int)a->logits_stride,
                  (int)a->vocab, (int)n2, (int)a->codebook_size, (int)a->eos_id, a->allow_eos, a->temperature, a->topk,
                  a->rng, (int)a->table, (int)a->tables, (int)a->codebooks, a->tokens, a->codes, a->eos_flag,
                  a->eos_sub, a->emb_table, a->row_in, a->next_row, a->next_row == nullptr ? nullptr : a->x_out, (int)a->width,
                  a->exp_tab, a->n_active);
    return mb_check_launch();
}

extern "C" int mb_gather_rows(const float *table, const int *ids, const float *position, float *out, size_t rows,
                              size_t width, mb_stream stream) {
    if (rows == 0 || width == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_gather_rows, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, table, ids, position, out, (int)width);
    return mb_check_launch();
}

extern "C" int mb_unfold_causal(const float *in, float *col, size_t rows, size_t channels, size_t kernel, mb_stream stream) {
    if (rows == 0 || channels == 0 || kernel == 0) return (int)cudaErrorInvalidValue;
    mb_launch(k_unfold_causal, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, in, col, (int)channels, (int)kernel);
    return mb_check_launch();
}

extern "C" int mb_advance_lens(int *lens, size_t batch, const int *n_active, mb_stream stream) {
    if (batch == 0) return 0;
    mb_launch(k_advance_lens, dim3(blocks_for(batch)), dim3(256), 0, (cudaStream_t)stream, lens, (int)batch, n_active);
    return mb_check_launch();
}

extern "C" int mb_frame_advance(int *lens, const unsigned *tokens_cur, unsigned *history,
                                int *frame_idx, const int *eos_flag, int *eos_frame, int *allow_eos,
                                size_t batch, size_t lane_stride, size_t tables,
                                const int *min_frames, size_t history_frames, const int *n_active,
                                mb_stream stream) {
    if (batch == 0 || frame_idx == nullptr) return (int)cudaErrorInvalidValue;
    const unsigned threads = batch < 1024 ? (unsigned)((batch + 31) / 32 * 32) : 1024u;
    mb_launch(k_frame_advance, dim3(1), dim3(threads), 0, (cudaStream_t)stream, 
        lens, tokens_cur, history, frame_idx, eos_flag, eos_frame, allow_eos, (int)batch,
        (int)lane_stride, (int)tables, min_frames, (int)history_frames, n_active);
    return mb_check_launch();
}

extern "C" int mb_pdl_enabled(void) {
    if (g_pdl < 0) {
        const char *env = getenv("MYNAH_B200_PDL");
        g_pdl = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    return g_pdl;
}
