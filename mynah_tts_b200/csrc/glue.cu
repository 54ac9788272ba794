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
// One CTA per row.  Dynamic shared memory: width floats (the row, then y).
template <bool STRICT>
__global__ void __launch_bounds__(256)
k_layernorm(const float *__restrict__ in, float *__restrict__ out, const float *__restrict__ gain,
            const float *__restrict__ bias, int width, float eps, int8_t *__restrict__ qx,
            float *__restrict__ sx, const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    extern __shared__ float row[];
    __shared__ float red[33];
    __shared__ float stat[2];
    const int r = blockIdx.x;
    if (n_active != nullptr && r >= *n_active) return;
    const float *x = in + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = x[i];
    __syncthreads();
    float mean, variance;
    if (STRICT) {
        // mean: one sequential chain over the row, as `mean += x[i]` does.
        if (threadIdx.x == 0) {
            float m = 0.0f;
            for (int i = 0; i < width; ++i) m = __fadd_rn(m, row[i]);
            stat[0] = __fdiv_rn(m, (float)width);
        }
        __syncthreads();
        mean = stat[0];
        // squares in parallel (each rounded once), then one sequential chain.
        float *sq = row + width;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float d = __fsub_rn(row[i], mean);
            sq[i] = __fmul_rn(d, d);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float v = 0.0f;
            for (int i = 0; i < width; ++i) v = __fadd_rn(v, sq[i]);
            stat[1] = v;
        }
        __syncthreads();
        variance = stat[1];
    } else {
        float s = 0.0f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) s += row[i];
        mean = __fdiv_rn(block_sum(s, red), (float)width);
        float v = 0.0f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float d = row[i] - mean;
            v = fmaf(d, d, v);
        }
        variance = block_sum(v, red);
    }
    const float scale =
        __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(variance, (float)width), eps)));
    float amax = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float y = __fadd_rn(
            __fmul_rn(__fmul_rn(__fsub_rn(row[i], mean), scale), gain[i]),
            bias == nullptr ? 0.0f : bias[i]);
        if (out != nullptr) out[(size_t)r * width + i] = y;
        if (qx != nullptr) {
            row[i] = y;  // each thread rereads only its own elements below
            amax = fmaxf(amax, fabsf(y));
        }
    }
    if (qx == nullptr) return;
    amax = block_max(amax, red);
    int8_t *q = qx + (size_t)r * width;
    if (amax == 0.0f) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) q[i] = 0;
        if (threadIdx.x == 0) sx[r] = 0.0f;
        return;
    }
    const float inv = __fdiv_rn(127.0f, amax);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        int v = round_half_away(__fmul_rn(row[i], inv));
        v = min(127, max(-127, v));
        q[i] = (int8_t)v;
    }
    if (threadIdx.x == 0) sx[r] = __fdiv_rn(amax, 127.0f);
}

// Per-row int8 activation quantization (src/qmat.c:93-113).
__global__ void __launch_bounds__(256)
k_quant_rows(const float *__restrict__ in, int width, int8_t *__restrict__ qx,
             float *__restrict__ sx, const int *__restrict__ n_active) {
    mb_pdl_wait();
    mb_pdl_trigger();
    __shared__ float red[33];
    const int r = blockIdx.x;
    if (n_active != nullptr && r >= *n_active) return;
    const float *x = in + (size_t)r * width;
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
    const size_t smem = width * sizeof(float) * (strict ? 2 : 1);
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
