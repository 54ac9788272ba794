/* Internal C ABI between the C11 host code (backend_b200.c, decoder_b200.c)
 * and the CUDA translation units.  Every function enqueues work on `stream`
 * and returns a cudaError_t value as int (0 = success); none synchronizes.
 * All pointers are device pointers unless the name says host.
 */
#ifndef MYNAH_B200_LAUNCH_H
#define MYNAH_B200_LAUNCH_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mb_stream; /* cudaStream_t */

/* Weight formats.  Values match the reference's enum (src/qmat.c:36). */
enum { MB_F32 = 0, MB_INT8 = 1, MB_INT4 = 2, MB_F16 = 3 };

/* GEMV epilogues. */
enum { MB_EPI_STORE = 0, MB_EPI_RESIDUAL = 1, MB_EPI_GELU = 2 };
enum { MB_FUSE_NONE = 0, MB_FUSE_LN = 1, MB_FUSE_QUANT = 2 };

/* Device tables that make strict-mode expf/tanhf return the host libm's bits
 * (libm_parity.cuh); either pointer may be NULL (then: correctly rounded). */
typedef struct {
    const uint32_t *tanh_tab;
    const uint32_t *exp_tab;
    const uint32_t *sin_tab;   /* built on first use by a strict codec */
} mb_libm_tables;
/* One run of the table build: host_vals_dev[i] is the host's tanhf(a) (kind 0),
 * expf(-a) (kind 1) or sinf(a) (kind 2) for the float a with bit pattern first_bits + i;
 * packs count/8 words at table_words.  status gets bit 4 if a difference does not fit
 * 4 bits. */
int mb_libm_delta(const float *host_vals_dev, uint32_t first_bits, size_t count, int kind,
                  uint32_t *table_words, int *status, mb_stream stream);

/* Per-device one-time kernel attribute setup (call with the device current,
 * outside stream capture). */
int mb_gemv_init(void);
int mb_attention_init(void);

/* ---- weight packing (once per tensor) ---------------------------------- */
int mb_pack_int8(const float *w, size_t n, size_t k, int8_t *q, float *scales, mb_stream stream);
int mb_pack_int4(const float *w, size_t n, size_t k, uint8_t *q, float *scales, mb_stream stream);
int mb_pack_f16(const float *w, size_t count, uint16_t *h, mb_stream stream);

/* ---- glue --------------------------------------------------------------- */
/* LayerNorm over `rows` rows of `width`; bias may be NULL.  When qx != NULL
 * the normalized row is also quantized per row (int8, scale to sx[row]); out
 * may then be NULL.  n_active (device int, may be NULL) masks rows >= *n_active.
 * strict = reference summation order. */
int mb_layernorm(const float *in, float *out, const float *gain, const float *bias,
                 size_t rows, size_t width, float eps, int8_t *qx, float *sx,
                 const int *n_active, int strict, mb_stream stream);
/* Per-row int8 activation quantization of f32 rows. */
int mb_quant_rows(const float *in, size_t rows, size_t width, int8_t *qx, float *sx,
                  const int *n_active, mb_stream stream);
int mb_gelu(float *data, size_t n, int strict, const uint32_t *tanh_tab, mb_stream stream);
int mb_residual_add(float *out, const float *in, size_t n, mb_stream stream);
int mb_scale(float *data, size_t n, float scale, mb_stream stream);
int mb_clip(float *data, size_t n, mb_stream stream);
int mb_bias_add(float *out, const float *bias, size_t rows, size_t cols, mb_stream stream);
/* Constrained first-on-ties argmax over `rows` logit rows of `vocab`; writes
 * tokens[row]; when codes != NULL also the stored code (non-codes collapse to
 * 0) and ORs eos_flag[row / tables_per_stream]. */
int mb_argmax_rows(const float *logits, size_t rows, size_t vocab, size_t codebook_size,
                   size_t eos_id, const int *allow_eos, int allow_eos_scalar,
                   unsigned *tokens, unsigned *codes, int *eos_flag, size_t tables_per_stream,
                   const int *n_active, mb_stream stream);
/* x[b] = mean_t(table_t[codes[b][t]]) + position[lens[b]] ; tables is a device
 * array of table base pointers. */
int mb_embed_frames(const float *const *tables, size_t n_tables, size_t vocab, size_t width,
                    const unsigned *codes, const float *position, const int *lens,
                    float *x, size_t batch, const int *n_active, int *status, mb_stream stream);
/* x[b] = rows[b] + position[lens[b]] */
int mb_add_position(const float *rows, const float *position, const int *lens, float *x,
                    size_t batch, size_t width, const int *n_active, mb_stream stream);
/* lens[b] += 1 for b < n_active */
/* x[b] = rows[b] + row for every live lane. */
int mb_add_row(const float *rows, const float *row, float *x, size_t batch, size_t width,
               const int *n_active, mb_stream stream);

/* One table of a stacked local-transformer frame for `batch` lanes: masked
 * first-on-ties pick, optional top-k draw with the lane's xorshift64 state
 * (src/graph.c:1551-1625), stored code, EOS report, and the embedding row of the
 * fed-back token copied to row_in as the next position's input. */
typedef struct {
    const float *logits;      /* [batch][logits_stride], vocab used */
    size_t logits_stride, vocab, codebook_size, eos_id, batch;
    const int *allow_eos;     /* [batch] or NULL (allowed) */
    const float *temperature; /* [batch] or NULL (greedy) */
    const unsigned *topk;     /* [batch] or NULL (greedy) */
    unsigned long long *rng;  /* [batch] xorshift64 states or NULL (greedy) */
    size_t table, tables, codebooks;
    unsigned *tokens;         /* [batch][tables]: the token fed back (EOS kept) */
    unsigned *codes;          /* [batch][tables]: the stored code (specials -> 0) */
    int *eos_flag;            /* [batch] set to 1 on EOS, or NULL */
    int *eos_sub;             /* [batch] min(table / codebooks) over EOS tables, or NULL */
    const float *emb_table;   /* [vocab][width]: audio_embeddings.<table>.weight */
    float *row_in;            /* [batch][width] */
    const float *next_row;    /* [width] or NULL: the next position's embedding row ... */
    float *x_out;             /* ... added to the fed-back row into x_out[batch][width] (mb_add_row's sum) */
    size_t width;
    int strict;
    const uint32_t *exp_tab;  /* strict: host-libm expf correction table or NULL */
    const int *n_active;
} mb_sample_args;
int mb_local_sample(const mb_sample_args *args, mb_stream stream);
size_t mb_local_sample_smem(size_t vocab);

/* out[t] = table[ids[t]] + position[t] for `rows` rows of `width` (ids checked by the caller). */
int mb_gather_rows(const float *table, const int *ids, const float *position, float *out, size_t rows,
                   size_t width, mb_stream stream);
/* col[t][i * kernel + k] = in[t - (kernel - 1) + k][i], zero before the first row. */
int mb_unfold_causal(const float *in, float *col, size_t rows, size_t channels, size_t kernel, mb_stream stream);
int mb_advance_lens(int *lens, size_t batch, const int *n_active, mb_stream stream);
/* End of one greedy frame for lanes below n_active: lens[b] += 1; append
 * tokens_cur[b][:] to history[*frame_idx][b][:] (rows of lane_stride lanes); record the first frame whose
 * eos_flag[b] is set in eos_frame[b] (-1 = none yet); then (one thread)
 * *frame_idx += 1 and, when min_frames (device int) is given,
 * allow_eos[:] = (*frame_idx >= *min_frames). */
int mb_frame_advance(int *lens, const unsigned *tokens_cur, unsigned *history, int *frame_idx,
                     const int *eos_flag, int *eos_frame, int *allow_eos, size_t batch,
                     size_t lane_stride, size_t tables, const int *min_frames, size_t history_frames,
                     const int *n_active, mb_stream stream);

/* ---- quantized matrix-vector products ---------------------------------- */
typedef struct {
    int qtype;            /* MB_* */
    const void *w;        /* packed weights [n][k] in the reference's layout */
    const float *scales;  /* int8: [n]; int4: [n][k/32]; else NULL */
    const float *bias;    /* [n] or NULL */
    size_t n, k;
    const int8_t *qx;     /* int8/int4: [batch][k] quantized activations */
    const float *sx;      /* int8/int4: [batch] activation scales */
    const float *x;       /* f32/f16: [batch][k] activations */
    float *out;           /* [batch][out_stride] */
    size_t out_stride;
    size_t batch;
    const int *n_active;  /* device int or NULL */
    int epilogue;         /* MB_EPI_* */
    int strict;           /* GELU epilogue: reference-order transcendental */
    const uint32_t *tanh_tab; /* strict GELU: host-libm correction table or NULL */
    /* Fused prologue (int8 weights, batch == 1): instead of reading qx/sx the
     * kernel makes them from the f32 row fx: MB_FUSE_LN layer-normalizes (gain, eps) and
     * quantizes it exactly as mb_layernorm with qx does, MB_FUSE_QUANT quantizes it as
     * mb_quant_rows does.  Every CTA repeats the row work; the step loses a launch. */
    int fuse;
    const float *fx;
    const float *fuse_gain;
    float fuse_eps;
    size_t groups;        /* >1: independent problems; pointers advance by the strides below */
    size_t w_group_stride, scale_group_stride, act_group_stride, out_group_stride;
} mb_gemv_args;
int mb_gemv(const mb_gemv_args *args, mb_stream stream);

/* The f32 logit heads and the constrained first-on-ties pick in one launch (the reference's
 * fused f32 greedy path, src/qmat.c:453-536): w [tables * vocab][k] f32, x [batch][k] f32;
 * candidates: ids below codebook_size, plus eos_id where allow_eos[stream]; writes
 * tokens[stream][table], the stored code (non-codes collapse to 0) and ORs eos_flag[stream].
 * cand_v / cand_i hold mb_heads_argmax_candidates() entries; counters [batch][tables] are zero
 * before the first launch (the kernel leaves them zero).  vocab a multiple of 32, k of 4. */
typedef struct {
    const float *w, *bias, *x;
    size_t tables, vocab, k, batch, codebook_size, eos_id;
    const int *allow_eos, *n_active;
    float *cand_v;
    unsigned *cand_i, *counters;
    unsigned *tokens, *codes;
    int *eos_flag;
} mb_heads_argmax_args;
size_t mb_heads_argmax_candidates(size_t batch, size_t tables, size_t vocab);
int mb_heads_argmax_f32_supported(size_t vocab, size_t k);
int mb_heads_argmax_f32(const mb_heads_argmax_args *args, mb_stream stream);

/* Tensor-core (tcgen05) form of the product: int8 weights from 16 lanes, int4 (group 32)
 * weights from 48 lanes; same arguments and same bits as mb_gemv.  qx_rows_alloc: rows
 * the activation buffer holds. */
int mb_gemm_tc_init(void);
int mb_gemm_tc_supported(int qtype, size_t n, size_t k, size_t batch);
int mb_gemm_tc(const mb_gemv_args *args, size_t qx_rows_alloc, int *status, mb_stream stream);

/* f16 weights on the tensor cores from 16 lanes (gemm_tc_f16.cu): the f32 activations a->x
 * are first split into two f16 planes in `split` (mb_gemm_tc_f16_split_halves() halves, rows
 * of `rows_alloc` streams), then one tcgen05 product reads both.  Two launches.  Agrees with
 * mb_gemv to f32 rounding of the sums, not bit for bit. */
int mb_gemm_tc_f16_init(void);
int mb_gemm_tc_f16_supported(size_t n, size_t k, size_t batch);
size_t mb_gemm_tc_f16_split_halves(size_t rows_alloc, size_t k_max);
int mb_gemm_tc_f16(const mb_gemv_args *args, void *split, size_t rows_alloc, int *status, mb_stream stream);

/* Plain f32 row-major sgemm for the non-hot seam entries (prefill, codec):
 * C = alpha*op(A)*op(B) + beta*C. */
int mb_sgemm(int trans_a, int trans_b, size_t m, size_t n, size_t k, float alpha,
             const float *a, size_t lda, const float *b, size_t ldb, float beta, float *c,
             size_t ldc, mb_stream stream);

/* ---- codec decoder (codec.cu) ------------------------------------------- */
/* Causal convolution out[o][t] = bias[o] + sum_{i,k} w[o][i][k] * in[i][t - (kernel-1-k) * dilation]
 * over [channels][length] rows, summed per output in the order p = i * kernel + k, with the
 * epilogues the codec's residual layers need.  kernel is 3, 7 or 11; (kernel-1)*dilation <= 50. */
typedef struct {
    const float *in;          /* [ic][length] */
    const float *w_packed;    /* mb_codec_pack_conv_weight's layout */
    const float *bias;        /* [oc] */
    const float *res;         /* optional [oc][length]: v = res + v (may be `out`) */
    float *out;               /* optional [oc][length] */
    const float *alpha;       /* optional [oc]: out_act = half-Snake(v), Snake on channels < oc / 2 */
    float *out_act;
    float *acc;               /* acc_mode != 0: the residual layer's branch sum */
    const float *alpha2;      /* acc_mode 3: half-Snake applied to the finished sum, or NULL */
    const uint32_t *sin_tab;  /* strict: host-libm sinf correction table or NULL */
    size_t ic, oc, length, kernel, dilation;
    int acc_mode;             /* 0 none; 1 acc = v; 2 acc += v; 3 acc = (acc + v) / 3 */
    int clip;                 /* clamp v to [-1, 1] */
    int strict;
    int sm_count;
} mb_codec_conv_args;
size_t mb_codec_conv_groups_alloc(size_t oc);
size_t mb_codec_conv_packed_floats(size_t oc, size_t ic, size_t kernel);
/* [oc][ic][kernel] (device) -> the packed layout (device). */
int mb_codec_pack_conv_weight(const float *w, float *packed, size_t oc, size_t ic, size_t kernel, mb_stream stream);
int mb_codec_conv1d(const mb_codec_conv_args *args, mb_stream stream);
/* FSQ de-index: codes [8][frames] -> latent [32][frames]. */
int mb_codec_fsq_latent(const unsigned *codes, float *latent, size_t frames, mb_stream stream);
/* Grouped causal transposed convolution, kernel = 2 * stride, ic / oc input channels per output
 * channel: in [ic][length] -> out [oc][length * stride]; w [ic][2 * stride]. */
int mb_codec_conv_transpose(const float *in, const float *w, const float *bias, float *out, size_t ic, size_t oc,
                            size_t length, size_t stride, int strict, mb_stream stream);
/* out = half-Snake(in) (in place when out == in). */
int mb_codec_half_snake(const float *in, float *out, const float *alpha, size_t channels, size_t length,
                        size_t snake_channels, int strict, const uint32_t *sin_tab, mb_stream stream);
/* columns[(i * kernel + k)][t] = in[i][t - (kernel-1-k) * dilation], zero before the start. */
int mb_codec_im2col(const float *in, float *col, size_t ic, size_t length, size_t kernel, size_t dilation,
                    mb_stream stream);

/* The same convolution on tcgen05 tensor cores (codec_tc.cu), fast mode: operands are f16
 * hi/lo planes, channels contiguous.  x_planes: [2][length][cp_in] halves (plane stride
 * x_plane_stride halves), cp = channels rounded up to 64, pad columns zero or finite under
 * zero weights.  act_planes receive half-Snake(v) in the same layout for the next convolution. */
typedef struct {
    const void *x_planes;
    size_t x_plane_stride;
    const void *w_packed;     /* mb_codec_tc_pack_weight's layout */
    float scale;              /* the power of two the packed weights carry */
    const float *channel_table; /* mb_codec_tc_channel_table: bias, the Snake constants of the epilogue */
    int has_alpha;            /* act_planes = half-Snake(v) with the table's alpha */
    int has_alpha2;           /* acc_mode 3: half-Snake with the table's alpha2 on the finished sum */
    const float *res;
    float *out;
    void *act_planes;
    size_t act_plane_stride;
    float *acc;
    size_t ic, oc, length, kernel, dilation;
    int acc_mode;
    int *status;              /* device status word: bits 8 / 16 on a bounded wait running out */
    int sm_count;
    /* Products over rows (text encoder, context prefill) use the same kernel with time = row:
     * x_planes [2][rows][ic], result row-major out[row][o] with row stride rows_stride (a multiple
     * of 4 floats), epilogue MB_EPI_STORE / _RESIDUAL / _GELU (fast form); no bias, no table. */
    float *rows_out;
    size_t rows_stride;
    int rows_epilogue;
} mb_codec_conv_tc_args;
/* f32 rows [rows][k] with row stride ld -> f16 hi/lo planes [rows][k] each. */
int mb_split_rows_f16(const float *x, void *hi, void *lo, size_t rows, size_t k, size_t ld, mb_stream stream);
int mb_codec_tc_init(void);
void mb_codec_tc_shape(size_t oc, size_t *n_tile, size_t *tiles, size_t *cp);
size_t mb_codec_tc_packed_halves(size_t oc, size_t ic, size_t kernel);
/* [oc][ic][kernel] f32 (device) -> f16 hi/lo planes of scale * w in the tensor-core layout. */
int mb_codec_tc_pack_weight(const float *w, void *packed, size_t oc, size_t ic, size_t kernel, float scale,
                            mb_stream stream);
/* table[o] = {bias[o], alpha[o], 1 / (alpha[o] + 1e-9), alpha2[o]} (4 floats per channel, 16-byte
 * aligned); alpha / alpha2 may be NULL. */
int mb_codec_tc_channel_table(const float *bias, const float *alpha, const float *alpha2, float *table, size_t oc,
                              mb_stream stream);
/* f32 [channels][length] -> half-Snake -> f16 hi/lo planes [length][cp]. */
int mb_codec_snake_planes(const float *in, const float *alpha, void *hi, void *lo, size_t channels, size_t length,
                          mb_stream stream);
int mb_codec_conv1d_tc(const mb_codec_conv_tc_args *args, mb_stream stream);

/* ---- attention ----------------------------------------------------------- */
typedef struct {
    const float *q;       /* [batch][q_stride], head h at h*head_width */
    size_t q_stride;
    const float *k_new;   /* self: new K rows [batch][q_stride] (appended at position); cross: NULL */
    const float *v_new;
    float *k_cache;       /* slot 0 base for this layer: [capacity][cache_stride] */
    float *v_cache;
    size_t slot_stride;   /* floats between consecutive slots' caches */
    const int *slots;     /* [batch] slot of each lane, NULL = identity */
    const int *lens;      /* [batch] position of each lane (valid = len+1); NULL = scalars below */
    size_t position, valid;
    const int *valid_per_slot; /* lens == NULL only: rows attended by the lane in slot s (<= valid), or NULL */
    size_t cache_stride, heads, head_width;
    size_t cache_rows;    /* rows addressable from k_cache/v_cache (all slots); 0 = up to valid/position */
    float scale;
    float *out;           /* [batch][out_stride] */
    size_t out_stride;
    int8_t *qx;           /* optional fused per-row quantization of out */
    float *sx;
    size_t batch;
    const int *n_active;
    int strict;
    const uint32_t *exp_tab; /* strict: host-libm correction table or NULL */
    /* scratch of the chunked kernel (fast mode): mb_attention_scratch_floats()
     * floats and mb_attention_counters() counters, the counters zero before
     * first use (the kernel leaves them zero).  Launches that share scratch
     * must not overlap on the device. */
    float *partials;
    unsigned *counters;
    int sm_count;         /* SMs of the device (sizes the split); 0 = one chunk per CTA */
    int *status;          /* device error word (nonzero = bad argument seen) */
    int early_prefetch;   /* 1: lane state and cache rows below the position were written at least two
                           * launches before this one, so the kernel may request its first cache tiles
                           * before it waits for its predecessor (programmatic dependent launch) */
    unsigned *launched;   /* optional: incremented by the number of kernels the call enqueued */
    int short_cache;      /* 1: a cache that never holds more than 32 rows (the local transformer's): take the
                           * one-CTA-per-stream kernel.  Strict mode: the same bits as the other kernels; fast
                           * mode: its own (sequential) sums, so a caller must use it for every call on that cache */
    int softmax_inverse;  /* strict: weights e * (1 / sum) as the reference's multi-row self attention forms
                           * them (softmax_row_inplace, src/graph.c:245-257), not e / sum */
} mb_attn_args;
int mb_attention(const mb_attn_args *args, mb_stream stream);
size_t mb_attention_scratch_floats(size_t batch, size_t heads, size_t max_valid, size_t head_width);
size_t mb_attention_counters(size_t batch, size_t heads);

/* The cross-attention block of one decoder layer for a batch of streams, one CTA per
 * stream (src/graph.c:3213-3256): layer norm of the residual row (gain_query) with int8
 * quantization, the query product, attention over the stream's constant cross K/V rows,
 * int8 quantization of the context, the output product added to the residual row, and the
 * next layer norm (gain_ff) with int8 quantization for the feed-forward product.  int8
 * weights only; the arithmetic and its order are those of the separate launches
 * (mb_layernorm, mb_gemv / mb_gemm_tc, mb_attention) in the same mode (strict or not), so the
 * bits are the same. */
typedef struct {
    float *x;                    /* [batch][width] residual rows, updated in place */
    const float *gain_query;     /* [width] */
    const float *gain_ff;        /* [width] */
    int qtype;                   /* MB_INT8 or MB_INT4: the format of both weights */
    const int8_t *wq;            /* int8 [xw][width] row-major; int4 [xw][width / 2] */
    const float *wq_scales;      /* int8 [xw]; int4 [xw][width / 32] */
    const int8_t *wo;            /* int8 [width][xw] row-major; int4 [width][xw / 2] */
    const float *wo_scales;      /* int8 [width]; int4 [width][xw / 32] */
    const float *k_cache;        /* cross K rows of this layer, slot 0 */
    const float *v_cache;
    size_t slot_stride;          /* floats between slots */
    size_t cache_rows;           /* rows spanned by all slots (tensor-map extent) */
    const int *slots;            /* [batch] or NULL (lane b uses slot b) */
    const int *n_active;
    size_t batch, width, xw, rows;   /* rows: most text states a stream attends over */
    const int *rows_per_slot;    /* [slots] text states of the stream in each slot (1 .. rows), or NULL: rows */
    float scale, eps;
    int8_t *qx;                  /* [batch][width] out: quantized second norm */
    float *sx;                   /* [batch] */
    int *status;
    int strict;                  /* reference summation order and host-libm expf (any lane count) */
    const uint32_t *exp_tab;     /* strict: host-libm correction table or NULL */
} mb_cross_block_args;
int mb_cross_block_init(void);
int mb_cross_block_supported(size_t width, size_t xw, size_t rows);
int mb_cross_block(const mb_cross_block_args *args, mb_stream stream);

#ifdef __cplusplus
}
#endif
#endif
