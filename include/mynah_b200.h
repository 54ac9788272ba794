/* C ABI of libmynah_b200: a B200 (sm_100a) backend for the Magpie decoder step
 * of mynah-tts.
 *
 * Part 1 is the drop-in seam: the symbols mynah-tts's src/backend.c binds for
 * its CUDA device (declared there at src/backend.c:105-135, defined by
 * gpu/cuda/backend_cuda.cu in the reference), with the same names, argument
 * order and error convention -- 0 on success, -1 on failure with a message
 * written to (error, error_capacity); nothing prints, nothing aborts.  Linking
 * this library in place of backend_cuda.o needs no change to the callers.
 * Five further `mynah_cuda_*` entries implement the resident-attention ops of
 * src/backend.h:135-179 that the reference wires only for its Metal device
 * (src/backend.c:404-428); assigning them in the CUDA branch of
 * mynah_backend_open lights up the resident decode step of
 * src/graph.c:3363-3488 unchanged.
 *
 * Part 2 is an extension the reference's seam has no counterpart for: weight
 * quantization behind the seam (the reference's quantized products bypass the
 * backend, src/qmat.c:773-788), a whole-step batched decoder object, and a
 * device-resident greedy loop.
 *
 * All pointers named dev_* are device pointers obtained from this library;
 * `weight`/`bias`/`gain` arguments of part 1 are HOST pointers that stay valid
 * and unchanged for the life of the backend: they key an internal device cache,
 * as in the reference (gpu/cuda/backend_cuda.cu:205-219).
 */
#ifndef MYNAH_B200_H
#define MYNAH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
/* Every declaration below is an exported symbol of the shared library. */
#pragma GCC visibility push(default)

/* ===================================================================== *
 * Part 1: the backend seam (src/backend.h of mynah-tts)
 * ===================================================================== */

/* src/backend.h:10-25 */
typedef int (*mynah_backend_matmul_fn)(void *, const float *, float *, size_t, size_t, size_t,
                                       const float *, const float *, char *, size_t);
typedef void (*mynah_backend_close_fn)(void *);
typedef int (*mynah_backend_self_test_fn)(void *, char *, size_t);
typedef int (*mynah_backend_sgemm_fn)(void *, int trans_a, int trans_b, size_t m, size_t n,
                                      size_t k, float alpha, const float *a, size_t lda,
                                      const float *b, size_t ldb, float beta, float *c,
                                      size_t ldc, char *, size_t);

/* Replaces mynah_backend_cuda_open (src/backend.c:106-109,
 * gpu/cuda/backend_cuda.cu:543-568).  Device = MYNAH_B200_DEVICE (default 0);
 * weight format = MYNAH_QUANT (f32 default | f16 | int8 | int4, the values of
 * src/qmat.c:571-576); MYNAH_B200_STRICT=1 selects reference-order reductions.
 * The returned matmul/sgemm take HOST buffers and synchronize. */
int mynah_backend_cuda_open(void **state, mynah_backend_matmul_fn *matmul,
                            mynah_backend_sgemm_fn *sgemm, mynah_backend_close_fn *close,
                            mynah_backend_self_test_fn *self_test, char *error,
                            size_t error_capacity);

/* src/backend.h:78-93,181-186 / src/backend.c:111-123 */
int mynah_cuda_upload(void *state, const float *host, size_t n, float **dev_ptr, char *error, size_t cap);
int mynah_cuda_download(void *state, const float *dev_ptr, float *host, size_t n, char *error, size_t cap);
int mynah_cuda_sync(void *state, char *error, size_t cap);
int mynah_cuda_dev_alloc(void *state, size_t n, float **dev_ptr, char *error, size_t cap);
void mynah_cuda_dev_free(void *state, float *dev_ptr);
int mynah_cuda_h2d(void *state, const float *host, float *dev_ptr, size_t n, char *error, size_t cap);
int mynah_cuda_d2h(void *state, const float *dev_ptr, float *host, size_t n, char *error, size_t cap);

/* Element-wise and normalization ops on device rows (src/backend.h:54-56,
 * 103-127; kernels gpu/cuda/backend_cuda.cu:33-108 in the reference). */
int mynah_cuda_gelu_dev(void *state, float *dev_data, size_t n, char *error, size_t cap);
int mynah_cuda_gelu_inplace(void *state, float *dev_data, size_t n, char *error, size_t cap);
int mynah_cuda_layer_norm_dev(void *state, const float *dev_in, float *dev_out, const float *gain,
                              const float *bias, size_t rows, size_t width, char *error, size_t cap);
int mynah_cuda_layer_norm_inplace(void *state, const float *dev_in, float *dev_out,
                                  const float *gain, size_t rows, size_t width, char *error,
                                  size_t cap);
int mynah_cuda_residual_add_dev(void *state, float *dev_out, const float *dev_in, size_t n,
                                char *error, size_t cap);
int mynah_cuda_residual_inplace(void *state, float *dev_out, const float *dev_in, size_t n,
                                char *error, size_t cap);

/* out[rows,ow] = in[rows,iw] @ W[ow,iw]^T + bias (src/backend.h:58,95-101,
 * 66-71).  With MYNAH_QUANT set, products of at most 16 rows and iw <= 8192
 * use the packed weight with per-row int8 activations exactly as
 * mynah_qmat_linear_resolved does on the CPU (src/qmat.c:768-818); larger
 * calls and int4 with iw not a multiple of 32 stay f32. */
int mynah_cuda_matmul_dev(void *state, const float *dev_in, float *dev_out, size_t rows, size_t iw,
                          size_t ow, const float *weight, const float *bias, char *error, size_t cap);
int mynah_cuda_matmul_d2d(void *state, const float *dev_in, float *dev_out, size_t rows, size_t iw,
                          size_t ow, const float *weight, const float *bias, char *error, size_t cap);
int mynah_cuda_matmul_to_dev(void *state, const float *host_in, float *dev_out, size_t rows,
                             size_t iw, size_t ow, const float *weight, const float *bias,
                             char *error, size_t cap);
int mynah_cuda_matmul_graph(void *state, const float *host_in, float *host_out, size_t rows,
                            size_t iw, size_t ow, const float *weight, const float *bias,
                            char *error, size_t cap);
int mynah_cuda_matvec_dev(void *state, const float *dev_in, float *dev_out, size_t K, size_t N,
                          const float *weight, const float *bias, char *error, size_t cap);
int mynah_cuda_sgemm_dev(void *state, int trans_a, int trans_b, size_t m, size_t n, size_t k,
                         float alpha, const float *dev_a, size_t lda, const float *dev_b,
                         size_t ldb, float beta, float *dev_c, size_t ldc, char *error, size_t cap);

/* Resident single-token attention and helpers: src/backend.h:135-179.  The
 * reference's CUDA file has no counterpart (its vtable leaves them NULL). */
int mynah_cuda_batch_begin(void *state, char *error, size_t cap);
int mynah_cuda_self_attention_dev(void *state, const float *dev_qkv, float *dev_k_cache,
                                  float *dev_v_cache, size_t position, size_t cache_stride,
                                  size_t valid, size_t heads, size_t head_width, float scale,
                                  float *dev_out, char *error, size_t cap);
int mynah_cuda_cross_attention_dev(void *state, const float *dev_q, const float *dev_k_cache,
                                   const float *dev_v_cache, size_t valid, size_t cache_stride,
                                   size_t heads, size_t head_width, float scale, float *dev_out,
                                   char *error, size_t cap);
int mynah_cuda_copy_dev(void *state, float *dev_dst, const float *dev_src, size_t n, char *error, size_t cap);
int mynah_cuda_scale_dev(void *state, float *dev_data, size_t n, float scale, char *error, size_t cap);
int mynah_cuda_clip_dev(void *state, float *dev_data, size_t n, char *error, size_t cap);
int mynah_cuda_argmax_dev(void *state, const float *dev_logits, size_t vocab, size_t codebook_size,
                          size_t eos_id, int allow_eos, unsigned *argmax, char *error, size_t cap);

/* Host-side GELU helpers the reference exports for calibration
 * (src/backend.h:63-64): data is a HOST buffer, processed on the device. */
int mynah_cuda_gelu_host(void *state, float *host_data, size_t n, char *error, size_t cap);
int mynah_cuda_gelu_host_f64(void *state, float *host_data, size_t n, char *error, size_t cap);

/* NanoCodec ops (src/backend.h:59-61,128-133).  snake_dev: device signal in place, HOST alpha.
 * im2col: device pointers.  conv1d: host weight/bias as cache keys; HOST input/output served
 * synchronously (the contract of the reference's CUDA backend, gpu/cuda/backend_cuda.cu:746-810)
 * and DEVICE input/output enqueued without a sync (what decode_codec_resident passes,
 * src/graph.c:2552-2556) -- the kind of `in` decides; kernels other than 3, 7, 11 return -1 so
 * the caller keeps its CPU path.  conv_transpose_dev (wired only for Metal in the reference;
 * an integrator who wires the resident-attention ops must wire it too, or decode_codec_resident
 * fails instead of falling back): the codec's shape only (one output channel per group, kernel
 * = 2 * stride).  The whole codec as one device-resident pass is mynah_b200_codec_decode. */
int mynah_cuda_snake_dev(void *state, float *dev_data, const float *alpha, size_t channels,
                         size_t length, size_t snake_channels, char *error, size_t cap);
int mynah_cuda_im2col(void *state, const float *in, float *cols, int in_ch, int length, int kernel,
                      int dilation, char *error, size_t cap);
int mynah_cuda_conv1d(void *state, const float *in, float *out, int in_ch, int out_ch, int length,
                      int kernel, int dilation, const float *weight, const float *bias,
                      char *error, size_t cap);
int mynah_cuda_conv_transpose_dev(void *state, const float *in, float *out, int in_ch, int out_ch,
                                  int length, int output_length, int kernel, int stride, int groups,
                                  const float *weight, const float *bias, char *error, size_t cap);

/* ===================================================================== *
 * Part 2: extensions (no counterpart in the reference's seam)
 * ===================================================================== */

enum { MYNAH_B200_F32 = 0, MYNAH_B200_INT8 = 1, MYNAH_B200_INT4 = 2, MYNAH_B200_F16 = 3 };

/* Explicit open: device ordinal, weight format (MYNAH_B200_*), strict flag.
 * mynah_backend_cuda_open is this with values taken from the environment. */
int mynah_b200_open(void **state, int device, int quant, int strict, char *error, size_t cap);
void mynah_b200_close(void *state);
/* Run all work of this backend on the caller's CUDA stream (cudaStream_t). */
int mynah_b200_set_stream(void *state, void *cuda_stream, char *error, size_t cap);
/* 1 when this (strict) backend reproduces the host libm's expf and tanhf bit
 * for bit: correction tables are built from the host's own libm the first time
 * a strict backend is opened on a device (about 220 MB of device memory, a few
 * seconds; MYNAH_B200_LIBM_TABLES=0 skips them and strict mode then uses the
 * correctly rounded functions). */
int mynah_b200_libm_exact(const void *state);
int mynah_b200_quant(const void *state);
int mynah_b200_strict(const void *state);
/* Device-time stopwatch: two CUDA events recorded on the backend's stream;
 * _stop waits for the second and returns the time between them. */
int mynah_b200_timer_start(void *state, char *error, size_t cap);
int mynah_b200_timer_stop(void *state, float *elapsed_ms, char *error, size_t cap);
/* Number of kernels this library has launched on `state` (graph replays count
 * their kernel nodes). */
unsigned long long mynah_b200_launch_count(const void *state);

/* Pack a HOST f32 weight [n,k] on the device with the reference's quantizers
 * (src/qmat.c:39-91,650-655) and copy the packed bytes and scales back:
 * int8 -> q[n*k] + scales[n]; int4 -> q[n*k/2] + scales[n*k/32]; f16 ->
 * q[n*k] halves, scales untouched. */
int mynah_b200_pack_weight(void *state, int quant, const float *host_w, size_t n, size_t k,
                           void *host_q, float *host_scales, char *error, size_t cap);
/* Per-row int8 activation quantization of HOST rows (src/qmat.c:93-113). */
int mynah_b200_quantize_act(void *state, const float *host_x, size_t rows, size_t k,
                            int8_t *host_q, float *host_sx, char *error, size_t cap);
/* HOST-buffer single op: out[count,n] = LN(x)[count,k] @ W[n,k]^T + bias, the
 * LayerNorm (gain only, eps 1e-5) skipped when ln_gain is NULL; W, bias and
 * ln_gain are cached by host pointer.  The reference's counterpart is
 * layer_norm + mynah_qmat_linear_resolved (src/graph.c:147-150,
 * src/qmat.c:768-818). */
int mynah_b200_qmat_linear(void *state, const float *weight, const float *x, float *out,
                           size_t count, size_t k, size_t n, const float *bias,
                           const float *ln_gain, char *error, size_t cap);
/* Device-resident form of the same op over `groups` independent problems laid
 * out back to back (weights from mynah_b200_pool_*): used to stream a pool of
 * distinct matrices larger than L2 through the product kernel in one launch
 * sequence.  dev_x is [groups][k], dev_out [groups][n]. */
int mynah_b200_pool_create(void *state, const float *host_w, size_t n, size_t k, size_t groups,
                           const float *host_bias, const float *host_gain, void **pool,
                           char *error, size_t cap);
void mynah_b200_pool_destroy(void *pool);
int mynah_b200_pool_linear(void *pool, const float *dev_x, float *dev_out, char *error, size_t cap);
size_t mynah_b200_pool_bytes_per_pass(const void *pool);

/* Diagnostic: mean device time (microseconds) of one int8 product
 * out[batch,n] = qx[batch,k] W[n,k]^T launched `iters` times back to back on
 * resident synthetic data; path 0 = SIMT kernel, 1 = tensor-core kernel
 * (batch >= 16); epilogue 0 store, 1 residual add, 2 GELU. */
int mynah_b200_time_product(void *state, size_t n, size_t k, size_t batch, int path, int epilogue,
                            size_t iters, float *us_per_launch, char *error, size_t cap);

/* ---- whole-step decoder --------------------------------------------------- */
/* Host weight pointers of one decoder layer, in the order of
 * decoder_layer_resolved (src/graph.c:2795-2804). */
typedef struct {
    const float *norm_self;         /* [width] */
    const float *norm_xattn_query;  /* [width] */
    const float *norm_pos_ff;       /* [width] */
    const float *qkv_w;             /* [3*width, width] */
    const float *o_self_w;          /* [width, width] */
    const float *q_cross_w;         /* [xattn_width, width] */
    const float *o_cross_w;         /* [width, xattn_width] */
    const float *ffn_up_w;          /* [4*width, width] */
    const float *ffn_down_w;        /* [width, 4*width] */
    /* optional (both or neither): the tensors decoder_cache_init uses to make the cross
     * K/V of a request (src/graph.c:3002-3016); they enable _slot_prefill */
    const float *norm_xattn_memory; /* [width] */
    const float *kv_cross_w;        /* cross_attention.kv_net.weight [2*xattn_width, width] */
} mynah_b200_layer_weights;

typedef struct {
    size_t layers, width, heads, xattn_width; /* head_width = width/heads, ffn = 4*width */
    size_t memory_length;  /* most text states (rows of cross K/V) a request may have; each slot
                            * keeps its own request's count (decoder_cache.memory_length,
                            * src/graph.c:2820) */
    size_t capacity;       /* self-KV rows per slot (src/graph.c:3804-3806) */
    size_t slots;          /* resident requests (each owns KV) */
    size_t max_batch;      /* most lanes of one launch sequence: slots stepped together, or rows of one
                            * request prefilled together (may exceed slots for the latter) */
    size_t max_positions;  /* rows of the position table */
    const mynah_b200_layer_weights *layer; /* [layers] */
    const float *position;  /* decoder.position_embeddings.weight [max_positions, width] */
    const float *norm_out;  /* decoder.norm_out.weight [width] */
    /* optional greedy front/back ends (tables == 0 disables them) */
    size_t tables, vocab, codebook_size, eos_id;
    const float *const *embeddings; /* tables x [vocab, width]  (audio_embeddings.N.weight) */
    const float *const *head_w;     /* tables x [vocab, width] */
    const float *const *head_b;     /* tables x [vocab] */
    /* nonzero: a quantized decoder also keeps f32 copies of the layer weights, which
     * _prefill of more than 16 rows multiplies with (as the reference does) */
    int keep_f32_weights;
} mynah_b200_decoder_desc;

/* Uploads and packs every weight once (format and strictness of `state`) and
 * allocates KV for `slots` requests.  Weight host pointers need only be valid
 * during this call. */
int mynah_b200_decoder_create(void *state, const mynah_b200_decoder_desc *desc, void **decoder,
                              char *error, size_t cap);
void mynah_b200_decoder_destroy(void *decoder);

/* Load one request into a slot: its cross K/V [layers][memory_length][xattn_width]
 * as decoder_cache_init leaves them (src/graph.c:3012-3027; memory_length is the
 * REQUEST's own text length, 1 .. the decoder's, and also the layer stride of the
 * two arrays), and optionally `length` rows of existing self K/V
 * [layers][capacity][width] (what decoder_gpu_attention_init uploads,
 * src/graph.c:2929-2953).  Cross attention of the slot then covers exactly its
 * memory_length rows, whatever the other slots of a batch hold. */
int mynah_b200_decoder_slot_load(void *decoder, size_t slot, const float *cross_k,
                                 const float *cross_v, size_t memory_length, const float *self_k,
                                 const float *self_v, size_t length, char *error, size_t cap);
/* Make a slot's cross K/V on the device from the text-encoder memory
 * [memory_length][width] (HOST; 1 .. the decoder's memory_length rows): what
 * decoder_cache_init computes on the CPU (src/graph.c:3002-3027).  The slot starts
 * at length 0. */
int mynah_b200_decoder_slot_prefill(void *decoder, size_t slot, const float *memory,
                                    size_t memory_length, char *error, size_t cap);
/* Copy a slot's cross K/V back: host arrays [layers][M][xattn_width] with M the DECODER's
 * memory_length; rows at and beyond the slot's own count are not part of the request. */
int mynah_b200_decoder_slot_read_cross(void *decoder, size_t slot, float *cross_k, float *cross_v,
                                       char *error, size_t cap);
int mynah_b200_decoder_slot_length(void *decoder, size_t slot, size_t *length, char *error, size_t cap);
int mynah_b200_decoder_slot_set_length(void *decoder, size_t slot, size_t length, char *error, size_t cap);
/* Copy a slot's self K/V back: host arrays [layers][capacity][width]. */
int mynah_b200_decoder_slot_read_kv(void *decoder, size_t slot, float *self_k, float *self_v,
                                    char *error, size_t cap);
/* Run only the first n layers (then the output norm); n = layers restores. */
int mynah_b200_decoder_set_layers(void *decoder, size_t n, char *error, size_t cap);

/* Push `count` new rows [count][width] (HOST) of the request in `slot` through the stack
 * together: the contract of decoder_run with count > 1 (src/graph.c:3286-3654, the context
 * prefill) -- position embedding, all layers with causal attention among the new rows and
 * over the rows already cached, K/V appended, the slot's length advanced by count, and the
 * output-norm row of the LAST new row in out_last [width] (HOST).  count <= max_batch.
 * As in the reference, a quantized model multiplies more than 16 rows with its f32 weights
 * (keep_f32_weights) and at most 16 with the packed ones.  Synchronous. */
int mynah_b200_decoder_prefill(void *decoder, size_t slot, const float *rows, size_t count,
                               float *out_last, char *error, size_t cap);

/* One decoder step for `batch` slots: the contract of decoder_step_batch
 * (src/graph.c:3127-3284) with HOST rows -- inputs[b] and outs[b] are `width`
 * floats; position embedding, all layers, output norm; each slot's length
 * advances by one.  Synchronous. */
int mynah_b200_decoder_step_batch(void *decoder, const unsigned *slots,
                                  const float *const *inputs, float *const *outs, size_t batch,
                                  char *error, size_t cap);
/* One greedy frame for `batch` slots with HOST buffers: codes [batch][tables]
 * in, tokens [batch][tables] out (optionally the output-norm rows
 * [batch][width]): embedding mean (src/graph.c:760-804), decoder step, logit
 * heads with the constrained first-on-ties pick (src/graph.c:1538-1566).
 * Synchronous; the caller applies its own EOS policy. */
int mynah_b200_decoder_frame_batch(void *decoder, const unsigned *slots, const unsigned *codes,
                                   const int *allow_eos, unsigned *tokens, float *hidden,
                                   size_t batch, char *error, size_t cap);
/* Device-resident greedy decode: lane b runs frames[b] frames starting from
 * codes[b][tables] (HOST, updated to the last stored codes); tokens
 * [max_frames][batch][tables] (HOST) receives every picked token (rows of
 * lanes that already finished are left zero); EOS is allowed from frame
 * min_frames on and is reported in eos_frame[b] (first frame, -1 if none) but
 * does not stop a lane.  One CUDA graph launch per frame, no host round trip
 * inside the loop.  elapsed_ms (optional) receives the device time of the
 * loop measured with events on the backend's stream. */
int mynah_b200_decoder_greedy(void *decoder, const unsigned *slots, size_t batch, unsigned *codes,
                              const size_t *frames, size_t min_frames, unsigned *tokens,
                              long *eos_frame, float *elapsed_ms, char *error, size_t cap);
/* ---- local transformer and sampler (src/graph.c:806-1656) -------------------
 * The small autoregressive transformer that turns one decoder output row into the
 * `tables` tokens of a stacked frame: table t's logits come from position t, whose
 * input is the decoder row (t = 0) or the embedding of table t-1's token.  It uses
 * the decoder's embedding tables and per-table projections (desc->embeddings,
 * head_w, head_b: audio_embeddings.N / local_transformer_out_projections.N). */
typedef struct {
    const float *norm_self;    /* local_transformer.layers.N.norm_self.weight [width] */
    const float *norm_pos_ff;  /* ...norm_pos_ff.weight [width] */
    const float *qkv_w;        /* ...self_attention.qkv_net.weight [3*width, width] */
    const float *o_w;          /* ...self_attention.o_net.weight [width, width] */
    const float *ffn_up_w;     /* ...pos_ff.proj.conv.weight [4*width, width] */
    const float *ffn_down_w;   /* ...pos_ff.o_net.conv.weight [width, 4*width] */
} mynah_b200_local_layer_weights;

typedef struct {
    size_t layers;             /* model.json local_transformer_layers, 1..4 (src/graph.c:1060) */
    const mynah_b200_local_layer_weights *layer;
    const float *position;     /* local_transformer.position_embeddings.weight [position_rows, width] */
    size_t position_rows;      /* >= tables */
    size_t codebooks;          /* tables = codebooks x frame_stacking_factor */
} mynah_b200_local_desc;

/* Uploads and packs the local transformer's weights and allocates its per-lane
 * KV (tables + 1 rows, src/graph.c:1200).  Once per decoder. */
int mynah_b200_decoder_local_attach(void *decoder, const mynah_b200_local_desc *desc, char *error,
                                    size_t cap);

/* Per-request sampler settings (local_batch_item, src/graph.c:1346-1362): greedy
 * when temperature <= 0 or topk <= 1, else a draw from the top-k with the
 * request's xorshift64 state, which the call advances. */
typedef struct {
    float temperature;
    unsigned topk;
    unsigned long long rng_state;
    int allow_eos;             /* used by _local_frame only; the loops apply min_frames */
} mynah_b200_sampler;

/* One stacked frame for `batch` requests: the contract of sample_local_frame_batch
 * (src/graph.c:1374-1656) with HOST buffers.  decoder_last [batch][width] in;
 * codes [batch][tables] (stored codes, specials collapsed to 0), values (optional,
 * the tokens fed back, EOS kept), saw_eos, eos_frame (smallest table / codebooks
 * where the greedy or drawn token was EOS, -1 if none) out.  Synchronous. */
int mynah_b200_decoder_local_frame(void *decoder, const float *decoder_last, size_t batch,
                                   mynah_b200_sampler *samplers, unsigned *codes, unsigned *values,
                                   int *saw_eos, long *eos_frame, char *error, size_t cap);

/* _greedy with the local transformer in place of the logit heads: per frame embed
 * the stored codes, step the decoder, run one stacked local frame (the loop of
 * synthesize_slots, src/graph.c:4083-4183, without the codec).  tokens receives the
 * fed-back tokens of every frame; samplers [batch] (NULL: all greedy) are advanced. */
int mynah_b200_decoder_generate(void *decoder, const unsigned *slots, size_t batch, unsigned *codes,
                                const size_t *frames, size_t min_frames,
                                mynah_b200_sampler *samplers, unsigned *tokens, long *eos_frame,
                                float *elapsed_ms, char *error, size_t cap);

/* frame_batch with the local transformer: codes [batch][tables] in (the previous
 * frame's stored codes), one decoder step, one stacked local frame; codes_out, values
 * (optional), saw_eos, eos_frame as _local_frame reports them; samplers advanced.
 * Synchronous. */
int mynah_b200_decoder_frame_batch_local(void *decoder, const unsigned *slots, const unsigned *codes,
                                         mynah_b200_sampler *samplers, unsigned *codes_out,
                                         unsigned *values, int *saw_eos, long *eos_frame,
                                         size_t batch, char *error, size_t cap);

/* Continuous batching (no counterpart in the reference, whose synthesize_slots steps
 * at most 16 requests that start together and whose server never admits into a
 * running batch): `count` requests share the decoder's slots; a waiting request
 * enters as soon as a slot is free (its cross K/V are made on the device, so the
 * layer weights must carry norm_xattn_memory / kv_cross_w), every live request
 * advances one sampled frame per step, and a request leaves when EOS is seen (allowed
 * once frames_done >= min_frames) or at max_frames (src/graph.c:3912-3913).  Because a
 * request's result does not depend on its batch, codes equal what the request
 * produces alone. */
typedef struct {
    const float *memory;         /* [memory_length][width] text-encoder states (HOST) */
    size_t memory_length;        /* this request's text states, 1 .. the decoder's memory_length */
    const unsigned *start_codes; /* [tables]: the frame embedded before the first step */
    size_t max_frames, min_frames;
    mynah_b200_sampler sampler;  /* advanced; allow_eos is ignored */
    unsigned *codes;             /* out: [max_frames][tables] stored codes (caller-allocated) */
    size_t frames_done;          /* out */
    long eos_frame;              /* out: frame in which EOS was seen, -1 if none */
    size_t admitted_at;          /* out: step at which the request entered a slot */
} mynah_b200_request;
int mynah_b200_decoder_serve(void *decoder, mynah_b200_request *requests, size_t count,
                             size_t *steps, char *error, size_t cap);

/* ---- text encoder (src/graph.c:709-748) -------------------------------------------
 * encode_text: token ids -> the text-encoder states the decoder cross-attends (the
 * `memory` of _slot_prefill and of mynah_b200_request).  Host weight pointers of one
 * layer, names as the reference resolves them (src/graph.c:662-699, 291-296, 386-391): */
typedef struct {
    const float *norm_self;    /* encoder.layers.N.norm_self.weight [width] */
    const float *norm_pos_ff;  /* ...norm_pos_ff.weight [width] */
    const float *qkv_w;        /* ...self_attention.qkv_net.weight [3*width, width] */
    const float *o_w;          /* ...self_attention.o_net.weight [width, width] */
    const float *ffn_proj_w;   /* ...pos_ff.proj.conv.weight [4*width, width, kernel] */
    const float *ffn_out_w;    /* ...pos_ff.o_net.conv.weight [width, 4*width, kernel] */
} mynah_b200_encoder_layer_weights;

typedef struct {
    size_t layers, width, heads, kernel;   /* the reference runs 12 heads and kernel 3 (src/graph.c:735) */
    size_t vocab;              /* rows of text_embedding.weight */
    size_t max_length;         /* text_max_length: rows of encoder.position_embeddings.weight, <= 1024 */
    const mynah_b200_encoder_layer_weights *layer;   /* [layers] */
    const float *embedding;    /* text_embedding.weight [vocab, width] */
    const float *position;     /* encoder.position_embeddings.weight [max_length, width] */
    const float *norm_out;     /* encoder.norm_out.weight [width] */
} mynah_b200_encoder_desc;

/* Uploads the weights (kept in f32 whatever the backend's format: the reference's encoder
 * never takes the quantized path).  Host pointers need only be valid during the call. */
int mynah_b200_encoder_create(void *state, const mynah_b200_encoder_desc *desc, void **encoder,
                              char *error, size_t cap);
void mynah_b200_encoder_destroy(void *encoder);
/* ids [count] (HOST) -> out [count][width] (HOST): the contract of encode_text; ids outside
 * the vocabulary and count outside 1..max_length are refused with the reference's messages.
 * Synchronous. */
int mynah_b200_encoder_encode(void *encoder, const int *ids, size_t count, float *out, char *error,
                              size_t cap);

/* ---- codec decoder (src/graph.c:2640-2780) -----------------------------------------
 * decode_codec: FSQ indices -> audio samples.  Host weight pointers under the names the
 * reference resolves (src/graph.c:2545-2626, 2360-2395): */
typedef struct {
    const float *in_alpha;    /* ...res_blocks.B.res_blocks.D.input_activation.activation.snake_act.alpha [C] */
    const float *in_w, *in_b; /* ...input_conv.conv.{weight [C, C, kernel], bias [C]} */
    const float *skip_alpha;  /* ...skip_activation.activation.snake_act.alpha [C] */
    const float *skip_w, *skip_b; /* ...skip_conv.conv.{weight [C, C, kernel], bias [C]} */
} mynah_b200_codec_block;

typedef struct {
    const float *alpha;       /* audio_decoder.activations.S.activation.snake_act.alpha [2C] */
    const float *up_w, *up_b; /* audio_decoder.up_sample_conv_layers.S.conv.{weight [2C, 1, 2 * rate], bias [C]} */
    mynah_b200_codec_block block[3][3];   /* audio_decoder.res_layers.S: [kernel 3, 7, 11][dilation 1, 3, 5] */
} mynah_b200_codec_stage;

typedef struct {
    size_t base;              /* channels after the first convolution: 864 in the reference; a multiple of 32 */
    size_t max_frames;        /* longest request, <= 4096; activations take base * 32 * 5 * 4 bytes per frame */
    const float *pre_w, *pre_b;       /* audio_decoder.pre_conv.conv.{weight [base, 32, 7], bias} */
    mynah_b200_codec_stage stage[5];  /* rates 8, 8, 4, 2, 2; channels halve per stage */
    const float *post_alpha;          /* audio_decoder.post_activation.activation.snake_act.alpha [base / 32] */
    const float *post_w, *post_b;     /* audio_decoder.post_conv.conv.{weight [1, base / 32, 3], bias [1]} */
    int arithmetic;           /* 0: the backend's mode; 1: reference order (bit-identical samples, SIMT);
                                 2: tensor cores (samples within 1e-4) whatever the backend's mode -- the
                                 audio comes after the token stream, so a strict decoder may pair with it */
} mynah_b200_codec_desc;

int mynah_b200_codec_create(void *state, const mynah_b200_codec_desc *desc, void **codec, char *error, size_t cap);
void mynah_b200_codec_destroy(void *codec);
size_t mynah_b200_codec_samples_per_frame(void);   /* 1024 */
/* codes [8][frames] (HOST, FSQ index per group and frame) -> samples [frames * 1024] (HOST),
 * clipped to [-1, 1]: the contract of decode_codec.  Synchronous. */
int mynah_b200_codec_decode(void *codec, const unsigned *codes, size_t frames, float *samples,
                            size_t *sample_count, char *error, size_t cap);
/* For stage-wise checks: stop_after = 1 returns the first convolution's output [base][frames],
 * 2 + s the output of stage s [base >> (s + 1)][its length]; 0 = the samples. */
int mynah_b200_codec_decode_partial(void *codec, const unsigned *codes, size_t frames, int stop_after,
                                    float *out, size_t out_capacity, size_t *count, char *error, size_t cap);
/* Device time of one decode, averaged over `repeats` back-to-back decodes after one warm-up. */
int mynah_b200_codec_time(void *codec, const unsigned *codes, size_t frames, int repeats,
                          float *ms_per_decode, char *error, size_t cap);

/* Bytes of weights one step reads, and of KV one slot at `length` reads. */
size_t mynah_b200_decoder_weight_bytes(const void *decoder);
size_t mynah_b200_decoder_kv_bytes(const void *decoder, size_t length);

/* Per-call-site device timing of the step (the reference's MYNAH_TIMING=1
 * phase report, src/graph.c:83-88, is the nearest counterpart).  While enabled
 * every step runs as individual launches, each bracketed by two CUDA events on
 * the backend's stream, instead of a graph replay; _read synchronizes and
 * returns, per class, the launches seen and their summed device time. */
#define MYNAH_B200_PROFILE_CLASSES 16
int mynah_b200_decoder_profile(void *decoder, int enable, char *error, size_t cap);
int mynah_b200_decoder_profile_read(void *decoder, unsigned long long *launches, double *ms,
                                    size_t n, char *error, size_t cap);
const char *mynah_b200_profile_class_name(size_t cls);

/* No counterpart in the reference.  Self-attention with the contract of
 * mynah_cuda_self_attention_dev for callers that are not allowed to allocate
 * device memory (a real-time audio thread, a plugin living in a host whose
 * memory pool is not its own, a context that must not grow): it takes no
 * backend state and never calls cudaMalloc/cudaFree or any allocating routine.
 * The kernel's scratch (per-chunk partial results, one merged row, arrival
 * counters) sits in a fixed ~450 KB array inside the library image that every
 * GPU loading the library holds until the process exits.
 * Limits: at most 4096 attended rows, heads*head_width <= 768, <= 32 heads,
 * head_width a power-of-two multiple of 4 up to 128, 16-byte aligned buffers;
 * anything else is refused with a message.  The first call on a device looks
 * up the array's device address (cudaGetSymbolAddress); make that first call
 * before any stream capture.  All calls share the one array: calls that overlap
 * on the GPU race, so serialize them.  cuda_stream is a cudaStream_t (may be
 * NULL); the work is enqueued, not synchronized. */
int mynah_b200_self_attention_static(const float *dev_qkv, float *dev_k_cache, float *dev_v_cache,
                                     size_t position, size_t cache_stride, size_t valid,
                                     size_t heads, size_t head_width, float scale, float *dev_out,
                                     void *cuda_stream, char *error, size_t cap);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif
