/* The text encoder on one B200 (extension of the backend seam), C11.
 *
 * Restates encode_text / transformer_stack of mynah-tts (src/graph.c:709-748, 634-707) as
 * one device-resident sequence per request: token embedding rows plus position rows, then
 * per layer LayerNorm -> qkv product -> causal self-attention among the rows -> output
 * product -> residual -> LayerNorm -> causal convolution (kernel 3) feed-forward as two
 * products over unfolded rows with the tanh GELU between -> residual, and the output norm.
 * Every product is f32 whatever the backend's weight format: the reference's `linear`
 * bypasses the quantized path here (src/graph.c:259-265).  The rows of a request ride as
 * lanes: the self-attention kernel reads K and V straight out of the qkv rows (cache stride
 * 3 * width) with lane t attending rows 0..t, weights e * (1 / sum) as softmax_row_inplace
 * forms them (src/graph.c:245-257, 446-450).  In fast mode the four products of a layer run on
 * the tensor cores (k_conv1d_tc of codec_tc.cu with time = row): the rows are split into f16
 * hi/lo planes and the kernel-3 convolutions read their taps as the same rows shifted, so no
 * unfolded copy is made; strict mode keeps the sequential f32 sums.
 */
#include "host_common.h"
#include "../../include/mynah_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    void *w;          /* tensor-core layout (fast mode): f16 hi/lo planes of scale * weight */
    float scale;
} enc_tc;

typedef struct {
    float *norm_self, *norm_ff;
    mb_dev_weight qkv, o, proj, out;      /* f32: [3W][W], [W][W], [F][W*K], [W][F*K] */
    enc_tc qkv_tc, o_tc, proj_tc, out_tc;
} enc_layer;

typedef struct {
    mb_state *st;
    size_t layers, width, heads, kernel, vocab, max_length, ffn;
    enc_layer *L;
    float *embedding, *position, *norm_out;
    float *x, *nrm, *qkv, *ctx, *hidden, *col, *out, *partials;
    int use_tc;       /* fast mode: products and convolutions on the tensor cores */
    void *planes;     /* f16 hi/lo planes of the rows that feed a product: [2][max_length][ffn] */
    unsigned *counters;
    int *d_ids, *d_lens, *d_count;
    int *h_ids;      /* pinned: ids, then positions */
    float *h_out;    /* pinned */
} mb_encoder;

static int e_malloc(void **p, size_t bytes, char *error, size_t cap) {
    *p = NULL;
    return mb_cuda((int)cudaMalloc(p, bytes ? bytes : 4u), "cudaMalloc(encoder)", error, cap);
}
/* Tensor-core layout of a weight [oc][ic][kernel] that already lies on the device in f32;
 * host_w only gives the largest magnitude, for the power-of-two scale. */
static int e_tc_pack(mb_encoder *e, enc_tc *dst, const mb_dev_weight *dev, const float *host_w, size_t oc, size_t ic,
                     size_t kernel, char *error, size_t cap) {
    float amax = 0.0f;
    for (size_t i = 0; i < oc * ic * kernel; ++i) {
        const float v = fabsf(host_w[i]);
        if (v > amax) amax = v;
    }
    int ex = 0;
    if (amax > 0.0f) {
        (void)frexpf(amax, &ex);
        ex = 14 - ex;
    }
    if (ex > 30) ex = 30;
    if (ex < -30) ex = -30;
    dst->scale = ldexpf(1.0f, ex);
    if (e_malloc(&dst->w, mb_codec_tc_packed_halves(oc, ic, kernel) * 2u, error, cap) != 0) return -1;
    MB_TRY(mb_codec_tc_pack_weight((const float *)dev->w, dst->w, oc, ic, kernel, dst->scale, e->st->stream), "pack weight");
    e->st->launches += 1u;
    return 0;
}

static int e_upload(float **dst, const float *host, size_t n, char *error, size_t cap) {
    if (e_malloc((void **)dst, n * sizeof(float), error, cap) != 0) return -1;
    return mb_cuda((int)cudaMemcpy(*dst, host, n * sizeof(float), cudaMemcpyHostToDevice), "upload", error, cap);
}

void mynah_b200_encoder_destroy(void *encoder) {
    mb_encoder *e = (mb_encoder *)encoder;
    if (e == NULL) return;
    cudaSetDevice(e->st->device);
    cudaStreamSynchronize(e->st->stream);
    if (e->L != NULL) {
        for (size_t l = 0; l < e->layers; ++l) {
            cudaFree(e->L[l].norm_self); cudaFree(e->L[l].norm_ff);
            mb_weight_release(&e->L[l].qkv); mb_weight_release(&e->L[l].o);
            mb_weight_release(&e->L[l].proj); mb_weight_release(&e->L[l].out);
            cudaFree(e->L[l].qkv_tc.w); cudaFree(e->L[l].o_tc.w); cudaFree(e->L[l].proj_tc.w); cudaFree(e->L[l].out_tc.w);
        }
        free(e->L);
    }
    void *dev[] = {e->embedding, e->position, e->norm_out, e->x, e->nrm, e->qkv, e->ctx, e->hidden, e->col, e->out,
                   e->partials, e->counters, e->d_ids, e->d_lens, e->d_count, e->planes};
    for (size_t i = 0; i < sizeof(dev) / sizeof(dev[0]); ++i) cudaFree(dev[i]);
    if (e->h_ids != NULL) cudaFreeHost(e->h_ids);
    if (e->h_out != NULL) cudaFreeHost(e->h_out);
    free(e);
}

int mynah_b200_encoder_create(void *state, const mynah_b200_encoder_desc *desc, void **encoder, char *error, size_t cap) {
    mb_state *st = (mb_state *)state;
    if (st == NULL || desc == NULL || encoder == NULL) {
        mb_set_error(error, cap, "invalid encoder arguments");
        return -1;
    }
    *encoder = NULL;
    if (desc->layers == 0 || desc->width == 0 || desc->heads == 0 || desc->width % desc->heads != 0 ||
        desc->kernel == 0 || desc->vocab == 0 || desc->max_length == 0 || desc->max_length > 1024u ||
        desc->layer == NULL || desc->embedding == NULL || desc->position == NULL || desc->norm_out == NULL) {
        mb_set_error(error, cap, "invalid encoder shape");
        return -1;
    }
    MB_TRY(cudaSetDevice(st->device), "cudaSetDevice");
    mb_encoder *e = (mb_encoder *)calloc(1, sizeof(*e));
    if (e == NULL) {
        mb_set_error(error, cap, "out of memory creating encoder");
        return -1;
    }
    e->st = st;
    e->layers = desc->layers; e->width = desc->width; e->heads = desc->heads; e->kernel = desc->kernel;
    e->vocab = desc->vocab; e->max_length = desc->max_length;
    e->ffn = 4u * desc->width;                                    /* src/graph.c:735 */
    const size_t W = e->width, F = e->ffn, K = e->kernel, T = e->max_length;
    {
        const char *no_tc = getenv("MYNAH_B200_NO_TC");
        e->use_tc = !st->strict && !(no_tc != NULL && strcmp(no_tc, "0") != 0) && W % 64u == 0;
    }
    int ok = 1;
#define E_TRY(expr) do { if (ok && (expr) != 0) ok = 0; } while (0)
    e->L = (enc_layer *)calloc(e->layers, sizeof(enc_layer));
    if (e->L == NULL) { mb_set_error(error, cap, "out of memory"); ok = 0; }
    for (size_t l = 0; ok && l < e->layers; ++l) {
        const mynah_b200_encoder_layer_weights *s = &desc->layer[l];
        enc_layer *L = &e->L[l];
        E_TRY(e_upload(&L->norm_self, s->norm_self, W, error, cap));
        E_TRY(e_upload(&L->norm_ff, s->norm_pos_ff, W, error, cap));
        E_TRY(mb_weight_build(st, s->qkv_w, 3u * W, W, MB_F32, &L->qkv, error, cap));
        E_TRY(mb_weight_build(st, s->o_w, W, W, MB_F32, &L->o, error, cap));
        E_TRY(mb_weight_build(st, s->ffn_proj_w, F, W * K, MB_F32, &L->proj, error, cap));
        E_TRY(mb_weight_build(st, s->ffn_out_w, W, F * K, MB_F32, &L->out, error, cap));
        if (e->use_tc) {
            E_TRY(e_tc_pack(e, &L->qkv_tc, &L->qkv, s->qkv_w, 3u * W, W, 1u, error, cap));
            E_TRY(e_tc_pack(e, &L->o_tc, &L->o, s->o_w, W, W, 1u, error, cap));
            E_TRY(e_tc_pack(e, &L->proj_tc, &L->proj, s->ffn_proj_w, F, W, K, error, cap));
            E_TRY(e_tc_pack(e, &L->out_tc, &L->out, s->ffn_out_w, W, F, K, error, cap));
        }
    }
    E_TRY(e_upload(&e->embedding, desc->embedding, e->vocab * W, error, cap));
    E_TRY(e_upload(&e->position, desc->position, T * W, error, cap));
    E_TRY(e_upload(&e->norm_out, desc->norm_out, W, error, cap));
    E_TRY(e_malloc((void **)&e->x, T * W * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->nrm, T * W * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->qkv, T * 3u * W * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->ctx, T * W * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->hidden, T * F * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->col, T * F * K * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->out, T * W * sizeof(float), error, cap));
    if (e->use_tc) E_TRY(e_malloc(&e->planes, 2u * T * F * 2u, error, cap));
    if (ok && e->use_tc) E_TRY(mb_cuda((int)cudaStreamSynchronize(st->stream), "cudaStreamSynchronize", error, cap));
    const size_t hw = W / e->heads;
    const size_t n_counters = mb_attention_counters(T, e->heads);
    E_TRY(e_malloc((void **)&e->partials, mb_attention_scratch_floats(T, e->heads, T, hw) * sizeof(float), error, cap));
    E_TRY(e_malloc((void **)&e->counters, n_counters * sizeof(unsigned), error, cap));
    E_TRY(e_malloc((void **)&e->d_ids, T * sizeof(int), error, cap));
    E_TRY(e_malloc((void **)&e->d_lens, T * sizeof(int), error, cap));
    E_TRY(e_malloc((void **)&e->d_count, sizeof(int), error, cap));
    if (ok) E_TRY(mb_cuda((int)cudaMemset(e->counters, 0, n_counters * sizeof(unsigned)), "memset", error, cap));
    E_TRY(mb_cuda((int)cudaMallocHost((void **)&e->h_ids, (2u * T + 1u) * sizeof(int)), "cudaMallocHost", error, cap));
    E_TRY(mb_cuda((int)cudaMallocHost((void **)&e->h_out, T * W * sizeof(float)), "cudaMallocHost", error, cap));
#undef E_TRY
    if (!ok) {
        mynah_b200_encoder_destroy(e);
        return -1;
    }
    *encoder = e;
    mb_clear_error(error, cap);
    return 0;
}

static int f32_product(mb_encoder *e, const mb_dev_weight *w, const float *act, float *out, size_t out_stride,
                       size_t rows, int epilogue) {
    mb_gemv_args g;
    memset(&g, 0, sizeof(g));
    mb_gemv_bind_weight(&g, w, NULL);
    g.x = act;
    g.out = out;
    g.out_stride = out_stride;
    g.batch = rows;
    g.n_active = e->d_count;
    g.epilogue = epilogue;
    g.strict = e->st->strict;
    g.tanh_tab = e->st->libm.tanh_tab;
    e->st->launches += 1u;
    return mb_gemv(&g, e->st->stream);
}

/* out[row][0..n) (=, +=, = gelu) sum over taps and inputs of w[o][i][tap] * act[row - (kernel-1-tap)][i]
 * on the tensor cores: the rows are split into f16 hi/lo planes, then one launch. */
static int tc_product(mb_encoder *e, const enc_tc *w, const float *act, size_t ic, size_t oc, size_t kernel, float *out,
                      size_t out_stride, size_t rows, int epilogue) {
    unsigned short *hi = (unsigned short *)e->planes, *lo = hi + e->max_length * ic;
    int rc = mb_split_rows_f16(act, hi, lo, rows, ic, ic, e->st->stream);
    if (rc != 0) return rc;
    mb_codec_conv_tc_args t;
    memset(&t, 0, sizeof(t));
    t.x_planes = hi; t.x_plane_stride = e->max_length * ic;
    t.w_packed = w->w; t.scale = w->scale;
    t.ic = ic; t.oc = oc; t.length = rows; t.kernel = kernel; t.dilation = 1u;
    t.rows_out = out; t.rows_stride = out_stride; t.rows_epilogue = epilogue;
    t.status = e->st->d_status; t.sm_count = e->st->sm_count;
    e->st->launches += 2u;
    return mb_codec_conv1d_tc(&t, e->st->stream);
}

int mynah_b200_encoder_encode(void *encoder, const int *ids, size_t count, float *out, char *error, size_t cap) {
    mb_encoder *e = (mb_encoder *)encoder;
    if (e == NULL || ids == NULL || out == NULL) {
        mb_set_error(error, cap, "invalid encoder buffers");
        return -1;
    }
    if (count == 0 || count > e->max_length) {
        mb_set_error(error, cap, "text length or embedding shape is invalid");      /* src/graph.c:714-717 */
        return -1;
    }
    for (size_t t = 0; t < count; ++t)
        if (ids[t] < 0 || (size_t)ids[t] >= e->vocab) {
            mb_set_error(error, cap, "text token id is outside vocabulary");        /* src/graph.c:726-731 */
            return -1;
        }
    mb_state *st = e->st;
    MB_TRY(cudaSetDevice(st->device), "cudaSetDevice");
    cudaStream_t s = st->stream;
    const size_t W = e->width, F = e->ffn, K = e->kernel, T = e->max_length;
    for (size_t t = 0; t < count; ++t) {
        e->h_ids[t] = ids[t];
        e->h_ids[T + t] = (int)t;
    }
    e->h_ids[2u * T] = (int)count;
    MB_TRY(cudaMemcpyAsync(e->d_ids, e->h_ids, count * sizeof(int), cudaMemcpyHostToDevice, s), "stage ids");
    MB_TRY(cudaMemcpyAsync(e->d_lens, e->h_ids + T, count * sizeof(int), cudaMemcpyHostToDevice, s), "stage positions");
    MB_TRY(cudaMemcpyAsync(e->d_count, e->h_ids + 2u * T, sizeof(int), cudaMemcpyHostToDevice, s), "stage count");
    int rc = 0;
#define R_TRY(expr) do { if (rc == 0) rc = (int)(expr); } while (0)
    R_TRY(mb_gather_rows(e->embedding, e->d_ids, e->position, e->x, count, W, s));
    st->launches += 1u;
    const float scale = 1.0f / sqrtf((float)(W / e->heads));
    for (size_t l = 0; l < e->layers && rc == 0; ++l) {
        const enc_layer *L = &e->L[l];
        R_TRY(mb_layernorm(e->x, e->nrm, L->norm_self, NULL, count, W, 1.0e-5f, NULL, NULL, e->d_count, st->strict, s));
        st->launches += 1u;
        if (e->use_tc) R_TRY(tc_product(e, &L->qkv_tc, e->nrm, W, 3u * W, 1u, e->qkv, 3u * W, count, MB_EPI_STORE));
        else R_TRY(f32_product(e, &L->qkv, e->nrm, e->qkv, 3u * W, count, MB_EPI_STORE));
        mb_attn_args a;
        memset(&a, 0, sizeof(a));
        a.q = e->qkv;
        a.q_stride = 3u * W;
        a.k_cache = e->qkv + W;          /* K and V live in the qkv rows themselves */
        a.v_cache = e->qkv + 2u * W;
        a.slot_stride = 0;
        a.lens = e->d_lens;              /* row t attends rows 0..t */
        a.valid = count;
        a.cache_rows = count;
        a.cache_stride = 3u * W;
        a.heads = e->heads;
        a.head_width = W / e->heads;
        a.scale = scale;
        a.out = e->ctx;
        a.out_stride = W;
        a.batch = count;
        a.n_active = e->d_count;
        a.strict = st->strict;
        a.exp_tab = st->libm.exp_tab;
        a.partials = e->partials;
        a.counters = e->counters;
        a.status = st->d_status;
        a.sm_count = st->sm_count;
        a.softmax_inverse = 1;
        unsigned launched = 0;
        a.launched = &launched;
        R_TRY(mb_attention(&a, s));
        st->launches += launched;
        if (e->use_tc) {
            /* the causal convolutions need no unfolded copy: a tap is the same rows a few rows up */
            R_TRY(tc_product(e, &L->o_tc, e->ctx, W, W, 1u, e->x, W, count, MB_EPI_RESIDUAL));
            R_TRY(mb_layernorm(e->x, e->nrm, L->norm_ff, NULL, count, W, 1.0e-5f, NULL, NULL, e->d_count, st->strict, s));
            R_TRY(tc_product(e, &L->proj_tc, e->nrm, W, F, K, e->hidden, F, count, MB_EPI_GELU));
            R_TRY(tc_product(e, &L->out_tc, e->hidden, F, W, K, e->x, W, count, MB_EPI_RESIDUAL));
            st->launches += 1u;
        } else {
            R_TRY(f32_product(e, &L->o, e->ctx, e->x, W, count, MB_EPI_RESIDUAL));
            R_TRY(mb_layernorm(e->x, e->nrm, L->norm_ff, NULL, count, W, 1.0e-5f, NULL, NULL, e->d_count, st->strict, s));
            R_TRY(mb_unfold_causal(e->nrm, e->col, count, W, K, s));
            R_TRY(f32_product(e, &L->proj, e->col, e->hidden, F, count, MB_EPI_GELU));
            R_TRY(mb_unfold_causal(e->hidden, e->col, count, F, K, s));
            R_TRY(f32_product(e, &L->out, e->col, e->x, W, count, MB_EPI_RESIDUAL));
            st->launches += 3u;
        }
    }
    R_TRY(mb_layernorm(e->x, e->out, e->norm_out, NULL, count, W, 1.0e-5f, NULL, NULL, e->d_count, st->strict, s));
    st->launches += 1u;
#undef R_TRY
    if (rc != 0) return mb_cuda(rc, "text encoder", error, cap);
    MB_TRY(cudaMemcpyAsync(e->h_out, e->out, count * W * sizeof(float), cudaMemcpyDeviceToHost, s), "read states");
    MB_TRY(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    int status = 0;
    MB_TRY(cudaMemcpy(&status, st->d_status, sizeof(int), cudaMemcpyDeviceToHost), "read status");
    if (status != 0) {
        cudaMemset(st->d_status, 0, sizeof(int));
        mb_set_error(error, cap, mb_status_message(status));
        return -1;
    }
    memcpy(out, e->h_out, count * W * sizeof(float));
    mb_clear_error(error, cap);
    return 0;
}
