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
 * forms them (src/graph.c:245-257, 446-450).
 */
#include "host_common.h"
#include "../../include/mynah_b200.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    float *norm_self, *norm_ff;
    mb_dev_weight qkv, o, proj, out;      /* f32: [3W][W], [W][W], [F][W*K], [W][F*K] */
} enc_layer;

typedef struct {
    mb_state *st;
    size_t layers, width, heads, kernel, vocab, max_length, ffn;
    enc_layer *L;
    float *embedding, *position, *norm_out;
    float *x, *nrm, *qkv, *ctx, *hidden, *col, *out, *partials;
    unsigned *counters;
    int *d_ids, *d_lens, *d_count;
    int *h_ids;      /* pinned: ids, then positions */
    float *h_out;    /* pinned */
} mb_encoder;

static int e_malloc(void **p, size_t bytes, char *error, size_t cap) {
    *p = NULL;
    return mb_cuda((int)cudaMalloc(p, bytes ? bytes : 4u), "cudaMalloc(encoder)", error, cap);
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
        }
        free(e->L);
    }
    void *dev[] = {e->embedding, e->position, e->norm_out, e->x, e->nrm, e->qkv, e->ctx, e->hidden, e->col, e->out,
                   e->partials, e->counters, e->d_ids, e->d_lens, e->d_count};
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
        R_TRY(f32_product(e, &L->qkv, e->nrm, e->qkv, 3u * W, count, MB_EPI_STORE));
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
        R_TRY(f32_product(e, &L->o, e->ctx, e->x, W, count, MB_EPI_RESIDUAL));
        R_TRY(mb_layernorm(e->x, e->nrm, L->norm_ff, NULL, count, W, 1.0e-5f, NULL, NULL, e->d_count, st->strict, s));
        R_TRY(mb_unfold_causal(e->nrm, e->col, count, W, K, s));
        R_TRY(f32_product(e, &L->proj, e->col, e->hidden, F, count, MB_EPI_GELU));
        R_TRY(mb_unfold_causal(e->hidden, e->col, count, F, K, s));
        R_TRY(f32_product(e, &L->out, e->col, e->x, W, count, MB_EPI_RESIDUAL));
        st->launches += 3u;
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
