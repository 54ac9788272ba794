/* Harness around the reference's quantized weight products.  TEST
 * INFRASTRUCTURE ONLY.
 *
 * Textually includes the reference's src/qmat.c (found through -I on the
 * compile line) to reach its `static` quantizers and dot kernels; the wrappers
 * only forward arguments.  Built into oracle/_ref/ next to the graph harness.
 */
#include "qmat.c"

#define REF_EXPORT __attribute__((visibility("default")))

REF_EXPORT void ref_quantize_weight_int8(const float *w, size_t n, size_t k, int8_t *q,
                                         float *scales) {
    quantize_weight_int8(w, n, k, q, scales);
}

REF_EXPORT void ref_quantize_weight_int4(const float *w, size_t n, size_t k, uint8_t *q,
                                         float *scales) {
    quantize_weight_int4(w, n, k, q, scales);
}

REF_EXPORT float ref_quantize_act_int8(int8_t *qx, const float *x, size_t k) {
    return quantize_act_int8(qx, x, k);
}

REF_EXPORT void ref_matvec_q8(float *out, const int8_t *qx, float sx, const int8_t *weights,
                              const float *scales, const float *bias, size_t rows, size_t cols) {
    matvec_q8(out, qx, sx, weights, scales, bias, rows, cols);
}

REF_EXPORT void ref_matvec_q4(float *out, const int8_t *qx, float sx, const uint8_t *weights,
                              const float *scales, const float *bias, size_t rows, size_t cols) {
    matvec_q4(out, qx, sx, weights, scales, bias, rows, cols);
}

/* y = x W^T + b through a private cache of the given type: the public entry
 * src/qmat.c:768-818 with a CPU backend for the f32 fallback. */
REF_EXPORT int ref_qmat_linear(int qtype, const float *w, const float *x, float *out,
                               size_t count, size_t k, size_t n, const float *bias,
                               char *error, size_t cap) {
    mynah_backend *backend = NULL;
    if (mynah_backend_open(MYNAH_TTS_DEVICE_CPU, &backend, error, cap) != 0) return -1;
    mynah_qmat_cache *cache = mynah_qmat_cache_new(qtype);
    int rc = -1;
    if (cache != NULL)
        rc = mynah_qmat_linear_resolved(cache, backend, "harness.linear", w, x, out, count, k, n,
                                        bias, error, cap);
    mynah_qmat_cache_free(cache);
    mynah_backend_close(backend);
    return rc;
}

/* Batched form, src/qmat.c:820-888; x is [batch][k], out [batch][n]. */
REF_EXPORT int ref_qmat_linear_batched(int qtype, const float *w, const float *x, float *out,
                                       size_t batch, size_t k, size_t n, const float *bias,
                                       char *error, size_t cap) {
    mynah_backend *backend = NULL;
    if (mynah_backend_open(MYNAH_TTS_DEVICE_CPU, &backend, error, cap) != 0) return -1;
    mynah_qmat_cache *cache = mynah_qmat_cache_new(qtype);
    const float **in_rows = (const float **)malloc(batch * sizeof(*in_rows));
    float **out_rows = (float **)malloc(batch * sizeof(*out_rows));
    int8_t *qx = (int8_t *)malloc(batch * k);
    float *sx = (float *)malloc(batch * sizeof(float));
    int rc = -1;
    if (cache != NULL && in_rows && out_rows && qx && sx) {
        for (size_t b = 0; b < batch; ++b) {
            in_rows[b] = x + b * k;
            out_rows[b] = out + b * n;
        }
        rc = mynah_qmat_linear_batched(cache, backend, "harness.batched", w, in_rows, out_rows,
                                       batch, k, n, bias, qx, sx, error, cap);
    }
    free(in_rows); free(out_rows); free(qx); free(sx);
    mynah_qmat_cache_free(cache);
    mynah_backend_close(backend);
    return rc;
}

REF_EXPORT int ref_self_tests(char *error, size_t cap) {
    if (mynah_kernels_self_test(error, cap) != 0) return -1;
    if (mynah_qmat_self_test(error, cap) != 0) return -2;
    if (mynah_backend_self_test(MYNAH_TTS_DEVICE_CPU, error, cap) != 0) return -3;
    return 0;
}
