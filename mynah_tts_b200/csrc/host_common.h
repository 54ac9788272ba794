/* Host-side state shared by backend_b200.c (the seam) and decoder_b200.c (the
 * whole-step decoder).  C11; the CUDA runtime's C API only. */
#ifndef MYNAH_B200_HOST_COMMON_H
#define MYNAH_B200_HOST_COMMON_H

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#include "launch.h"

/* A weight resident on the device in one of the four formats. */
typedef struct {
    const float *host;   /* cache key (seam) or NULL (decoder-owned) */
    size_t n, k;
    int qtype;           /* effective format, MB_* */
    void *w;             /* packed weights */
    float *scales;       /* int8 [n], int4 [n*k/32], else NULL */
    size_t bytes;        /* packed bytes + scale bytes */
} mb_dev_weight;

typedef struct {
    const float *host;
    size_t n;
    float *dev;
} mb_dev_vector;

typedef struct mb_state {
    int device, quant, strict;
    cudaStream_t stream;
    int own_stream;
    mb_dev_weight *weights;
    size_t weight_count, weight_cap;
    mb_dev_vector *vectors;
    size_t vector_count, vector_cap;
    /* seam scratch (grown on demand, never during stream capture) */
    float *d_in, *d_out;
    size_t d_in_cap, d_out_cap;      /* floats */
    int8_t *d_qx;
    float *d_sx;
    size_t d_qx_cap, d_sx_cap;
    float *d_partials;
    unsigned *d_counters;
    size_t d_partials_cap, d_counters_cap;
    unsigned *d_token;               /* 1 element */
    int *d_status;
    int sm_count;
    cudaEvent_t timer0, timer1;
    mb_libm_tables libm;             /* strict mode: host-libm correction tables */
    int libm_exact;                  /* 1 when both tables were built */
    unsigned long long launches;
} mb_state;

static inline void mb_set_error(char *error, size_t cap, const char *message) {
    if (error != NULL && cap > 0) snprintf(error, cap, "%s", message);
}
static inline void mb_clear_error(char *error, size_t cap) {
    if (error != NULL && cap > 0) error[0] = '\0';
}
/* Returns 0 when rc is success, else writes "what: <cuda error>" and -1. */
static inline int mb_cuda(int rc, const char *what, char *error, size_t cap) {
    if (rc == (int)cudaSuccess) return 0;
    if (error != NULL && cap > 0)
        snprintf(error, cap, "%s: %s", what, cudaGetErrorString((cudaError_t)rc));
    return -1;
}
#define MB_TRY(expr, what)                                              \
    do {                                                                \
        if (mb_cuda((int)(expr), (what), error, cap) != 0) return -1;   \
    } while (0)

/* What a nonzero device status word says.  Bits: 1 a token id outside the embedding tables
 * (src/graph.c:794-797); 2 a cache tile of an attention kernel never arrived (bounded TMA
 * wait ran out); 8 / 16 a tensor-core product's operand copy / its MMAs never completed
 * (bounded waits ran out).  Several bits: the message of the lowest hardware bit wins, since
 * the outputs of that step are then stale whatever the tokens were. */
static inline const char *mb_status_message(int status) {
    if (status & 2) return "an attention kernel's wait for a cache tile ran out; the step's outputs are stale";
    if (status & 8) return "a tensor-core product's wait for an operand copy ran out; the step's outputs are stale";
    if (status & 16) return "a tensor-core product's wait for its MMAs ran out; the step's outputs are stale";
    if (status & 1) return "audio token id is outside vocabulary";
    return "device status word is set";
}

/* Strict mode: the host-libm sinf correction table of this device, built on first call. */
const uint32_t *mb_libm_sin_table(mb_state *st);

/* Upload a host f32 weight [n,k] and pack it as `qtype` (falls back to f32
 * when int4 cannot represent k).  The caller owns *out (mb_weight_release). */
int mb_weight_build(mb_state *st, const float *host_w, size_t n, size_t k, int qtype,
                    mb_dev_weight *out, char *error, size_t cap);
void mb_weight_release(mb_dev_weight *w);
/* Cached by host pointer for the life of the backend. */
int mb_weight_cached(mb_state *st, const float *host_w, size_t n, size_t k, int qtype,
                     const mb_dev_weight **out, char *error, size_t cap);
int mb_vector_cached(mb_state *st, const float *host_v, size_t n, const float **out, char *error,
                     size_t cap);
/* Fill the weight-side fields of a product descriptor. */
void mb_gemv_bind_weight(mb_gemv_args *g, const mb_dev_weight *w, const float *dev_bias);

#endif
