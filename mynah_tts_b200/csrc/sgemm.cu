// Plain f32 row-major sgemm for the backend-seam entries that are not on the
// per-token path (context prefill, codec): C = alpha*op(A)*op(B) + beta*C with
// cblas-style transposes (src/backend.h:14-25 in mynah-tts).  Each thread owns
// one element of C and accumulates over k in index order with separately
// rounded products, which is the reference's scalar fallback order
// (src/backend.c:353-366); 16x16 tiles of A and B are staged in shared memory.
#include "common.cuh"
#include "launch.h"

namespace {

constexpr int TILE = 16;

__global__ void __launch_bounds__(TILE * TILE)
k_sgemm(int trans_a, int trans_b, long m, long n, long k, float alpha, const float *__restrict__ a,
        long lda, const float *__restrict__ b, long ldb, float beta, float *__restrict__ c, long ldc) {
    mb_pdl_wait();
    mb_pdl_trigger();
    __shared__ float as[TILE][TILE + 1];
    __shared__ float bs[TILE][TILE + 1];
    const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    const long row = (long)blockIdx.y * TILE + ty;
    const long col = (long)blockIdx.x * TILE + tx;
    float sum = 0.0f;
    for (long p0 = 0; p0 < k; p0 += TILE) {
        const long pa = p0 + tx, pb = p0 + ty;
        as[ty][tx] = (row < m && pa < k) ? (trans_a ? a[pa * lda + row] : a[row * lda + pa]) : 0.0f;
        bs[ty][tx] = (col < n && pb < k) ? (trans_b ? b[col * ldb + pb] : b[pb * ldb + col]) : 0.0f;
        __syncthreads();
        const int lim = (int)min((long)TILE, k - p0);
        for (int p = 0; p < lim; ++p) sum = __fadd_rn(sum, __fmul_rn(as[ty][p], bs[p][tx]));
        __syncthreads();
    }
    if (row < m && col < n) {
        float *dst = c + row * ldc + col;
        // beta == 0 must not read C (it may be uninitialized), as in BLAS.
        *dst = beta == 0.0f ? __fmul_rn(alpha, sum)
                            : __fadd_rn(__fmul_rn(alpha, sum), __fmul_rn(beta, *dst));
    }
}

}  // namespace

extern "C" int mb_sgemm(int trans_a, int trans_b, size_t m, size_t n, size_t k, float alpha,
                        const float *a, size_t lda, const float *b, size_t ldb, float beta, float *c,
                        size_t ldc, mb_stream stream) {
    if (m == 0 || n == 0 || k == 0) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)((n + TILE - 1) / TILE), (unsigned)((m + TILE - 1) / TILE));
    mb_launch(k_sgemm, dim3(grid), dim3(TILE * TILE), 0, (cudaStream_t)stream, trans_a, trans_b, (long)m, (long)n,
                                                           (long)k, alpha, a, (long)lda, b,
                                                           (long)ldb, beta, c, (long)ldc);
    return mb_check_launch();
}
