/* Minimal CBLAS declarations for building the unmodified grad.cpp decode path
 * against a wheel-bundled OpenBLAS. TEST INFRASTRUCTURE ONLY (oracle side).
 *
 * grad.cpp references exactly four CBLAS entry points
 * (include/grad/transformer/blas_wrapper.h:81,126,131,136,153). The OpenBLAS
 * copies shipped inside Python wheels export them under a prefix
 * (scipy_cblas_*), selected with -DGRADREF_BLAS_PREFIX_SCIPY. */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };

#ifdef GRADREF_BLAS_PREFIX_SCIPY
#define cblas_sdot scipy_cblas_sdot
#define cblas_saxpy scipy_cblas_saxpy
#define cblas_sscal scipy_cblas_sscal
#define cblas_sgemm scipy_cblas_sgemm
#endif

float cblas_sdot(int n, const float* x, int incx, const float* y, int incy);
void cblas_saxpy(int n, float alpha, const float* x, int incx, float* y, int incy);
void cblas_sscal(int n, float alpha, float* x, int incx);
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int m,
                 int n, int k, float alpha, const float* a, int lda, const float* b, int ldb,
                 float beta, float* c, int ldc);

#ifdef __cplusplus
}
#endif
