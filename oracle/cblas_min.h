/*
 * cblas_min.h -- the handful of standard CBLAS declarations the reference's
 * OpenBLAS code path needs (its Private.h does `#include <cblas.h>`; this
 * image has an OpenBLAS shared object but no header).  Test infrastructure
 * for building the reference from its own sources; not part of the product.
 * Installed as `cblas.h` in the private include directory of that build.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                 float alpha, const float *a, int lda, const float *b, int ldb,
                 float beta, float *c, int ldc);
void cblas_sgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int m, int n, float alpha, const float *a, int lda,
                 const float *x, int incx, float beta, float *y, int incy);
void cblas_sger(CBLAS_ORDER order, int m, int n, float alpha, const float *x, int incx,
                const float *y, int incy, float *a, int lda);
void cblas_saxpy(int n, float alpha, const float *x, int incx, float *y, int incy);
void cblas_sscal(int n, float alpha, float *x, int incx);
void openblas_set_num_threads(int n);
int openblas_get_num_threads(void);
#ifdef __cplusplus
}
#endif
