/* Minimal declarations of the CBLAS entry points the reference's CPU path calls
 * (cblas_sgemm at models/layers/convolutional_layer.cc:389 and
 * models/layers/connected_layer.cc:261; cblas_saxpy / cblas_sscal in the
 * recurrent and update code).  The image ships OpenBLAS 0.3.15 inside the
 * opencv wheel but no development header; this shim stands in for <cblas.h>
 * when the reference sources are compiled as the parity checker.
 * Test infrastructure only: nothing in the product links against it. */
#ifndef NB_ORACLE_CBLAS_SHIM_H
#define NB_ORACLE_CBLAS_SHIM_H
#ifdef __cplusplus
extern "C" {
#endif

typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE {
    CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113, CblasConjNoTrans = 114
} CBLAS_TRANSPOSE;

void cblas_sgemm(const enum CBLAS_ORDER order, const enum CBLAS_TRANSPOSE ta,
                 const enum CBLAS_TRANSPOSE tb, const int m, const int n, const int k,
                 const float alpha, const float *a, const int lda, const float *b,
                 const int ldb, const float beta, float *c, const int ldc);
void cblas_saxpy(const int n, const float alpha, const float *x, const int incx,
                 float *y, const int incy);
void cblas_sscal(const int n, const float alpha, float *x, const int incx);
void openblas_set_num_threads(int num_threads);

#ifdef __cplusplus
}
#endif
#endif
