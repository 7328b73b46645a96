/* TEST INFRASTRUCTURE. The CBLAS declarations the reference's math/gemm.cc needs on its non-MKL path
 * (blaze/blaze/math/gemm.cc:26,43,61,79,313,326). The reference links OpenBLAS (version unpinned,
 * blaze/blaze/CMakeLists.txt:58); here the four entry points are defined in oracle/ref_dense_glue.cc,
 * which forwards to an OpenBLAS found at run time or, when there is none, to a plain k-ascending loop. */
#ifndef ORACLE_REF_SHIM_CBLAS_H_
#define ORACLE_REF_SHIM_CBLAS_H_
#ifdef __cplusplus
extern "C" {
#endif
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, float alpha,
                 const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc);
void cblas_dgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, double alpha,
                 const double* A, int lda, const double* B, int ldb, double beta, double* C, int ldc);
void cblas_sgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int M, int N, float alpha, const float* A, int lda,
                 const float* x, int incx, float beta, float* y, int incy);
void cblas_dgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int M, int N, double alpha, const double* A, int lda,
                 const double* x, int incx, double beta, double* y, int incy);
#ifdef __cplusplus
}
#endif
#endif
