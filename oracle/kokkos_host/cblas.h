/* The two entries of the standard CBLAS interface that the reference's host GEMM
 * path calls (include/pet/gemm.hpp, PET_HAVE_CBLAS), declared here because this
 * image carries an optimised BLAS (the OpenBLAS inside the scipy wheel) but no
 * header for it. ref_driver.cpp defines them and forwards to that library.
 * TEST INFRASTRUCTURE ONLY. */
#ifndef PET_ORACLE_CBLAS_H
#define PET_ORACLE_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef CBLAS_LAYOUT CBLAS_ORDER;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                 const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc);
void cblas_dgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, double alpha,
                 const double* A, int lda, const double* B, int ldb, double beta, double* C, int ldc);
#ifdef __cplusplus
}
#endif
#endif
