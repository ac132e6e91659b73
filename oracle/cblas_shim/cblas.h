/* Test infrastructure, not product code.
 *
 * Minimal <cblas.h> for building the reference with HAVE_CBLAS against the OpenBLAS that the
 * scipy wheel ships (libscipy_openblas, LP64, symbols prefixed scipy_).  The reference calls
 * cblas_sgemm only (src/ops_matrix.c, src/attention.c, src/conv.c, src/transformer.c); the enum
 * values are the ones the CBLAS standard fixes. */
#ifndef DNN_ORACLE_CBLAS_SHIM_H
#define DNN_ORACLE_CBLAS_SHIM_H
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void scipy_cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int m, int n, int k,
                       float alpha, const float *a, int lda, const float *b, int ldb, float beta, float *c, int ldc);
#define cblas_sgemm scipy_cblas_sgemm
#endif
