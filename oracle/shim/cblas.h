// Oracle build shim (test infrastructure, not product code).
// Maps the standard CBLAS names the reference CPU backend calls
// (src/backend/CPUBackend.cpp:167-303) onto the LP64 exports of the OpenBLAS
// that ships inside scipy's wheel, because this image has no system CBLAS
// headers or MKL.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef int blasint;
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE {
  CblasNoTrans = 111,
  CblasTrans = 112,
  CblasConjTrans = 113
} CBLAS_TRANSPOSE;
void scipy_cblas_sgemm(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, blasint, blasint, blasint,
                       float, const float*, blasint, const float*, blasint, float, float*,
                       blasint);
void scipy_cblas_saxpy(blasint, float, const float*, blasint, float*, blasint);
void scipy_cblas_sscal(blasint, float, float*, blasint);
void scipy_cblas_scopy(blasint, const float*, blasint, float*, blasint);
float scipy_cblas_sdot(blasint, const float*, blasint, const float*, blasint);
void scipy_openblas_set_num_threads(int);
int scipy_openblas_get_num_threads(void);
char* scipy_openblas_get_config(void);
#ifdef __cplusplus
}
#endif
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_saxpy scipy_cblas_saxpy
#define cblas_sscal scipy_cblas_sscal
#define cblas_scopy scipy_cblas_scopy
#define cblas_sdot scipy_cblas_sdot
