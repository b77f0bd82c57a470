// Test-side shim (not product code, not reference code).
//
// The reference's CPU attention path (cpp/chunk_attn/kernel_cpu_mkl.cpp:2) includes Intel
// oneMKL's <mkl_cblas.h>, which is not installed. libtorch_cpu.so exports the Fortran BLAS
// entry point sgemm_ from the oneMKL it embeds, so the three CBLAS calls the reference makes
// (kernel_cpu_mkl.cpp:41,74,105,153,185) are mapped onto it here. Row-major C = op(A)*op(B)
// equals column-major C^T = op(B)^T * op(A)^T, hence the swapped operands.
#pragma once

typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;

extern "C" void sgemm_(const char* transa, const char* transb, const int* m, const int* n,
                       const int* k, const float* alpha, const float* a, const int* lda,
                       const float* b, const int* ldb, const float* beta, float* c,
                       const int* ldc);

static inline void cblas_sgemm(CBLAS_LAYOUT, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N,
                               int K, float alpha, const float* A, int lda, const float* B,
                               int ldb, float beta, float* C, int ldc) {
    const char a = (ta == CblasTrans) ? 'T' : 'N';
    const char b = (tb == CblasTrans) ? 'T' : 'N';
    sgemm_(&b, &a, &N, &M, &K, &alpha, B, &ldb, A, &lda, &beta, C, &ldc);
}

static inline void cblas_saxpby(int n, float a, const float* x, int incx, float b, float* y,
                                int incy) {
    for (int i = 0; i < n; i++) {
        y[i * incy] = a * x[i * incx] + b * y[i * incy];
    }
}
