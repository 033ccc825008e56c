// cuSPARSE SpMM called the way the reference calls it, for head-to-head checks and timing.
//
// NOT part of the product: libdrone_b200.so never links or loads this file.  It exists so
// that tests and the benchmark can compare against the library routine the reference's
// GraphSum layers delegate to (cuda_gcn/src/cuda/cuda_module.cu:166-169 cusparseCreateCsr,
// :191-194 cusparseCreateDnMat row-major ld=dim, :233-246 cusparseSpMM with alpha=1, beta=0,
// op N/N, CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT and a work buffer from cusparseSpMM_bufferSize).
#include <cuda_runtime.h>
#include <cusparse.h>
#include <cstdio>

struct RefSpmm {
    cusparseHandle_t handle = nullptr;
    cusparseSpMatDescr_t mat = nullptr;
    cusparseDnMatDescr_t x = nullptr, y = nullptr;
    void *buffer = nullptr;
    size_t buffer_bytes = 0;
    cusparseSpMMAlg_t alg = CUSPARSE_SPMM_ALG_DEFAULT;
};

#define REF_CHECK(call)                                                                      \
    do {                                                                                     \
        cusparseStatus_t s__ = (call);                                                       \
        if (s__ != CUSPARSE_STATUS_SUCCESS) {                                                \
            fprintf(stderr, "cusparse_spmm: %s failed: %s\n", #call, cusparseGetErrorString(s__)); \
            return -1;                                                                       \
        }                                                                                    \
    } while (0)

extern "C" {

// alg: 0 = CUSPARSE_SPMM_ALG_DEFAULT (what the reference uses), 2 = CSR_ALG2, 3 = CSR_ALG3
int ref_cusparse_spmm_create(RefSpmm **out, int n_rows, int n_cols, int nnz, int *d_rowptr, int *d_col,
                             float *d_val, int F, float *d_X, float *d_Y, int alg, void *stream) {
    RefSpmm *r = new RefSpmm();
    r->alg = alg == 2 ? CUSPARSE_SPMM_CSR_ALG2 : alg == 3 ? CUSPARSE_SPMM_CSR_ALG3 : CUSPARSE_SPMM_ALG_DEFAULT;
    REF_CHECK(cusparseCreate(&r->handle));
    REF_CHECK(cusparseSetStream(r->handle, (cudaStream_t)stream));
    REF_CHECK(cusparseCreateCsr(&r->mat, n_rows, n_cols, nnz, d_rowptr, d_col, d_val, CUSPARSE_INDEX_32I,
                                CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    REF_CHECK(cusparseCreateDnMat(&r->x, n_cols, F, F, d_X, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    REF_CHECK(cusparseCreateDnMat(&r->y, n_rows, F, F, d_Y, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    const float alpha = 1.0f, beta = 0.0f;
    REF_CHECK(cusparseSpMM_bufferSize(r->handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                      &alpha, r->mat, r->x, &beta, r->y, CUDA_R_32F, r->alg, &r->buffer_bytes));
    if (cudaMalloc(&r->buffer, r->buffer_bytes > 0 ? r->buffer_bytes : 16) != cudaSuccess) return -2;
    if (r->alg != CUSPARSE_SPMM_ALG_DEFAULT)
        REF_CHECK(cusparseSpMM_preprocess(r->handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                          &alpha, r->mat, r->x, &beta, r->y, CUDA_R_32F, r->alg, r->buffer));
    *out = r;
    return 0;
}

int ref_cusparse_spmm_run(RefSpmm *r) {
    const float alpha = 1.0f, beta = 0.0f;
    REF_CHECK(cusparseSpMM(r->handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha,
                           r->mat, r->x, &beta, r->y, CUDA_R_32F, r->alg, r->buffer));
    return 0;
}

long long ref_cusparse_spmm_buffer_bytes(RefSpmm *r) { return (long long)r->buffer_bytes; }

int ref_cusparse_spmm_destroy(RefSpmm *r) {
    if (!r) return 0;
    cusparseDestroySpMat(r->mat);
    cusparseDestroyDnMat(r->x);
    cusparseDestroyDnMat(r->y);
    cusparseDestroy(r->handle);
    cudaFree(r->buffer);
    delete r;
    return 0;
}

}  // extern "C"
