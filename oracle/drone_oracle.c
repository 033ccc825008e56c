/*
 * drone_oracle.c — CPU restatement of DRONE's sparse-aggregation path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the
 * tests, the smoke check and the CPU-baseline leg of the benchmark load it; no
 * product code path may call it.
 *
 * Parity status: the reference ships no golden vectors for GCN outputs,
 * gradients, exchange results or PageRank values ("parity unpinned" by the
 * reference's own tests).  What it does hold, and what this oracle is pinned
 * against in tests/test_oracle.py, is the cuSPARSE SpMM known-answer case of
 * cuda_gcn/src/tools/sparse.cu:28-49 (4x4, 9 nonzeros, times a 4x3 dense) and
 * the transpose print-out case of cuda_gcn/src/tools/test.cu:47-70.  Where a
 * GPU is present the tests also run the reference's own compiled code beside it
 * (oracle/_ref, built from the reference sources by oracle/Makefile): local
 * numbering and coefficients of build_graph, CUDAGraphSum::forward / backward
 * on one and two workers, the first-epoch loss of CUDAGCN::train_epoch, and
 * the pr / cc / sssp jobs (tests/test_reference_gpu.py,
 * tests/test_reference_jobs_gpu.py).
 *
 * The sparse x dense product itself lives in a third-party dependency that is
 * not in the reference tree: cuSPARSE (cusparseSpMM, CSR, fp32, row-major,
 * CUSPARSE_SPMM_ALG_DEFAULT; the toolkit here ships libcusparse 12.5.10).  Its
 * published contract is C = alpha*op(A)*op(B) + beta*C; the functions below
 * restate that contract in double precision at the reference's call sites.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------- */
/* A1: local graph build.  cuda_gcn/src/cuda/graph.cu:54-103                  */
/* Local ids are handed out in first-seen order over the edge list (u before  */
/* v for each edge, :67-70); CSR is by SOURCE vertex, destinations kept in    */
/* edge-list order inside a row (:94-103).                                    */
/* g2l must hold globalV ints, l2g globalV ints, index globalV+1, dst E.      */
/* Returns the number of local vertices.                                      */
/* ------------------------------------------------------------------------- */
int oracle_build_graph(int globalV, int E, const int *u, const int *v, int *g2l, int *l2g, int *index,
                       int *dst) {
    int n = 0;
    for (int i = 0; i < globalV; ++i) g2l[i] = -1;
    for (int i = 0; i < E; ++i) {
        if (g2l[u[i]] < 0) { g2l[u[i]] = n; l2g[n] = u[i]; ++n; }
        if (g2l[v[i]] < 0) { g2l[v[i]] = n; l2g[n] = v[i]; ++n; }
    }
    int *fill = (int *)calloc((size_t)n + 1, sizeof(int));
    for (int i = 0; i <= n; ++i) index[i] = 0;
    for (int i = 0; i < E; ++i) index[g2l[u[i]] + 1]++;
    for (int i = 0; i < n; ++i) index[i + 1] += index[i];
    for (int i = 0; i < E; ++i) {
        const int lu = g2l[u[i]];
        dst[index[lu] + fill[lu]++] = g2l[v[i]];
    }
    free(fill);
    return n;
}

/* ------------------------------------------------------------------------- */
/* A2: edge coefficients.  cuda_gcn/src/cuda/cuda_kernel.cu:144-155           */
/*   values[i] = 1.0 / sqrtf(1.0 * outDegree[u] * in_degree[v])               */
/* The product is a double, sqrtf takes it narrowed to float, the division is */
/* in double and the store narrows to float.                                  */
/* ------------------------------------------------------------------------- */
void oracle_csr_values_f32(const int *index, const int *dst, const int *in_degree, const int *out_degree,
                           int n, float *values) {
    for (int u = 0; u < n; ++u)
        for (int i = index[u]; i < index[u + 1]; ++i) {
            const int v = dst[i];
            values[i] = (float)(1.0 / sqrtf((float)(1.0 * out_degree[u] * in_degree[v])));
        }
}

/* Same coefficient without any float rounding (for error budgeting). */
void oracle_csr_values_f64(const int *index, const int *dst, const int *in_degree, const int *out_degree,
                           int n, double *values) {
    for (int u = 0; u < n; ++u)
        for (int i = index[u]; i < index[u + 1]; ++i)
            values[i] = 1.0 / sqrt((double)out_degree[u] * (double)in_degree[dst[i]]);
}

/* ------------------------------------------------------------------------- */
/* A4/A6 forward: out[v,:] += coef(u,v) * in[u,:] for every edge u->v.         */
/* cuda_gcn/src/cuda/cuda_kernel.cu:203-218 (hand-written form) and the       */
/* cuSPARSE call it was replaced by, cuda_gcn/src/cuda/cuda_module.cu:233-246  */
/* (matAT x in).  Coefficients are the float values of A2; accumulation is in  */
/* double.  out is overwritten.                                               */
/* ------------------------------------------------------------------------- */
void oracle_graphsum_forward_f64(const float *in, double *out, const int *index, const int *dst,
                                 const float *values, int dim, int n) {
    memset(out, 0, sizeof(double) * (size_t)n * (size_t)dim);
    for (int u = 0; u < n; ++u)
        for (int i = index[u]; i < index[u + 1]; ++i) {
            const int v = dst[i];
            const double c = values[i];
            for (int j = 0; j < dim; ++j) out[(size_t)v * dim + j] += c * (double)in[(size_t)u * dim + j];
        }
}

/* A5/A6 backward: in_grad[u,:] += coef(u,v) * out_grad[v,:].                  */
/* cuda_gcn/src/cuda/cuda_kernel.cu:236-248; cuSPARSE call at                  */
/* cuda_gcn/src/cuda/cuda_module.cu:323-336 (matA x out.grad).                 */
void oracle_graphsum_backward_f64(double *in_grad, const float *out_grad, const int *index, const int *dst,
                                  const float *values, int dim, int n) {
    memset(in_grad, 0, sizeof(double) * (size_t)n * (size_t)dim);
    for (int u = 0; u < n; ++u)
        for (int i = index[u]; i < index[u + 1]; ++i) {
            const int v = dst[i];
            const double c = values[i];
            for (int j = 0; j < dim; ++j)
                in_grad[(size_t)u * dim + j] += c * (double)out_grad[(size_t)v * dim + j];
        }
}

/* ------------------------------------------------------------------------- */
/* cusparseSpMM contract at the reference's call sites (alpha=1, beta=0, CSR,  */
/* row-major dense, cuda_gcn/src/cuda/cuda_module.cu:191-194,233-246):         */
/*   Y[r,:] = sum_k val[k] * X[col[k],:], double accumulation.                 */
/* abs_out, when not NULL, receives sum_k |val[k]*X[col[k],:]|, the scale      */
/* against which a float summation error is judged.                            */
/* ------------------------------------------------------------------------- */
void oracle_spmm_csr_f64(int n_rows, const int *rowptr, const int *col, const float *val, const float *X,
                         int ldx, double *Y, double *abs_out, int ldy, int F) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int r = 0; r < n_rows; ++r) {
        double *y = Y + (size_t)r * ldy;
        double *a = abs_out ? abs_out + (size_t)r * ldy : NULL;
        for (int j = 0; j < F; ++j) y[j] = 0.0;
        if (a) for (int j = 0; j < F; ++j) a[j] = 0.0;
        for (int k = rowptr[r]; k < rowptr[r + 1]; ++k) {
            const double c = val[k];
            const float *x = X + (size_t)col[k] * ldx;
            for (int j = 0; j < F; ++j) {
                const double t = c * (double)x[j];
                y[j] += t;
                if (a) a[j] += fabs(t);
            }
        }
    }
}

/* The same product in float, row-parallel over `threads` host threads: the     */
/* timed CPU baseline ("port" of the path to the host cores).                   */
void oracle_spmm_csr_f32(int n_rows, const int *rowptr, const int *col, const float *val, const float *X,
                         int ldx, float *Y, int ldy, int F, int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(dynamic, 512)
    for (int r = 0; r < n_rows; ++r) {
        float *y = Y + (size_t)r * ldy;
        for (int j = 0; j < F; ++j) y[j] = 0.f;
        for (int k = rowptr[r]; k < rowptr[r + 1]; ++k) {
            const float c = val[k];
            const float *x = X + (size_t)col[k] * ldx;
            for (int j = 0; j < F; ++j) y[j] += c * x[j];
        }
    }
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* A3: explicit transpose with values, as cusparseCsr2cscEx2 produces it       */
/* (cuda_gcn/src/cuda/cuda_module.cu:171-185): column pointers, row indices    */
/* ascending inside a column, values carried along.                            */
/* ------------------------------------------------------------------------- */
void oracle_transpose_csr(int n_rows, int n_cols, const int *rowptr, const int *col, const float *val,
                          int *t_rowptr, int *t_col, float *t_val) {
    for (int i = 0; i <= n_cols; ++i) t_rowptr[i] = 0;
    const int nnz = rowptr[n_rows];
    for (int k = 0; k < nnz; ++k) t_rowptr[col[k] + 1]++;
    for (int i = 0; i < n_cols; ++i) t_rowptr[i + 1] += t_rowptr[i];
    int *fill = (int *)calloc((size_t)n_cols + 1, sizeof(int));
    for (int r = 0; r < n_rows; ++r)
        for (int k = rowptr[r]; k < rowptr[r + 1]; ++k) {
            const int c = col[k];
            const int pos = t_rowptr[c] + fill[c]++;
            t_col[pos] = r;
            t_val[pos] = val[k];
        }
    free(fill);
}
