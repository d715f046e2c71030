/* C interface of the circuit simulator's device kernels (libnangila_kernels.so): an FP64 CSR
 * matrix kept resident on the GPU, y = A x on it, and a Jacobi-preconditioned BiCGSTAB solve.
 * Every function returns 0 on success or a cudaError_t value; nangila_spmv_bicgstab returns -1 when
 * it stopped without reaching the tolerance. */
#pragma once
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct NangilaSpmv NangilaSpmv;

NangilaSpmv* nangila_spmv_create(void);
void nangila_spmv_destroy(NangilaSpmv* ctx);

/* Copies an n x n CSR matrix (host arrays, 0-based, row_ptr[n] == nnz) to the current device and
 * builds its row-block table. Replaces any matrix loaded before. */
int nangila_spmv_load(NangilaSpmv* ctx, int n, int nnz, const int* row_ptr, const int* col, const double* val);
/* New values for the loaded pattern (a Newton iteration or a PVT corner changes values, not structure). */
int nangila_spmv_update_values(NangilaSpmv* ctx, const double* val);
/* y = A x with host vectors (copied in and out; the call the reference's bridge offers). */
int nangila_spmv_host(NangilaSpmv* ctx, const double* h_x, double* h_y);
/* y = A x with device vectors, queued on `stream`; no copies, no synchronisation. */
int nangila_spmv_device(NangilaSpmv* ctx, const double* d_x, double* d_y, cudaStream_t stream);
/* 0, or cudaErrorTimeout when a kernel of this context gave up waiting for one of its own bulk copies
 * (reads one word back from the device, so it synchronises). */
int nangila_spmv_status(NangilaSpmv* ctx);
int nangila_spmv_dims(const NangilaSpmv* ctx, int* n, int* nnz, int* n_blocks);

/* Row-block table for a CSR pattern: out[0] = 0, out[b + 1] = first row after block b. Returns the
 * number of blocks; with out == NULL only counts. Host function. */
int nangila_spmv_build_row_blocks(const int* row_ptr, int n, int* out, int max_out);
/* The kernel alone, on device arrays the caller owns (e.g. torch tensors). */
int nangila_spmv_launch(const int* d_row_ptr, const int* d_col, const double* d_val, const double* d_x, double* d_y,
                        const int* d_row_blocks, int n_blocks, cudaStream_t stream);

/* Solves A x = b from x = 0. h_b, h_x: host vectors of length n. */
int nangila_spmv_bicgstab(NangilaSpmv* ctx, const double* h_b, double* h_x, double tol, int max_iter, int* iterations,
                          double* rel_residual);

#ifdef __cplusplus
}
#endif
