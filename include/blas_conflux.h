/* Linear-algebra and reduction entry points.
 *
 * Same names and signatures as the reference's src/cuda/blas_conflux.h:6-235.
 * The reference forwards these to cuBLAS / cuTENSOR / Thrust (src/cuda/blas/ *.cu);
 * here every one launches a hand-written sm_100a kernel.  All calls are
 * asynchronous on the stream the handle (or StreamWrapper) was created for.
 *
 * Scalar conventions are the reference's: gemm/gemv/ger/scale/clip take
 * alpha/beta as double by value; axpy/reduce/contraction/permutate take
 * pointers to scalars of the element type.  axpy's alpha may be a host OR a
 * device pointer (the dot backward passes device memory,
 * src/ndtensor.zig:1146-1150); the library inspects the pointer.
 *
 * Results of dot / nrm2 / reduce_sum / max_fwd are written to DEVICE memory.
 */
#ifndef ZG_B200_BLAS_CONFLUX_H
#define ZG_B200_BLAS_CONFLUX_H

#include "decls.h"

/* blas_conflux.h:6-13 (blas/dot.cu): result[0] = sum x_i*y_i */
EXTERN_C void dot(dtype id, CublasWrapper w, const void* a_data, const void* b_data, void* result, len_t n);

/* blas_conflux.h:15-26 (blas/gemv.cu): y = alpha*op(A)x + beta*y, A row-major [m,n] */
EXTERN_C void gemv(dtype id, CublasWrapper w, const void* a_data, const void* b_data, void* c_data,
                   len_t m, len_t n, bool trans_a, double alpha, double beta);

/* blas_conflux.h:28-44 (blas/gemm.cu): row-major C = alpha*op(A)op(B) + beta*C,
 * argument meaning as HostDevice.matmul (src/device/host_device.zig:242-250) */
EXTERN_C void gemm(dtype id, CublasWrapper w, const void* a_data, const void* b_data, void* c_data,
                   len_t m, len_t n, len_t k, bool trans_a, bool trans_b,
                   len_t lda, len_t ldb, len_t ldc, double alpha, double beta);

/* blas_conflux.h:46-56 (blas/ger.cu): C[m,n] += alpha * a b^T */
EXTERN_C void ger(dtype id, CublasWrapper w, const void* a_data, const void* b_data, void* c_data,
                  len_t m, len_t n, len_t ldc, double alpha);

/* blas_conflux.h:58-64 (blas/nrm2.cu): y[0] = ||x||_2 */
EXTERN_C void nrm2(dtype id, CublasWrapper w, const void* x, void* y, len_t n);

/* blas_conflux.h:66-74 (blas/clip_nrm2.cu): if ||x|| > max: x *= max/(||x||+delta);
 * cur_nrm2 is a 1-element device scratch that receives the norm */
EXTERN_C void clip_nrm2(dtype id, CublasWrapper w, void* x, void* cur_nrm2, len_t n, double max_nrm2, double delta);

/* blas_conflux.h:76-92 (blas/max.cu) */
EXTERN_C void max_fwd(dtype id, StreamWrapper w, const void* x, void* y, len_t n);
EXTERN_C void max_bwd(dtype id, StreamWrapper w, const void* x_val, void const* y_val, const void* y_grd, void* x_grd, len_t n);

/* blas_conflux.h:94-100 (blas/sum.cu): result[0] = sum |a_i|  (asum, as the
 * host backend's cblas_sasum, src/device/host_device.zig:315-321) */
EXTERN_C void reduce_sum(dtype id, CublasWrapper w, const void* a_data, void* result, len_t n);

/* blas_conflux.h:102-108 (blas/scale.cu): a *= alpha */
EXTERN_C void scale(dtype id, CublasWrapper w, void* a_data, len_t n, double alpha);

/* blas_conflux.h:110-117 (blas/axpy.cu): y += (*alpha) * x */
EXTERN_C void axpy(dtype id, CublasWrapper w, const void* x, void* y, len_t n, const void* alpha);

/* blas_conflux.h:119-161 (blas/{addition,subtraction,multiplication,division}.cu):
 * z[i] = x[i mod x_len] (op) y[i mod y_len], z_len = max(x_len, y_len) */
EXTERN_C void addition(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t x_len, len_t y_len, len_t z_len);
EXTERN_C void subtraction(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t x_len, len_t y_len, len_t z_len);
EXTERN_C void multiplication(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t x_len, len_t y_len, len_t z_len);
EXTERN_C void division(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t x_len, len_t y_len, len_t z_len);

/* blas_conflux.h:164-202: "plans" describe a contraction / reduction /
 * permutation by mode letters, exactly as src/device/cuda_device.zig:284-316
 * and :431-470 build them.  Plans are cached by the library and stay valid
 * until the handle is destroyed; scratch_len is always 0 (no workspace). */
EXTERN_C CutensorPlanWrapper get_contraction_plan(CutensorWrapper w, dtype id,
    const len_t* x_dims, const unsigned char* x_syms, len_t x_dims_len,
    const len_t* y_dims, const unsigned char* y_syms, len_t y_dims_len,
    const len_t* z_dims, const unsigned char* z_syms, len_t z_dims_len);
EXTERN_C CutensorPlanWrapper get_reduce_plan(CutensorWrapper w, dtype id,
    const len_t* src_dims, const unsigned char* src_syms, len_t src_dims_len,
    const len_t* dst_dims, const unsigned char* dst_syms, len_t dst_dims_len, BINARY_OP op);
EXTERN_C CutensorPlanWrapper get_permutate_plan(CutensorWrapper w, dtype id,
    const len_t* src_dims, const unsigned char* src_syms, len_t src_dims_len,
    const len_t* dst_dims, const unsigned char* dst_syms, len_t dst_dims_len);

/* blas_conflux.h:204-213 (blas/reduce.cu): y = alpha*reduce(x) + beta*y */
EXTERN_C void reduce(CutensorWrapper w, void* plan, const void* x_vals, void* y_vals,
                     void* scratch, len_t scratch_len, const void* alpha, const void* beta);
/* blas_conflux.h:215-223 (blas/permutate.cu): y = alpha*perm(x) */
EXTERN_C void permutate(CutensorWrapper w, void* plan, const void* x_vals, void* y_vals,
                        void* scratch, len_t scratch_len, const void* alpha);
/* blas_conflux.h:225-235 (blas/contraction.cu): y = alpha*A.x + gamma*y (batched GEMM) */
EXTERN_C void contraction(CutensorWrapper w, void* plan, const void* A_vals, const void* x_vals, void* y_vals,
                          void* scratch, len_t scratch_len, const void* alpha, const void* gamma);

#endif
