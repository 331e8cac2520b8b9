/* Activation / softmax / NLL entry points.
 *
 * Same names and signatures as the reference's src/cuda/nn_conflux.h:6-118
 * (implemented there with Thrust and cuDNN in src/cuda/nn/ *.cu).  The
 * CudnnWrapper arguments are stream-bound op contexts (cuda_utils.h).
 */
#ifndef ZG_B200_NN_CONFLUX_H
#define ZG_B200_NN_CONFLUX_H

#include "decls.h"

/* nn_conflux.h:6-21 (nn/relu.cu): y = max(x,0) ; x_grd += (x>0) ? y_grd : 0 */
EXTERN_C void relu_fwd(dtype id, StreamWrapper w, const void* x, void* y, len_t n);
EXTERN_C void relu_bwd(dtype id, StreamWrapper w, const void* x, const void* y_grd, void* x_grd, len_t n);

/* nn_conflux.h:23-39 (nn/smax_vec.cu): softmax / log-softmax of one vector;
 * bwd accumulates: x_grd += y*(y_grd - sum(y*y_grd)) */
EXTERN_C void smax_vec_fwd(dtype id, CudnnWrapper w, const void* x, void* y, len_t n, smaxtype smaxop);
EXTERN_C void smax_vec_bwd(dtype id, CudnnWrapper w, const void* y_val, const void* y_grd, void* x_grd, len_t n);

/* nn_conflux.h:41-59 (nn/smax_2D_row.cu): row softmax of [m,n] */
EXTERN_C void smax_2D_row_fwd(dtype id, CudnnWrapper w, const void* x, void* y, len_t m, len_t n);
EXTERN_C void smax_2D_row_bwd(dtype id, CudnnWrapper w, const void* y_val, const void* y_grd, void* x_grd, len_t m, len_t n);

/* nn_conflux.h:61-69 (nn/clamp.cu): y = min(max(lower,x),upper) */
EXTERN_C void clamp(dtype id, StreamWrapper w, const void* x, void* y, len_t n, double lower, double upper);

/* nn_conflux.h:71-91 (nn/nll_loss_1d_index.cu): dst[0] = -log_softmax(src)[trg]
 * (src is log-probabilities already when inplace_smax is false);
 * bwd: x_grd = softmax(x) - onehot(trg) */
EXTERN_C void nll_loss_1D_index_fwd(dtype id, CudnnWrapper w, void* src, len_t trg, void* dst, len_t n, bool inplace_smax, reduxtype reduxop);
EXTERN_C void nll_loss_1D_index_bwd(dtype id, CudnnWrapper w, const void* x_val, void* x_grd, len_t trg, len_t n, reduxtype reduxop);

/* nn_conflux.h:93-111 (nn/nll_loss_1d_encode.cu): same with a one-hot/probability target vector */
EXTERN_C void nll_loss_1D_encode_fwd(dtype id, CudnnWrapper w, void* src, const void* trg, void* dst, len_t n, bool inplace_smax, reduxtype reduxop);
EXTERN_C void nll_loss_1D_encode_bwd(dtype id, CudnnWrapper w, const void* x_val, const void* y_val, void* x_grd, len_t n, reduxtype reduxop);

/* nn_conflux.h:113-118 (nn/exp.cu): y = exp(x) */
EXTERN_C void pow_exp(dtype id, StreamWrapper w, const void* x, void* y, len_t n);

#endif
