/* Shared C types of the zigrad CUDA device ABI (libamalgamate.so).
 *
 * Name- and layout-compatible with the reference's src/cuda/decls.h:1-47, so
 * that `@cImport` in src/cuda/root.zig:1-5 binds unchanged.  Additions over
 * the reference are marked NEW.
 */
#ifndef ZG_B200_DECLS_H
#define ZG_B200_DECLS_H

#ifdef __cplusplus
#define EXTERN_C extern "C"
#else
#define EXTERN_C extern
#endif

#include <stdbool.h>
#include <stddef.h>
#include <stdlib.h>

typedef unsigned long len_t;   /* Zig usize */

/* element type tag passed as the first argument of most entry points */
typedef unsigned char dtype;
static const dtype SINGLE = 0;  /* f32 */
static const dtype DOUBLE = 1;  /* f64 */
static const dtype BF16 = 2;    /* NEW: bfloat16 storage (GEMM operands/outputs, Adam weight copy) */

static const len_t CUDA_PAGE_SIZE = 4096;

/* opaque by-value handles (one pointer each) */
typedef struct { void* ptr; } StreamWrapper;
typedef struct { void* ptr; } CublasWrapper;    /* here: a stream-bound op context, no cuBLAS behind it */
typedef struct { void* ptr; } CutensorWrapper;  /* here: a stream-bound op context, no cuTENSOR behind it */
typedef struct { void* ptr; } CudnnWrapper;     /* here: a stream-bound op context, no cuDNN behind it */
typedef struct { void* ptr; } GraphWrapper;
typedef struct { void* ptr; } DevicePropertiesWrapper;
typedef struct { void* ptr; } MemmapWrapper;

typedef struct { void* plan; len_t scratch_len; } CutensorPlanWrapper;

typedef unsigned char reduxtype;
static const reduxtype RDX_NONE = 0;
static const reduxtype RDX_MEAN = 1;
static const reduxtype RDX_SUM = 2;

typedef unsigned char smaxtype;
static const smaxtype SMAX_FAST = 0;
static const smaxtype SMAX_MAX = 1;
static const smaxtype SMAX_LOG = 2;

typedef unsigned char randtype;
static const randtype UNIFORM = 0;
static const randtype NORMAL = 1;

typedef enum { ADD, MIN, MAX, MUL } BINARY_OP;

#endif
