/* Device, stream, memory, graph-capture and virtual-memory entry points.
 *
 * Same names and signatures as the reference's src/cuda/cuda_utils.h:7-55
 * (implemented there in src/cuda/cuda_utils.cu); what differs is behaviour
 * on error: nothing here calls exit() -- a failure is recorded in a sticky
 * status that zg_last_error() (zg_b200.h) returns, and allocation entry
 * points return NULL so the Zig side maps them to error.DeviceOOM
 * (src/device/cuda_device.zig:486-492).
 */
#ifndef ZG_B200_CUDA_UTILS_H
#define ZG_B200_CUDA_UTILS_H

#include "decls.h"

/* ---- memory (cuda_utils.h:7-16; cuda_utils.cu:9-48,152-302) ---- */
EXTERN_C void* mem_alloc(len_t nbytes, StreamWrapper stream);              /* stream-ordered; NULL on OOM */
EXTERN_C void mem_free(void* dptr, StreamWrapper stream);
EXTERN_C void memcpy_HtoD(void* dptr, void const* hptr, len_t nbytes, StreamWrapper stream);
EXTERN_C void memcpy_DtoH(void* hptr, void const* dptr, len_t nbytes, StreamWrapper stream);
EXTERN_C void memcpy_DtoD(void* dst, void const* src, len_t nbytes, StreamWrapper stream);
EXTERN_C void mem_fill(dtype id, void* data, len_t n, const void* value, StreamWrapper stream);
EXTERN_C void mem_sequence(dtype id, void* data, len_t n, const void* init, const void* step, StreamWrapper stream);
EXTERN_C void mem_random(dtype id, void* x, len_t n, randtype op, unsigned seed, StreamWrapper stream);
EXTERN_C void mem_take(dtype id, const void* src, len_t src_len, const len_t* idxs, len_t idxs_len, void* dst, StreamWrapper stream);
EXTERN_C len_t mem_page_size(unsigned device_id);

/* ---- device (cuda_utils.h:19-24; cuda_utils.cu:50-98) ---- */
EXTERN_C DevicePropertiesWrapper init_device(unsigned device_number);      /* binds the primary context */
EXTERN_C void check_last_error(void);
EXTERN_C void device_synchronize(void);
EXTERN_C len_t device_total_memory(unsigned device_number);
EXTERN_C unsigned device_count(void);

/* ---- streams (cuda_utils.h:26-29) ---- */
EXTERN_C StreamWrapper init_stream(void);
EXTERN_C void deinit_stream(StreamWrapper stream);
EXTERN_C void stream_synchronize(StreamWrapper stream);

/* ---- op contexts (cuda_utils.h:31-41).  The reference creates cuBLAS, cuDNN
 * and cuTENSOR handles here; this library has no such dependency, so each
 * "handle" is a small context that remembers the stream it was made for. ---- */
EXTERN_C CublasWrapper init_cublas_handle(StreamWrapper stream);
EXTERN_C void deinit_cublas_handle(CublasWrapper handle);
EXTERN_C CudnnWrapper init_cudnn_handle(StreamWrapper stream);
EXTERN_C void deinit_cudnn_handle(CudnnWrapper handle);
EXTERN_C CutensorWrapper init_cutensor_handle(StreamWrapper stream);
EXTERN_C void deinit_cutensor_handle(CutensorWrapper handle);

/* ---- CUDA-graph capture of the device stream (cuda_utils.h:43-47;
 * cuda_utils.cu:214-243) ---- */
EXTERN_C GraphWrapper open_capture(StreamWrapper stream);
EXTERN_C void save_capture(GraphWrapper graph, StreamWrapper stream);
EXTERN_C void free_capture(GraphWrapper graph, StreamWrapper stream);
EXTERN_C void run_capture(GraphWrapper graph, StreamWrapper stream);

/* ---- virtual-memory arena used by the Zig CachingAllocator's DataHandler
 * (cuda_utils.h:49-55; cuda_utils.cu:305-430; src/device/cuda_device.zig:21-81) ---- */
EXTERN_C void* mem_map(unsigned device_id, size_t virtual_buffer_size);
EXTERN_C void mem_unmap(unsigned device_id, void* base_address, size_t virtual_buffer_size);
EXTERN_C MemmapWrapper init_memmap(unsigned device_id);
EXTERN_C void reset_memmap(MemmapWrapper map);
EXTERN_C void deinit_memmap(MemmapWrapper map);
EXTERN_C void mem_map_alloc(MemmapWrapper map, void* address, len_t size);

#endif
