/*
 * Source-compatible stand-ins for the per-kernel C headers the reference emits when it exports
 * a CuTe-DSL kernel (module struct, tensor descriptors, `cute_dsl_<prefix>_wrapper`).  A consumer
 * written against those headers -- cute/main.cpp, cute/main_rotary.cpp -- compiles unchanged
 * against the headers under artifacts/ and links libgigaslop_b200 instead of the exported object.
 *
 * What the consumers rely on (and what is reproduced here):
 *   - CUTE_DSL_CUDA_ERROR_CHECK(err): prints, never aborts                      (cute/main.cpp:83)
 *   - <P>_Kernel_Module_t with a `module` member, <P>_Kernel_Module_Load / _Unload; Load prepares
 *     every visible device                                                      (cute/main.cpp:95-96,173)
 *   - `_mlir_<P>_cuda_init` / `_mlir_<P>_cuda_load_to_device` with C linkage     (cute/main.cpp:14-15)
 *   - <P>_Tensor_mA_t / mB / mC: { void* data; int32 dynamic_shapes[3]; int64 dynamic_strides[2]; }
 *     = (rows, inner extent, batch) and (row stride, batch stride) in elements  (cute/main.cpp:98-120)
 *   - pointer-only descriptors for scales and sin/cos tables                    (cute/main_rotary.cpp:153-156)
 *   - wrapper returns int32 (0 = ok), takes the module first, launches on the legacy default stream
 * Buffers stay owned by the caller; nothing is allocated.
 */
#ifndef GIGASLOP_B200_CUTE_DSL_ABI_H_
#define GIGASLOP_B200_CUTE_DSL_ABI_H_

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "gigaslop_b200.h"

#ifndef CUTE_DSL_CUDA_ERROR_CHECK
#define CUTE_DSL_CUDA_ERROR_CHECK(err)                                                              \
  {                                                                                                 \
    cudaError_t gsb_e_ = (err);                                                                     \
    if (gsb_e_ != cudaSuccess)                                                                      \
      printf("Got Cuda Error %s: %s\n", cudaGetErrorName(gsb_e_), cudaGetErrorString(gsb_e_));      \
  }
#endif

#define GSB200_CAT2_(a, b) a##b
#define GSB200_CAT_(a, b) GSB200_CAT2_(a, b)

/* strided [rows, inner, batch] descriptor; the inner mode has unit stride */
#define GSB200_DECL_STRIDED_(P, name)      \
  typedef struct {                         \
    void* data;                            \
    int32_t dynamic_shapes[3];             \
    int64_t dynamic_strides[2];            \
  } GSB200_CAT_(P, GSB200_CAT_(_Tensor_, GSB200_CAT_(name, _t)));

/* pointer-only descriptor (the caller guarantees the extent) */
#define GSB200_DECL_POINTER_(P, name) \
  typedef struct {                    \
    void* data;                       \
  } GSB200_CAT_(P, GSB200_CAT_(_Tensor_, GSB200_CAT_(name, _t)));

#ifdef __cplusplus
#define GSB200_EXTERN_C_ extern "C"
#else
#define GSB200_EXTERN_C_
#endif

/* module type + load / unload for prefix P */
#define GSB200_DECL_MODULE_(P)                                                                        \
  typedef struct {                                                                                    \
    cudaLibrary_t module;                                                                             \
  } GSB200_CAT_(P, _Kernel_Module_t);                                                                 \
  GSB200_EXTERN_C_ void GSB200_CAT_(GSB200_CAT_(_mlir_, P), _cuda_init)(void**);                      \
  GSB200_EXTERN_C_ void GSB200_CAT_(GSB200_CAT_(_mlir_, P), _cuda_load_to_device)(void**);            \
  static inline void GSB200_CAT_(P, _Kernel_Module_Load)(GSB200_CAT_(P, _Kernel_Module_t) * m) {      \
    cudaLibrary_t* lib = &m->module;                                                                  \
    cudaError_t rc = cudaSuccess;                                                                     \
    void* init_args[2] = {(void*)&lib, (void*)&rc};                                                   \
    GSB200_CAT_(GSB200_CAT_(_mlir_, P), _cuda_init)(init_args);                                       \
    CUTE_DSL_CUDA_ERROR_CHECK(rc);                                                                    \
    int32_t dev = 0, ndev = 0;                                                                        \
    CUTE_DSL_CUDA_ERROR_CHECK(cudaGetDeviceCount(&ndev));                                             \
    void* load_args[3] = {(void*)&lib, (void*)&dev, (void*)&rc};                                      \
    for (dev = 0; dev < ndev; ++dev) {                                                                \
      GSB200_CAT_(GSB200_CAT_(_mlir_, P), _cuda_load_to_device)(load_args);                           \
      CUTE_DSL_CUDA_ERROR_CHECK(rc);                                                                  \
    }                                                                                                 \
  }                                                                                                   \
  static inline void GSB200_CAT_(P, _Kernel_Module_Unload)(GSB200_CAT_(P, _Kernel_Module_t) * m) {    \
    m->module = 0; /* the code lives in libgigaslop_b200; nothing to unload */                        \
  }

/* batch handling shared by the wrappers: the reference kernels take L batches through the third mode */
#define GSB200_BATCH_PTR_(desc, l, esz) ((char*)(desc)->data + (int64_t)(l) * (desc)->dynamic_strides[1] * (esz))

#endif /* GIGASLOP_B200_CUTE_DSL_ABI_H_ */
