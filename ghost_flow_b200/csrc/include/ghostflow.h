/* C interface of ghost_flow_b200 (libghostflow.so): the 14 entry points and the error enum of GhostFlow's C ABI
 * (ghostflow-ffi/src/lib.rs:60-337), so a C program written against the reference links unchanged.
 * Tensors are opaque, dense, row-major float32 arrays on the host. Every function that can fail returns a
 * GhostFlowError and leaves a message for ghostflow_get_last_error() (per thread). */
#ifndef GHOSTFLOW_H
#define GHOSTFLOW_H

#include <stdint.h>
#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum GhostFlowError {
  Success = 0,
  InvalidShape = 1,
  InvalidData = 2,
  NullPointer = 3,
  AllocationFailed = 4,
  ComputationFailed = 5,
  Unknown = 99
} GhostFlowError;

typedef struct GhostFlowTensor GhostFlowTensor;

GhostFlowError ghostflow_init(void);
/* Heap-allocated version string; release it with ghostflow_free_string. */
const char* ghostflow_version(void);
void ghostflow_free_string(char* s);

GhostFlowError ghostflow_tensor_create(const float* data, uintptr_t data_len, const uintptr_t* shape,
                                       uintptr_t shape_len, GhostFlowTensor** out);
GhostFlowError ghostflow_tensor_zeros(const uintptr_t* shape, uintptr_t shape_len, GhostFlowTensor** out);
GhostFlowError ghostflow_tensor_ones(const uintptr_t* shape, uintptr_t shape_len, GhostFlowTensor** out);
void ghostflow_tensor_free(GhostFlowTensor* tensor);

/* out_shape must have room for the tensor's rank (query it first with out_shape == NULL). */
GhostFlowError ghostflow_tensor_shape(const GhostFlowTensor* tensor, uintptr_t* out_shape, uintptr_t* out_ndim);
/* out_data must have room for the element count (query it first with out_data == NULL). */
GhostFlowError ghostflow_tensor_data(const GhostFlowTensor* tensor, float* out_data, uintptr_t* out_len);

/* add / mul broadcast like NumPy; matmul takes [m,k] x [k,n] or batched [...,m,k] x [...,k,n]. */
GhostFlowError ghostflow_tensor_add(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out);
GhostFlowError ghostflow_tensor_mul(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out);
GhostFlowError ghostflow_tensor_matmul(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out);
GhostFlowError ghostflow_tensor_reshape(const GhostFlowTensor* tensor, const uintptr_t* new_shape,
                                        uintptr_t new_shape_len, GhostFlowTensor** out);

/* Message of the last failure on this thread (owned by the library; empty string if none). */
const char* ghostflow_get_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* GHOSTFLOW_H */
