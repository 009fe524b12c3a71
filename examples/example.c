/* Uses the C interface of libghostflow.so the way ghostflow-ffi/examples/example.c does:
 *   gcc examples/example.c -Ighost_flow_b200/csrc/include -Lghost_flow_b200/lib -lghostflow -o example
 *   LD_LIBRARY_PATH=ghost_flow_b200/lib ./example */
#include <stdio.h>

#include "ghostflow.h"

int main(void) {
  if (ghostflow_init() != Success) return 1;
  const char* v = ghostflow_version();
  printf("version: %s\n", v);
  ghostflow_free_string((char*)v);

  float a_data[] = {1, 2, 3, 4, 5, 6};
  float b_data[] = {1, 0, 0, 1, 1, 1};
  uintptr_t a_shape[] = {2, 3}, b_shape[] = {3, 2};
  GhostFlowTensor *a = NULL, *b = NULL, *c = NULL, *ones = NULL, *sum = NULL, *flat = NULL;
  if (ghostflow_tensor_create(a_data, 6, a_shape, 2, &a) != Success) return 2;
  if (ghostflow_tensor_create(b_data, 6, b_shape, 2, &b) != Success) return 2;
  if (ghostflow_tensor_matmul(a, b, &c) != Success) { printf("error: %s\n", ghostflow_get_last_error()); return 3; }
  uintptr_t shape[8], ndim = 0, len = 0;
  float out[16];
  ghostflow_tensor_shape(c, shape, &ndim);
  ghostflow_tensor_data(c, out, &len);
  printf("matmul -> [%lu, %lu]: %g %g %g %g\n", (unsigned long)shape[0], (unsigned long)shape[1], out[0], out[1], out[2], out[3]);
  if (out[0] != 4 || out[1] != 5 || out[2] != 10 || out[3] != 11) return 4;

  uintptr_t o_shape[] = {2, 2};
  ghostflow_tensor_ones(o_shape, 2, &ones);
  ghostflow_tensor_add(c, ones, &sum);
  uintptr_t f_shape[] = {4};
  ghostflow_tensor_reshape(sum, f_shape, 1, &flat);
  ghostflow_tensor_data(flat, out, &len);
  printf("add + reshape -> %lu values: %g %g %g %g\n", (unsigned long)len, out[0], out[1], out[2], out[3]);

  /* a failing call reports through the error string */
  GhostFlowTensor* bad = NULL;
  if (ghostflow_tensor_matmul(a, a, &bad) == InvalidShape) printf("expected failure: %s\n", ghostflow_get_last_error());

  ghostflow_tensor_free(a); ghostflow_tensor_free(b); ghostflow_tensor_free(c);
  ghostflow_tensor_free(ones); ghostflow_tensor_free(sum); ghostflow_tensor_free(flat);
  return 0;
}
