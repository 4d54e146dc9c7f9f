// Tensor-core decode-on-codes kernel (placeholder until the kernel lands: reports that it
// does not handle the launch, so the general-shape kernel runs).
#include "common.cuh"

int tq_launch_decode_mma(tq_ctx*, int, const void*, int, int, int, int, float*, float*,
                         cudaStream_t, bool* handled) {
  *handled = false;
  return TQ_OK;
}
