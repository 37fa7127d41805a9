// Host interface of the tensor-core Q4_K GEMV (gemv_q4k_mma.cu): used by the launchers in matvec_q4k.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gemvmma {

// Whether rows of `blocks_per_row` super-blocks fit the kernel's shared-memory operand table.
bool supported(int blocks_per_row);
// Whether the kernel needs only half an SM for such rows (two launches can then be resident together).
bool fits_half_sm(int blocks_per_row);

// y = dequant(w) . x + addend (addend may be null or alias y); asynchronous on `stream`, launched with
// programmatic dependent launch.  `speculate`: convert x and start computing while the previous kernel of
// the stream may still run; the result is published only after x has been re-checked against what
// was converted (exact either way; a stale x costs a second pass).  `timeouts`: device counter
// bumped by a CTA whose bounded wait ran out.
cudaError_t launch(const uint8_t* w, const float* x, const float* addend, float* y, int rows, int blocks_per_row,
                   int hold_trigger, int speculate, unsigned* timeouts, int sm_count, cudaStream_t stream);

}  // namespace gemvmma
