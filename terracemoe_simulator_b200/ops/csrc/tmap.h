// Tensor-map construction shared by the TMA-fed kernels (defined in gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace tb200 {

// bf16 tensor map with 128-byte swizzle; dims / box innermost first, strides in bytes for dims
// 1 .. rank - 1.  Encoded maps are cached by (base, geometry), so a training loop pays the
// driver call once per operand.  Returns TB200_OK or an error code.
int make_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box);

}  // namespace tb200
