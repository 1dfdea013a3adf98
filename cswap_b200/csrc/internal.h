// Declarations shared between the translation units of the library.
#pragma once
#include <cuda_runtime.h>

#include "../../include/cswap_b200.h"

namespace csw {

// records the runtime error for csw_last_cuda_error() and returns CSW_ERR_CUDA
csw_status cuda_fail(cudaError_t e);

// SM count and the device status word of the CURRENT device (created on first
// use; the word is zero unless a kernel gave up on a bounded wait)
csw_status device_state(int* sm_count, int** d_status);

}  // namespace csw
