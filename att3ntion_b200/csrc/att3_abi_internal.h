// Error plumbing shared by the translation units behind the C ABI.
#pragma once

#include <cuda_runtime.h>

#include "../../include/att3_b200.h"

namespace att3 {

// Records `msg` as the calling thread's last error and returns `code`.
int set_error(int code, const char* fmt, ...);
int set_cuda_error(cudaError_t e, const char* where);

// True when the current device can run the sm_100a kernels; otherwise records
// ATT3_ERR_UNSUPPORTED with the reason.
bool require_sm100(const char* who);

// Streaming multiprocessor count of the current device (cached per device).
int sm_count();

// Launch counters behind att3_launch_count().
void count_launch(int which, int n = 1);

}  // namespace att3
