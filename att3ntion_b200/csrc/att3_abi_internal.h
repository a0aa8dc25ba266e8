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

// Kernel ids of att3_timing_read().
enum KernelId { K_SG_FWD = 0, K_SG_BWD = 1, K_SG_REDUCE = 2, K_DENSE_FWD = 3, K_DENSE_BWD = 4, K_HG_AUX = 5, K_COUNT = 6 };

// Brackets one kernel launch with CUDA events on its stream while timing is
// enabled (att3_timing_enable); a no-op otherwise.
class TimedLaunch {
public:
    TimedLaunch(int kernel_id, cudaStream_t stream);
    ~TimedLaunch();
private:
    int id_;
    cudaStream_t stream_;
    cudaEvent_t start_ = nullptr;
};

}  // namespace att3
