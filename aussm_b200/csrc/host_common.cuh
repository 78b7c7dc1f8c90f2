// Host-side services shared by the translation units of libaussm_b200.so.
#pragma once

#include <cuda_runtime.h>

namespace aussm {

// Message of the last failure on the calling thread (printf-style); read back by aussm_b200_last_error().
void set_error(const char* fmt, ...);

// Every kernel launch of the library is counted (process-wide, atomic); aussm_b200_kernel_launches() reports
// the total, so that a caller can state how many of the library's kernels a region launched.
void count_launch(int n = 1);
unsigned long long launch_count();

// Process-wide tuning value read by the drop-in operators: steps per time window (0 = automatic).
int window_steps_option();
// 1 (default): scans whose channels under-fill the GPU are cut into time segments; 0: never.
int time_split_option();

// Address of the device status word of the current device (nullptr on failure), and a synchronising
// read-and-clear of it.  A kernel that gives up on a bounded wait records why there and returns.
int* device_status_ptr();
cudaError_t read_and_clear_device_status(cudaStream_t stream, int* value);

}  // namespace aussm
