// Host-side helpers shared by the C-ABI translation units: device check and launch check.
#pragma once
#include <cuda_runtime.h>

#include "../../include/nativebit_b200.h"

namespace nb {

// Records `e` as this thread's last CUDA error text and maps it to a status.
int record_cuda_error(cudaError_t e);

// Stores a message as this thread's last error text (what nb_last_cuda_error() returns).
void set_last_error(const char* msg);

// NB_OK when the current device is compute capability 10.x, else NB_ERR_ARCH / NB_ERR_LAUNCH.
int check_device();

// cudaGetLastError() after a launch -> status.
int check_launch();

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace nb
