// Device error words of the tcgen05 kernels: each kernel family keeps one int per GPU that a
// bounded wait sets when it gives up (0 = none did). The host executor queues a copy of the
// three words behind every forward pass and turns a non-zero word into CS1_ERR_DEVICE_CHECK,
// the way the reference surfaces every device failure as an error
// (src/models/qwen3_5/native/src/cuda.rs:177-187).
#pragma once
#include <cuda_runtime.h>

namespace s1 {
// Device address of the current device's word of each family.
int gemm_error_address(int** p);
int attn_error_address(int** p);
int gdn_error_address(int** p);
// Queues out[0..2] = {gemm, attention, delta rule} words of the current device on `st`.
int collect_status(int* out3_device, cudaStream_t st);
// Zeroes the three words of the current device (waits for the device).
int clear_status();
}  // namespace s1
