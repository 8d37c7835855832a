// The vision-tower entry points of the C ABI (reference: src/backends/cuda/qwen3_5/ops.h:127-142,
// vision.cu). The reference's loader refuses a library that lacks any of these symbols, so
// they are exported; the operations themselves belong to the image half of the model,
// which this library does not implement, and every call reports CS1_ERR_UNSUPPORTED.
#include "cs1_ops.h"

extern "C" {
int cs1_vision_linear(void*, const void*, const void*, const void*, void*, int, int, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_gemm_f32(void*, const float*, const float*, float*, int, int, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_norm(const void*, const void*, const void*, void*, int, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_position(void*, const void*, const int*, const float*, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_rope(const void*, const float*, const float*, void*, void*, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_attention(const void*, const void*, const void*, void*, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_bias(void*, const void*, size_t, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_gelu(void*, size_t, int, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_add(void*, const void*, size_t, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_to_float(const void*, float*, size_t, void*) { return CS1_ERR_UNSUPPORTED; }
int cs1_vision_lora_add(void*, const float*, size_t, float, void*) { return CS1_ERR_UNSUPPORTED; }
}
