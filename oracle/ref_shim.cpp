// C entry points around the reference's own Q8_0 quantizer
// (src/core/quants.h:37-176, src/core/quants.cpp:7-18) and soft-fp16
// (src/core/float.h:32-144), compiled from the reference tree where it lies.
// Test infrastructure only: used to pin oracle/oracle.cpp and the product's
// quantizers bit for bit, and to generate tests/golden/.
#include "src/core/quants.h"

extern "C" {
// 36-byte blocks: [fp32 scale][32 x int8].
int ref_q8_0_quantize(const float *src, int8_t *dst, size_t h, size_t w) {
  return vkllama::qint8_0_quantize(src, dst, h, w).ok() ? 0 : 1;
}
int ref_q8_0_dequantize(const int8_t *src, float *dst, size_t h, size_t w) {
  return vkllama::qint8_0_dequantize(src, dst, h, w).ok() ? 0 : 1;
}
unsigned ref_q8_0_bytes_per_block(void) {
  return vkllama::get_dtype_property(vkllama::Q8_0).bytes_per_block;
}
unsigned short ref_fp32_to_fp16(float f) { return __fp32_to_fp16(f).u16; }
float ref_fp16_to_fp32(unsigned short u) { return __fp16_to_fp32(u); }
}
