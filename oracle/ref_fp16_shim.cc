// Thin exports around the reference's own half-precision converters, compiled from the
// reference tree where it lies (no reference source is copied).  TEST INFRASTRUCTURE ONLY.
// Wraps 3rdparty/compiler-rt/builtin_fp16.h the same way src/runtime/builtin_fp16.cc:31-43 does.
#include <builtin_fp16.h>

extern "C" {
uint16_t ref_f32_to_f16(float a) {
  return __truncXfYf2__<float, uint32_t, 23, uint16_t, uint16_t, 10>(a);
}
float ref_f16_to_f32(uint16_t a) {
  return __extendXfYf2__<uint16_t, uint16_t, 10, float, uint32_t, 23>(a);
}
uint16_t ref_f64_to_f16(double a) {
  return __truncXfYf2__<double, uint64_t, 52, uint16_t, uint16_t, 10>(a);
}
}
