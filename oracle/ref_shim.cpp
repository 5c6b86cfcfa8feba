// C-callable view of the reference's own MX codec header, used only to pin the
// oracle's restated codecs.  Compiled against lib/golden/mx_fp_math.h where it
// lies in the reference tree (include path given by the Makefile); no reference
// source is copied.  TEST INFRASTRUCTURE ONLY.
#include "mx_fp_math.h"

extern "C" {
float    ref_fp8_e4m3_decode(uint8_t c)   { return mx::fp8_e4m3_decode(c); }
uint8_t  ref_fp8_e4m3_to_code(float v)    { return mx::fp8_e4m3_to_code(v); }
float    ref_fpe8m0_decode(uint8_t c)     { return mx::fpe8m0_decode(c); }
float    ref_fp6_e3m2_decode(uint8_t c)   { return mx::fp6_e3m2_decode(c); }
float    ref_fp4_e2m1_decode(uint8_t c)   { return mx::fp4_e2m1_decode(c); }
uint8_t  ref_bf16_bits_to_fp4_e2m1_code(uint16_t b) { return mx::bf16_bits_to_fp4_e2m1_code(b); }
uint16_t ref_f32_to_bf16_rne(float x)     { return mx::f32_to_bf16_rne(x); }
uint8_t  ref_bf16_bits_to_fp6_e3m2_code(uint16_t b) { return mx::bf16_bits_to_fp6_e3m2_code(b); }
float    ref_fp_quantize_trunc(float x, int e, int m) { return mx::fp_quantize_trunc(x, e, m); }
}
