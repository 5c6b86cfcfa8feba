// C-callable view of the reference attention kernel's own P-requantization helpers
// (kernels/flash_attention_mx_gqa/flash_mx_impl.hpp:29-77: bf16_to_e4m3<RNE>, bf16_floor_log2,
// bf16_to_e4m3_scaled), used only to pin the oracle's restated P rule.  The header is compiled where it
// lies in the reference tree, against the reference's own lib/include (include paths given by the
// Makefile); its device-only inline functions are never called, so they are never emitted.  No reference
// source is copied.  TEST INFRASTRUCTURE ONLY.
#include <math.h>
#include <stdint.h>
#include "flash_mx_impl.hpp"

extern "C" {
uint8_t ref_bf16_to_e4m3_scaled(uint16_t b, int se) { return bf16_to_e4m3_scaled(b, se); }
int     ref_bf16_floor_log2(uint16_t b)             { return bf16_floor_log2(b); }
uint8_t ref_bf16_to_e4m3_trunc(uint16_t b)          { return bf16_to_e4m3<false>(b); }
uint8_t ref_bf16_to_e4m3_rne(uint16_t b)            { return bf16_to_e4m3<true>(b); }
}
