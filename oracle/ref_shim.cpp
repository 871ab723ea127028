// Thin C-ABI shim over the reference's own MX scalar helpers, compiled from where the
// header lies in the reference tree (never copied into this repository). It exists to pin the
// oracle's restatement of the MXFP4 element quantiser against the reference's real code.
//
// TEST INFRASTRUCTURE ONLY: built into oracle/_ref/libtpx_mxref.so by oracle/Makefile when the
// reference tree is present; loaded by tests/golden/make_golden.py and by the oracle pin tests.
//
// The three entry points call, in the order the reference's MxFP4Quant does
// (src/csrc/qtypes.cpp:69-76, :87-98, :147-150), the functions of src/csrc/mxfp_quant.h.
#include <cstdint>
#include TPX_REF_MXFP_HEADER

extern "C" {

// MxFP4Quant(float max): shared scale from the block absmax. Returns the stored UE8M0 byte.
uint8_t ref_mx_scale_byte(float absmax, int* flush_tile, float* scale_fp_out) {
  int shared_exp = (int)get_biased_exponent(absmax);
  *flush_tile = (shared_exp == 0);
  float scale_fp = mx_get_shared_scale(shared_exp, /*scale_bits=*/8, /*elem_max_norm=*/6.0f);
  *scale_fp_out = scale_fp;
  return (uint8_t)get_biased_exponent(scale_fp);
}

// MxFP4Quant::quantize(val): the rounded value the code chain is matched against.
float ref_e2m1_round(float scaled_in) {
  return quantize_elemwise(scaled_in, /*bits=*/3, /*exp_bits=*/2, /*max_norm=*/6.0f, rd_even, true, true);
}

// get_fp_scale(byte): 2^(byte-127), byte 0 -> 0.0
float ref_fp_scale(int byte) { return get_fp_scale(byte); }

}  // extern "C"
