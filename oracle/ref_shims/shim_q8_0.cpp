// brotensor's own Q8_0 host reference, built from the reference tree (see
// shim_q4k.cpp for how). TEST INFRASTRUCTURE ONLY.
#define main static ref_q8_0_unused_main
#include "tests/test_q8_0_parity.cpp"
#undef main

extern "C" {
int ref_q8_0_available() { (void)&ref_q8_0_unused_main; return 1; }
void ref_q8_0_quantize_block(const float* src, unsigned char* out34) {
    quantize_q8_0_block(src, *reinterpret_cast<Q8Block*>(out34));
}
void ref_q8_0_dequant_block(const unsigned char* blk34, float* dst32) {
    dequant_q8_0_block(*reinterpret_cast<const Q8Block*>(blk34), dst32);
}
}
