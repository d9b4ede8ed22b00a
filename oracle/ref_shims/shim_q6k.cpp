// brotensor's own Q6_K host reference, built from the reference tree (see
// shim_q4k.cpp for how). TEST INFRASTRUCTURE ONLY.
#define main static ref_q6k_unused_main
#include "tests/test_q6k_parity.cpp"
#undef main

extern "C" {
int ref_q6k_available() { (void)&ref_q6k_unused_main; return 1; }
void ref_q6k_quantize_block(const float* src, unsigned char* out210) {
    quantize_q6k_block(src, *reinterpret_cast<Q6KBlock*>(out210));
}
void ref_q6k_dequant_block(const unsigned char* blk210, float* dst256) {
    dequant_q6k_block(*reinterpret_cast<const Q6KBlock*>(blk210), dst256);
}
}
