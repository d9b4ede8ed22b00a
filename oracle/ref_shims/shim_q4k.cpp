// Builds brotensor's own Q4_K host reference (quantizer, 6-bit scale packing,
// block decode) into oracle/_ref by including the reference's parity test from
// where it lies in the reference tree; its main() becomes an unused static
// function. Nothing from the reference is copied into this repository.
// TEST INFRASTRUCTURE ONLY.
#define main static ref_q4k_unused_main
#include "tests/test_q4k_parity.cpp"
#undef main

extern "C" {
int ref_q4k_available() { (void)&ref_q4k_unused_main; return 1; }
void ref_q4k_quantize_block(const float* src, unsigned char* out144) {
    quantize_q4k_block(src, *reinterpret_cast<Q4KBlock*>(out144));
}
void ref_q4k_dequant_block(const unsigned char* blk144, float* dst256) {
    dequant_q4k_block(*reinterpret_cast<const Q4KBlock*>(blk144), dst256);
}
void ref_q4k_pack_sc_m(unsigned char* scales12, const unsigned char* sc8, const unsigned char* m8) {
    pack_sc_m(scales12, sc8, m8);
}
void ref_q4k_unpack_sc_m(const unsigned char* scales12, unsigned char* sc8, unsigned char* m8) {
    unpack_sc_m(scales12, sc8, m8);
}
}
