// Generates an m = 11 mantissa LUT ("MBM_11.bin", 2^22 bytes) for the
// large-LUT (L2-resident) code path.  TEST INFRASTRUCTURE ONLY.
// Compiled by oracle/build.sh with -I<reference>/cuda -D__device__= so that the
// reference's 32-bit MBM functional model (cuda/FPmultMBM_fast32.inl:41-126)
// is used where it lies.  The loop restates lut/lut_gen.cc:86-127 with
// MANTISSA_BITWIDTH = 11: operands 1.i and 1.j at exponent 127, one byte per
// pair = carry flag (result exponent above 127) | low 8 bits of the top-11
// result mantissa bits.  With byte entries an 11-bit mantissa does not fit;
// the truncation is the reference format's own behaviour.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "FPmultMBM_fast32.inl"

int main(int argc, char** argv) {
  const int m = 11;
  const char* path = argc > 1 ? argv[1] : "MBM_11.bin";
  FILE* f = std::fopen(path, "wb");
  if (!f) return 1;
  const uint32_t one = 0x3f800000u;
  const uint32_t mask = ((1u << m) - 1u) << (23 - m);
  for (uint32_t i = 0; i < (1u << m); ++i) {
    for (uint32_t j = 0; j < (1u << m); ++j) {
      uint32_t at = one | (i << (23 - m)), bt = one | (j << (23 - m));
      float a, b;
      std::memcpy(&a, &at, 4);
      std::memcpy(&b, &bt, 4);
      float c = FPmultMBM_fast32(a, b);
      uint32_t ct;
      std::memcpy(&ct, &c, 4);
      uint8_t mant = static_cast<uint8_t>((ct & mask) >> (23 - m));
      uint8_t carry = ((ct & 0x7f800000u) > one) ? 0x80 : 0x00;
      uint8_t byte = carry | mant;
      std::fwrite(&byte, 1, 1, f);
    }
  }
  std::fclose(f);
  return 0;
}
