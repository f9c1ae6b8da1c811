// Host-side wrapper around the REFERENCE's own device primitive.
// TEST INFRASTRUCTURE ONLY.  Compiled by oracle/build.sh with
// -I<reference>/cuda, so cuda/AMsimulator.inl is read where it lies in the
// reference checkout and never copied here.  The four definitions below turn
// its CUDA-only spellings into host C++: the texture object becomes a byte
// pointer and tex1Dfetch a plain load.
#include <cstdint>
#include <cstring>

#define __device__
#define __inline__ inline
typedef const uint8_t* cudaTextureObject_t;
template <typename T>
static inline T tex1Dfetch(cudaTextureObject_t lut, uint32_t i) {
  return static_cast<T>(lut[i]);
}

#include "AMsimulator.inl"  // reference: cuda/AMsimulator.inl:13-36

extern "C" uint32_t ref_am_mul_bits(uint32_t at, uint32_t bt, const uint8_t* lut, int m) {
  float a, b;
  std::memcpy(&a, &at, 4);
  std::memcpy(&b, &bt, 4);
  // approx_mul_lut.h:26-28
  const uint32_t mant_mask = ((1u << m) - 1u) << (23 - m);
  const uint8_t a_shift = static_cast<uint8_t>(23 - 2 * m);
  const uint8_t b_shift = static_cast<uint8_t>(23 - m);
  const float r = AMsimulator(a, b, lut, mant_mask, a_shift, b_shift, static_cast<uint8_t>(m));
  uint32_t out;
  std::memcpy(&out, &r, 4);
  return out;
}

// Bulk form so an exhaustive sweep does not pay one FFI call per product.
extern "C" void ref_am_mul_bits_array(const uint32_t* at, const uint32_t* bt, uint32_t* out,
                                      uint64_t n, const uint8_t* lut, int m) {
  for (uint64_t i = 0; i < n; ++i) out[i] = ref_am_mul_bits(at[i], bt[i], lut, m);
}

// The reference's direct 32-bit models (cuda/FPmultMBM_fast32.inl:41-126,
// cuda/Mitchell_32.inl), device functions compiled as host C++.  Both files define the
// same four mask macros with the same values.
#undef MANTISSA_MASK
#undef EXPONENT_MASK
#undef MANTISSA_MASK_INV
#undef SIGN_MASK
#include "FPmultMBM_fast32.inl"
#undef MANTISSA_MASK
#undef EXPONENT_MASK
#undef MANTISSA_MASK_INV
#undef SIGN_MASK
#include "Mitchell_32.inl"

extern "C" void ref_direct_mul_bits_array(const uint32_t* at, const uint32_t* bt, uint32_t* out, uint64_t n,
                                          int mbm) {
  for (uint64_t i = 0; i < n; ++i) {
    float a, b;
    std::memcpy(&a, &at[i], 4);
    std::memcpy(&b, &bt[i], 4);
    const float r = mbm ? FPmultMBM_fast32(a, b) : FPmultMitch_fast32(a, b);
    std::memcpy(&out[i], &r, 4);
  }
}
