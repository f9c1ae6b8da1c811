// Host-side wrapper around ONE of the reference's functional multiplier models
// (lut/FPmultMBM_fast1x.inl, lut/Mitchell_1x.inl, lut/bfloat.inl), selected with
// the same -D switch the reference's lut/lut_gen.cc uses.  TEST INFRASTRUCTURE
// ONLY.  Compiled by oracle/build.sh with -I<reference>/lut, once per model,
// into oracle/_ref/libref_model_<MODEL>_<m>.so; the model sources are read
// where they lie.  Used to repeat the reference's own LUT-vs-model sweep
// (lut/test.cc:70-101) against the oracle's AM primitive.
#include <cmath>
#include <cstdint>
#include <cstring>

#if defined(FMBM16_MULTIPLIER)
#include "FPmultMBM_fast16.inl"
#define REF_MODEL(a, b) FPmultMBM_fast16((a), (b))
#elif defined(FMBM14_MULTIPLIER)
#include "FPmultMBM_fast14.inl"
#define REF_MODEL(a, b) FPmultMBM_fast14((a), (b))
#elif defined(FMBM12_MULTIPLIER)
#include "FPmultMBM_fast12.inl"
#define REF_MODEL(a, b) FPmultMBM_fast12((a), (b))
#elif defined(FMBM10_MULTIPLIER)
#include "FPmultMBM_fast10.inl"
#define REF_MODEL(a, b) FPmultMBM_fast10((a), (b))
#elif defined(MITCHEL16_MULTIPLIER)
#include "Mitchell_16.inl"
#define REF_MODEL(a, b) FPmultMitch_fast16((a), (b))
#elif defined(MITCHEL14_MULTIPLIER)
#include "Mitchell_14.inl"
#define REF_MODEL(a, b) FPmultMitch_fast14((a), (b))
#elif defined(MITCHEL12_MULTIPLIER)
#include "Mitchell_12.inl"
#define REF_MODEL(a, b) FPmultMitch_fast12((a), (b))
#elif defined(MITCHEL10_MULTIPLIER)
#include "Mitchell_10.inl"
#define REF_MODEL(a, b) FPmultMitch_fast10((a), (b))
#elif defined(BFLOAT)
#include "bfloat.inl"
#define REF_MODEL(a, b) bfloat16mul((a), (b))
#else
#error "select a model with -D<MULTIPLIER>"
#endif

extern "C" float ref_model_mul(float a, float b) { return REF_MODEL(a, b); }

extern "C" void ref_model_mul_array(const uint32_t* at, const uint32_t* bt, uint32_t* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) {
    float a, b;
    std::memcpy(&a, &at[i], 4);
    std::memcpy(&b, &bt[i], 4);
    const float c = REF_MODEL(a, b);
    std::memcpy(&out[i], &c, 4);
  }
}
