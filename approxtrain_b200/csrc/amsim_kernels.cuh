// LUT-GEMM kernels for the AM-Simulator path, written for sm_100a.
//
// Every op of the path is one of two kernels over an abstract product
//     Out[p, q] = sum_k AM(V[p, k], U[k, q])
// where V is the operand that varies across the lanes of a warp and U the one
// that is uniform across a warp:
//
//   gather_gemm  V is gathered along k (NHWC patch rows, dense rows): conv
//                forward, conv input gradient, dense forward / input gradient,
//                batched matmul.  One ascending-k FP32 chain per output.
//   fgrad_gemm   V is gathered along p (channels of one filter tap) and the
//                reduction runs over output pixels: conv filter gradient and
//                dense weight gradient, optionally split along k.
//
// Why this shape.  Each product needs one byte from a 2^m x 2^m table.  The
// table sits in shared memory with one row per value of the WARP-UNIFORM
// operand (row = 2^m bytes, at most 128 = one word per bank), so the 32 byte
// reads of one LDS all fall into a single bank row and are served in one
// wavefront: the table lookup is conflict free by construction, whatever the
// data.  The table is placed at a shared-memory address aligned to its size,
// so "row bits | column bits | base" is a pure OR.  The inner loop per product
// is: one 3-input logic op forming the address, LDS.U8, an integer
// multiply-add that rebuilds the product's significand/exponent bits next to
// the lane operand's sign+exponent, and one FFMA with the uniform operand's
// power of two (the product of a float and a power of two is exact, so the
// FFMA rounds exactly like the reference's "accumulator + product" add).
// What bounds it: each lookup returns 4 bytes per lane through the 128-byte/clk
// shared-memory return path, i.e. 32 products per clock per SM at most; the
// operand words fetched from shared memory share that path (the lane operand
// is ONE packed word per element; the uniform operand is kept as two words,
// sign+exponent and table row, because unpacking it in the loop costs more
// issue slots than the second broadcast load costs wavefronts).  Tensor cores
// cannot be used: no product is a hardware multiply.
//
// Besides the plain grid (one CTA per 128 x 64 tile) gather_gemm has a balanced
// mode (equal runs of (tile, reduction block) pairs over exactly the resident
// CTAs, shared tiles combined in CTA order by the CTA that finishes last), a
// cluster mode (the same split through distributed shared memory, used under
// graph capture) and a narrow-output mode (several warps share a column group);
// fgrad_exact_thin serves outputs too small for the 128 x 64 tiles.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace amsim {

constexpr int BK = 16;  // reduction steps per shared-memory stage
constexpr int BQ = 64;  // q extent of a CTA tile (4 warps x 16)
constexpr int TR = 16;  // q values per warp, held as registers
constexpr int TC = 4;   // consecutive p values per lane
constexpr int US = BQ + 4;  // padded U row (words): 2-way instead of 16-way store conflicts for k-contiguous loads
// One double-buffered U tile, in words.  Additive tables keep a second tile right behind the
// first: sign+exponent words in the first, mantissa-field words in the second, so the inner
// loop (pure arithmetic there, shared memory has room) does not unpack them per k-step.
constexpr int U_TILE_WORDS = 2 * BK * US;
// (the shared-memory table path stores the uniform operand the same way: sign+exponent word
// and table-row word apart saves the per-k-step unpacking for one more broadcast load: +0.6 %)
__host__ __device__ constexpr bool lm_split_u(int lm) { return lm == 2 /* LM_ADD */ || lm == 0 /* LM_SMEM */; }

#ifndef AMSIM_CTAS1
#define AMSIM_CTAS1 3
#endif
#ifndef AMSIM_KUNROLL
#define AMSIM_KUNROLL 1
#endif
#define AMSIM_STR2(x) #x
#define AMSIM_STR(x) AMSIM_STR2(x)
#define AMSIM_UNROLL_K _Pragma(AMSIM_STR(unroll AMSIM_KUNROLL))

// Division by a run-time constant: n / d for n < 2^31.
struct FastDiv {
  uint32_t mul, shr, d;
};

inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d ? d : 1;
  if (f.d == 1) {
    f.mul = 0;
    f.shr = 0;
    return f;
  }
  uint32_t lg = 0;
  while ((1ull << lg) < f.d) ++lg;  // ceil(log2 d)
  const uint32_t p = 31 + lg;
  f.mul = (uint32_t)(((1ull << p) + f.d - 1) / f.d);
  f.shr = p - 32;
  return f;
}

__host__ __device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv& f) {
#ifdef __CUDA_ARCH__
  return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.shr);
#else
  return f.d == 1 ? n : (uint32_t)(((uint64_t)n * f.mul) >> 32) >> f.shr;
#endif
}

// How a flat index decomposes into (image, row, col) of a grid, and how a
// filter tap displaces it into the source tensor.  Covers the forward patch
// gather (cuda_kernel.cu:39-58 of the reference), the stride-dilated,
// back-padded gather of the input gradient (:467-500) and the filter-gradient
// gather (:331-350).
struct Gather {
  int PH, PW;          // grid the flat index runs over
  int ps_h, ps_w;      // grid step in source coordinates
  int off_t, off_l;    // padding subtracted
  int lim_h, lim_w;    // source coordinate must be in [0, lim)
  int dil_h, dil_w;    // ... and a multiple of this (1 except input gradient)
  int SH, SW, SC;      // source tensor rows, cols, channels
  int KW;              // filter columns (tap = kh * KW + kw)
  FastDiv d_img, d_pw, d_sc, d_kw, d_dh, d_dw;
};

// Bounds-checking debug build (-DAMSIM_BOUNDS_CHECK; stands in for compute-sanitizer's memcheck):
// every access of the kernels to a caller's tensor or to scratch is first compared with that
// buffer's extent and natural alignment.  A bad access is NOT made: the first one is recorded
// (source line, buffer, byte offset) in a device word the host reads back with
// amsim_debug_bounds_report(), a bad load yields 0, a bad store is dropped, and the kernel carries
// on, so the context stays usable.  In a normal build AMSIM_IN() is the constant true.
constexpr int BUF_V = 0, BUF_U = 1, BUF_O = 2, BUF_WS = 3;
#ifdef AMSIM_BOUNDS_CHECK
struct Bounds {
  const char* lo[4];
  const char* hi[4];
  unsigned long long* report;  // 0 = clean; else line << 44 | (buffer + 1) << 40 | low 40 bits of the byte offset
};
__device__ __noinline__ void amsim_bounds_record(const Bounds& b, int which, const void* p, int line) {
  const unsigned long long off = (unsigned long long)((const char*)p - b.lo[which]) & ((1ull << 40) - 1);
  atomicCAS(b.report, 0ull, ((unsigned long long)line << 44) | ((unsigned long long)(which + 1) << 40) | off);
}
__device__ __forceinline__ bool amsim_in(const Bounds& b, int which, const void* p, size_t bytes, int line) {
  const char* a = (const char*)p;
  if (a >= b.lo[which] && a + bytes <= b.hi[which] && ((uintptr_t)a & (bytes - 1)) == 0) return true;
  amsim_bounds_record(b, which, p, line);
  return false;
}
#define AMSIM_IN(prm_, which_, ptr_, type_) amsim_in((prm_).bnd, which_, ptr_, sizeof(type_), __LINE__)
#else
#define AMSIM_IN(prm_, which_, ptr_, type_) true
#endif

struct Params {
  const float* V;
  const float* U;
  float* O;
  int P, Q, K;  // extents of p, q and the reduction
  Gather g;
  // U element for reduction index k = tap * g.SC + kk and column q sits at
  //   U[tap' * u_tap + kk * u_sk + q * u_sq],
  //   tap' = u_t0 + (tap / g.KW) * u_tj + (tap % g.KW) * u_ti
  // (negative steps fold the spatial flip of cuda/reverseNswapdim23.cu into the
  // index map; steps larger than one select the taps of one stride phase).
  long long u_tap;
  int u_sk, u_sq, u_t0, u_tj, u_ti;
  long long o_sp, o_sq;         // Out[p, q] at O[row(p) * o_sp + q * o_sq]
  // row(p) = p, or for a strided output grid (one stride phase of an input
  // gradient): p -> (n, yy, xx) over g.PH x g.PW, row = (n*o_h + yy*o_sh + o_a)*o_w + xx*o_sw + o_b
  int o_strided, o_h, o_w, o_sh, o_sw, o_a, o_b;
  long long v_bs, u_bs, o_bs;   // per-blockIdx.z (batch) offsets
  const uint8_t* lut;           // encoded table, rows of `rowstride` bytes
  int lut_bytes;                // multiple of 16
  int m;
  uint32_t mult;                // 1 << (23 - m)
  uint32_t rowstride;           // 1 << m
  uint32_t rmask;               // ((1 << m) - 1) << m : row bits of a table address
  uint32_t cmask;               // (1 << m) - 1        : column bits
  uint32_t cadj;                // global-table path: 2^23 - 128 * mult (carry bit of a raw byte)
  const uint8_t* lut_raw;       // global-table path (m > 7): raw bytes, rows by the uniform operand
  uint32_t lut_align;           // power of two >= lut_bytes: alignment of the table in shared memory
  // gather_gemm, fast mode: CTAs of one thread-block cluster split the reduction and
  // combine their register tiles through distributed shared memory (1 = no split)
  int ksplit;
  int tile_bytes;               // bytes reserved before the table (operand tiles, or the exchange buffer)
  int lut_mode;                 // LM_SMEM / LM_GLOBAL / LM_ADD (host-side dispatch)
  int v_first;                  // the lane operand V is the multiplier's first operand (int32 kernels)
  // gather_gemm epilogue: out = act(acc + bias[q]); both optional (exact FP32 add, then max with 0)
  // out = act(acc * alpha * scale[q] + bias[q]): every factor optional, each step one FP32 operation
  const float* bias;
  const float* scale;
  float alpha;                  // used when has_alpha
  int has_alpha;
  int relu;
  // gather_gemm, matmul with a transposed first operand: V[p, k] sits at V[k * v_ld + p]
  int v_trans;
  long long v_ld;
  int u_vec;                    // gather_gemm: 128-bit loads of U along q (1) or along k (2); 0 = scalar
  int exact_only;               // deterministic kernels: never take the fast arithmetic, even for hazard-free stages
  // fgrad only
  int k_chunk, splits;
  float* ws;                    // [splits][P][Q] partial sums when splits > 1
  // gather_gemm, balanced mode: the (tile, reduction block) pairs of the whole problem are
  // dealt out in equal contiguous runs to the CTAs of a grid that exactly fills the GPU; a tile
  // whose reduction is shared between CTAs goes through `ws` (two register-tile slots per CTA)
  long long sk_iters;           // tiles * reduction blocks per tile
  int sk_ptiles, sk_qtiles;     // tile grid (q runs fastest, then p, then batch)
  int sk_grid;                  // CTAs of the balanced launch
  int* sk_count;                // per tile: CTAs that have parked their share (zero before the launch)
  long long v_elems, u_elems, o_elems;  // extents of V, U and O in elements (bounds-checking build)
#ifdef AMSIM_BOUNDS_CHECK
  Bounds bnd;
#endif
};

__device__ __forceinline__ uint32_t lds_u8(uint32_t saddr) {
  uint32_t v;
  asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(saddr));
  return v;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// How gather_gemm spreads the reduction.
constexpr int GM_PLAIN = 0;     // one CTA per tile, whole reduction
constexpr int GM_CLUSTER = 1;   // a thread-block cluster shares a tile's reduction
constexpr int GM_BALANCED = 2;  // equal runs of (tile, reduction block) per CTA, partial tiles via workspace

// Where the products' table bits come from.
constexpr int LM_SMEM = 0;    // 2^m x 2^m byte table in shared memory (m <= 7)
constexpr int LM_GLOBAL = 1;  // raw table in global memory, L2-resident (m = 8..11)
constexpr int LM_ADD = 2;     // additive table, entry(i, j) == i + j for every pair (Mitchell-type
                              // multipliers): the lookup is an integer add of the operands' mantissa
                              // fields, no table access at all; detected when the LUT is opened

constexpr int LM_GLOBAL16 = 5;  // table of 16-bit entries in global memory (carry << 15 | top 15 mantissa bits)
__host__ __device__ constexpr bool lm_global(int lm) { return lm == LM_GLOBAL || lm == LM_GLOBAL16; }
// Table term of one product from a table in global memory: (carry << 23) + mantissa bits.
template <int LM>
__device__ __forceinline__ uint32_t global_entry(const uint8_t* __restrict__ lut_g, uint32_t idx, uint32_t mult,
                                                 uint32_t cadj) {
  if (LM == LM_GLOBAL16) {
    const uint32_t v = __ldg(reinterpret_cast<const uint16_t*>(lut_g) + idx);
    return ((v & 0x7FFFu) << 8) + ((v >> 15) << 23);
  }
  const uint32_t v = __ldg(lut_g + idx);
  return v * mult + (v >> 7) * cadj;
}
constexpr int LM_DIRECT_MBM = 3;  // no table: the 32-bit minimally-biased model computed per product
constexpr int LM_DIRECT_MIT = 4;  // no table: the 32-bit Mitchell model computed per product
__host__ __device__ constexpr bool lm_direct(int lm) { return lm == LM_DIRECT_MBM || lm == LM_DIRECT_MIT; }

// Direct simulation of the reference's 32-bit multipliers (cuda/FPmultMBM_fast32.inl:13-126,
// cuda/Mitchell_32.inl), for mantissa widths too large for a table.  Sign and exponent come
// from the exact FP32 product; the mantissa is the approximate one; the exponent moves by
// ("approximate mantissa product reached 2") - ("exact mantissa product, rounded to 24 bits,
// reached 2").  An exact product that is inf/NaN passes through, one that is zero or
// subnormal gives +0.  The rounded exact mantissa product is taken from an FP32 multiply of
// 1.ma and 1.mb (same round-to-nearest-even at the same bit as the reference's 48-bit
// integer product with hand rounding).
template <bool MBM>
__device__ __forceinline__ uint32_t direct_mul_bits(uint32_t at, uint32_t bt) {
  const uint32_t eb = __float_as_uint(__fmul_rn(__uint_as_float(at), __uint_as_float(bt)));
  const uint32_t eexp = (eb >> 23) & 0xFFu;
  if (eexp == 255u) return eb;
  if (eexp == 0u) return 0u;
  const uint32_t ma = at & 0x7FFFFFu, mb = bt & 0x7FFFFFu;
  const uint32_t exact_two =
      __fmul_rn(__uint_as_float(0x3F800000u | ma), __uint_as_float(0x3F800000u | mb)) >= 2.0f ? 1u : 0u;
  const uint32_t s = ma + mb;
  const uint32_t carry = s >> 23;  // s < 2^24
  uint32_t t = s & 0x7FFFFFu;
  if (MBM) {
    t += 0xA0000u >> carry;                    // 2^-4 + 2^-6, halved after a carry
    if (carry && t >= 0x800000u) t = s;        // correction would overflow: dropped
  }
  uint32_t w = (0x800000u + t) << carry;
  const uint32_t approx_two = w >= 0x1000000u ? 1u : 0u;
  w >>= approx_two;
  return (eb & 0x80000000u) + ((eexp - exact_two + approx_two) << 23) + (w & 0x7FFFFFu);
}

// ---- operand encodings -------------------------------------------------------
// Lane operand (V): one word = sign+exponent bits | table column.
//   fast:  a zero exponent field (zero or denormal) becomes the word 0, which
//          the inner loop predicates off: the product is exactly 0.
//   exact: the raw fields, nothing special-cased (the reference pushes zeros
//          and denormals through the table like any other value).
//   additive table: the word keeps the top-m mantissa bits in place instead of
//          a column index (sign | exponent | truncated mantissa).
template <bool EXACT, int LM>
__device__ __forceinline__ uint32_t enc_v(uint32_t bits, int m) {
  if (lm_direct(LM)) return bits;  // the model works on the raw operands
  uint32_t w;
  if (LM == LM_ADD) {
    w = bits & ~((1u << (23 - m)) - 1u);
  } else {
    const uint32_t idx = (bits >> (23 - m)) & ((1u << m) - 1u);
    w = (bits & 0xFF800000u) | idx;
  }
  if (EXACT) return w;
  return (bits & 0x7F800000u) ? w : 0u;
}

// Deterministic mode on fast arithmetic.  The fast inner loop (IMAD + FFMA) produces the
// reference's bits whenever no product of a stage can hit one of the reference's special
// behaviours: exponent sum <= 127 (the reference returns 0), exponent overflow (it wraps into
// the sign), or an exponent-0 operand meeting an operand >= 2 (it returns a non-zero residue).
// Staging collects, per stage, whether any operand lies outside a window that rules all of
// that out; a stage with a hazard runs the bit-by-bit loop instead.  Typical activations,
// weights and gradients (magnitudes 2^-63 .. 2^63, zeros) never leave the window.
constexpr uint32_t HZ_V0 = 1u, HZ_VBIG = 2u, HZ_U0 = 4u, HZ_UBIG = 8u, HZ_OUT = 16u;
__device__ __forceinline__ uint32_t hazard_bits(uint32_t bits, bool is_u) {
  const uint32_t e = (bits >> 23) & 0xFFu;
  uint32_t h = 0;
  if (e == 0u) h |= is_u ? HZ_U0 : HZ_V0;
  else if (e - 64u > 126u) h |= HZ_OUT;            // outside [64, 190]
  if (e >= 128u) h |= is_u ? HZ_UBIG : HZ_VBIG;
  return h;
}
__device__ __forceinline__ bool hazard_free(uint32_t h) {
  return !(h & HZ_OUT) && !((h & HZ_V0) && (h & HZ_UBIG)) && !((h & HZ_U0) && (h & HZ_VBIG));
}

// One reduction step of a 16 (q) x 4 (p) register tile.
//   vrow : 4 consecutive lane-operand words (sign+exponent | column)
//   urow : 16 uniform-operand words (sign+exponent | column << m)
//   lut_base : shared-memory address of the table (aligned to its size)
//   LM   : LM_SMEM table in shared memory at lut_base; LM_GLOBAL raw table in global
//          memory at lut_g; LM_ADD no table (additive: an integer add of mantissa fields).
// NZEXP: the lane words carry the deterministic encoding (exponent-0 operands keep their
// fields), so "operand is zero" is read from the exponent field instead of the whole word.
template <bool EXACT, int LM, bool NZEXP = false>
__device__ __forceinline__ void mac_step(float (&acc)[TR][TC], const uint32_t* __restrict__ vrow,
                                         const uint32_t* __restrict__ urow, const uint32_t lut_base,
                                         const uint32_t rmask, const uint32_t mult, const uint32_t cmask,
                                         const uint32_t cadj, const uint8_t* __restrict__ lut_g) {
  const uint4 cw = *reinterpret_cast<const uint4*>(vrow);
  const uint32_t w[TC] = {cw.x, cw.y, cw.z, cw.w};
  uint32_t ci[TC], cs[TC];
  int cn[TC];
  bool nz[TC];
#pragma unroll
  for (int t = 0; t < TC; ++t) {
    ci[t] = lm_global(LM) ? (w[t] & cmask) : ((w[t] & 0xFFu) | lut_base);
    nz[t] = NZEXP ? (w[t] & 0x7F800000u) != 0u : w[t] != 0u;
    if (EXACT) {
      // AMsimulator.inl:26-33: exponent sum - 127, folded into the lane word
      // (additive table: the word's mantissa field stays in, it IS the table term)
      cs[t] = (LM == LM_ADD ? w[t] : (w[t] & 0xFF800000u)) - 0x3F800000u;
      cn[t] = (int)(0x3F800000u - (w[t] & 0x7F800000u));
    } else {
      cs[t] = LM == LM_ADD ? w[t] : (w[t] & 0xFF800000u);
    }
  }
#pragma unroll
  for (int g4 = 0; g4 < TR / 4; ++g4) {
    const uint4 u4 = *reinterpret_cast<const uint4*>(urow + 4 * g4);
    const uint32_t uu[4] = {u4.x, u4.y, u4.z, u4.w};
    uint32_t dd[4] = {0u, 0u, 0u, 0u};
    if (lm_split_u(LM)) {  // the second word of the uniform operand: mantissa field (additive) or table row bits
      const uint4 d4 = *reinterpret_cast<const uint4*>(urow + U_TILE_WORDS + 4 * g4);
      dd[0] = d4.x; dd[1] = d4.y; dd[2] = d4.z; dd[3] = d4.w;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t pp = lm_split_u(LM) ? uu[r] : (uu[r] & 0xFF800000u);
      const int ee = (int)(uu[r] & 0x7F800000u);
      const uint32_t du = dd[r];
#pragma unroll
      for (int t = 0; t < TC; ++t) {
        if (lm_direct(LM)) {  // both models are symmetric in their operands
          acc[4 * g4 + r][t] = __fadd_rn(acc[4 * g4 + r][t], __uint_as_float(direct_mul_bits<LM == LM_DIRECT_MBM>(w[t], uu[r])));
          continue;
        }
        // e = (carry << 23) + (mantissa bits << (23 - m)), AMsimulator.inl:22-23,31
        uint32_t e;
        if (LM == LM_ADD) {
          e = du;  // entry(i, j) << (23 - m) == (i << (23 - m)) + (j << (23 - m)); the j term is in cs
        } else if (lm_global(LM)) {
          e = global_entry<LM>(lut_g, (uu[r] & rmask) | ci[t], mult, cadj);
        } else {
          e = lds_u8(dd[r] | ci[t]) * mult;
        }
        if (EXACT) {
          // bits = sign + ((ea + eb - 127 + carry) << 23) + mantissa, uint32 wrap
          const uint32_t bits = e + (pp + cs[t]);
          // product is +0 when ea + eb <= 127 (AMsimulator.inl:28); adding +0
          // never changes a non-negative-zero accumulator, so skip the add.
          if (ee > cn[t]) acc[4 * g4 + r][t] = __fadd_rn(acc[4 * g4 + r][t], __uint_as_float(bits));
        } else {
          const float y = __uint_as_float(e + cs[t]);
          const float sacc = __fmaf_rn(__uint_as_float(pp), y, acc[4 * g4 + r][t]);
          acc[4 * g4 + r][t] = nz[t] ? sacc : acc[4 * g4 + r][t];
        }
      }
    }
  }
}

__device__ __forceinline__ void copy_lut_to_smem(uint8_t* lut_s, const uint8_t* __restrict__ lut, int bytes,
                                                 int tid, int nthreads) {
  const uint4* src = reinterpret_cast<const uint4*>(lut);
  uint4* dst = reinterpret_cast<uint4*>(lut_s);
  for (int i = tid; i < bytes / 16; i += nthreads) dst[i] = __ldg(src + i);
}

// Uniform operand (U): one word = sign+exponent bits | table row bits.
template <int LM>
__device__ __forceinline__ uint32_t enc_u(uint32_t bits, int m) {
  if (lm_direct(LM)) return bits;
  if (LM == LM_ADD) return bits & ~((1u << (23 - m)) - 1u);  // sign | exponent | truncated mantissa
  return (bits & 0xFF800000u) | (((bits >> (23 - m)) & ((1u << m) - 1u)) << m);
}

// Stores one encoded uniform-operand word (additive tables: its two halves in the two tiles).
template <int LM>
__device__ __forceinline__ void store_u(uint32_t* dst, uint32_t bits, int m) {
  const uint32_t w = enc_u<LM>(bits, m);
  if (lm_split_u(LM)) {
    dst[0] = w & 0xFF800000u;
    dst[U_TILE_WORDS] = w & 0x007FFFFFu;
  } else {
    dst[0] = w;
  }
}
template <int LM>
__device__ __forceinline__ void store_u4(uint32_t* dst, const float (&f)[4], int m) {
  uint4 w;
  w.x = enc_u<LM>(__float_as_uint(f[0]), m);
  w.y = enc_u<LM>(__float_as_uint(f[1]), m);
  w.z = enc_u<LM>(__float_as_uint(f[2]), m);
  w.w = enc_u<LM>(__float_as_uint(f[3]), m);
  if (lm_split_u(LM)) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(w.x & 0xFF800000u, w.y & 0xFF800000u, w.z & 0xFF800000u, w.w & 0xFF800000u);
    *reinterpret_cast<uint4*>(dst + U_TILE_WORDS) =
        make_uint4(w.x & 0x007FFFFFu, w.y & 0x007FFFFFu, w.z & 0x007FFFFFu, w.w & 0x007FFFFFu);
  } else {
    *reinterpret_cast<uint4*>(dst) = w;
  }
}

template <int WP>
struct SmemLayout {
  static constexpr int NT = WP * 128;
  static constexpr int BP = WP * 128;
  static constexpr int VS = BP + 4;  // padded row: conflict-free 4-row scatter
  static constexpr int V_WORDS = 2 * BK * VS;
  static constexpr int U_WORDS = 2 * U_TILE_WORDS;  // the second tile is used by additive tables only
  static constexpr int FLAG_WORDS = 2 * 4 * WP;  // deterministic kernels: one hazard word per stage and warp
  static constexpr int TILE_BYTES = (V_WORDS + U_WORDS + FLAG_WORDS) * 4;
  // tiles, then the table at the next multiple of its alignment
  static constexpr int EXCHANGE_BYTES = TR * TC * NT * 4;  // one register tile per thread
  static size_t bytes(int tile_bytes, int lut_bytes, int lut_align) { return (size_t)tile_bytes + lut_align + lut_bytes; }
};

// -----------------------------------------------------------------------------
// gather_gemm: V gathered along k.  grid = (ceil(P/BP), ceil(Q/64), batch).
// -----------------------------------------------------------------------------
// Writes one thread's 16 (q) x 4 (p) register tile: out = act(acc + bias[q]) at Out[row(p), q].
__device__ __forceinline__ void store_out_tile(const Params& prm, float (&acc)[TR][TC], float* __restrict__ Og,
                                               const int prow0, const int qcol0) {
  const Gather& g = prm.g;
  const bool vec_out = prm.o_sq == 1 && (prm.o_sp & 3) == 0 && (prm.o_bs & 3) == 0 &&
                       ((reinterpret_cast<uintptr_t>(prm.O) & 15) == 0);
#pragma unroll
  for (int c = 0; c < TC; ++c) {
    const int pg = prow0 + c;
    if (pg >= prm.P) continue;
    long long row = pg;
    if (prm.o_strided) {
      const uint32_t n = fdiv((uint32_t)pg, g.d_img);
      const uint32_t rem = (uint32_t)pg - n * (uint32_t)(g.PH * g.PW);
      const uint32_t yy = fdiv(rem, g.d_pw);
      const uint32_t xx = rem - yy * (uint32_t)g.PW;
      row = ((long long)n * prm.o_h + (long long)yy * prm.o_sh + prm.o_a) * prm.o_w + (long long)xx * prm.o_sw + prm.o_b;
    }
    float* orow = Og + row * prm.o_sp;
#pragma unroll
    for (int g4 = 0; g4 < TR / 4; ++g4) {
      const int qg = qcol0 + 4 * g4;
      float o[4] = {acc[4 * g4][c], acc[4 * g4 + 1][c], acc[4 * g4 + 2][c], acc[4 * g4 + 3][c]};
      if (prm.bias != nullptr || prm.relu || prm.scale != nullptr || prm.has_alpha) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (prm.has_alpha) o[r] = __fmul_rn(o[r], prm.alpha);
          if (prm.scale != nullptr && qg + r < prm.Q) o[r] = __fmul_rn(o[r], __ldg(prm.scale + qg + r));
          if (prm.bias != nullptr && qg + r < prm.Q) o[r] = __fadd_rn(o[r], __ldg(prm.bias + qg + r));
          if (prm.relu) o[r] = o[r] < 0.f ? 0.f : o[r];
        }
      }
      if (vec_out && qg + 3 < prm.Q) {
        if (AMSIM_IN(prm, BUF_O, orow + qg, float4)) *reinterpret_cast<float4*>(orow + qg) = make_float4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if (qg + r < prm.Q && AMSIM_IN(prm, BUF_O, orow + (long long)(qg + r) * prm.o_sq, float)) orow[(long long)(qg + r) * prm.o_sq] = o[r];
      }
    }
  }
}

// First reduction block of CTA c in a balanced launch of `grid` CTAs over `iters` blocks.
__device__ __forceinline__ long long balanced_begin(long long c, long long iters, int grid) {
  return c * iters / grid;
}

// QS (fast mode, plain grid, narrow outputs Q <= 64 / QS): the CTA's four warps would mostly idle
// on a 64-column tile, so the tile is 64 / QS columns wide and QS warps share each 16-column
// group, taking every QS-th reduction step; their register tiles are added in warp order at the end.
template <int WP, bool EXACT, bool VEC, int MODE, int LM, int QS = 1>
__global__ void __launch_bounds__(WP * 128, WP == 1 ? AMSIM_CTAS1 : 2) gather_gemm(const Params prm) {
  using L = SmemLayout<WP>;
  constexpr int NT = L::NT, BP = L::BP, VS = L::VS;
  constexpr int BQE = BQ / QS;  // columns this CTA produces
  static_assert(QS == 1 || (WP == 1 && !EXACT && MODE == GM_PLAIN), "warps share columns only in plain fast launches");
  constexpr int NU = BK * BQ / NT;  // U elements staged per thread
  constexpr bool CLUSTER = MODE == GM_CLUSTER;
  constexpr bool BALANCED = MODE == GM_BALANCED;

  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* Vs = reinterpret_cast<uint32_t*>(smem);
  uint32_t* Us = Vs + L::V_WORDS;
  uint32_t* Fs = Us + L::U_WORDS;  // per stage and warp: hazard bits of the staged operands
  constexpr bool HAZARD_CHECK = EXACT && !lm_direct(LM);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t lut_base = (smem_base + prm.tile_bytes + prm.lut_align - 1) & ~(prm.lut_align - 1);
  uint8_t* lut_s = smem + (lut_base - smem_base);

  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int wp = w % WP, wq = (w / WP) / QS, ksub = (w / WP) % QS;  // column group, share of the reduction steps
  const int ksplit = CLUSTER ? prm.ksplit : 1;   // cluster size along x
  const int krank = blockIdx.x % ksplit;         // this CTA's slice of the reduction
  const Gather& g = prm.g;
  const int nkb_all = (prm.K + BK - 1) / BK;

  uint32_t* flag_s = Fs;  // balanced mode (fast kernels only, where Fs is otherwise unused): "this CTA completes the tile"
  // Balanced mode: this CTA's run of (tile, reduction block) pairs; otherwise one pass.
  long long run_at = 0, run_end = 0;
  if (BALANCED) {
    run_at = balanced_begin(blockIdx.x, prm.sk_iters, prm.sk_grid);
    run_end = balanced_begin((long long)blockIdx.x + 1, prm.sk_iters, prm.sk_grid);
    if (run_at >= run_end) return;
  }
  // ---- the segment being staged: a tile and a range of its reduction blocks ----------------
  // (in balanced mode the staging moves on to the next segment during the last stage of the
  // current one, so these are variables; the tile being accumulated is kept in seg_at)
  int tile_p = 0, tile_q = 0, tile_z = 0, kb_begin = 0, nkb = 0, p0 = 0, q0 = 0;
  const float* __restrict__ Vg = prm.V;
  const float* __restrict__ Ug = prm.U;
  auto decode_tile = [&](long long at, int& tp, int& tq, int& tz, int& kb0, int& kb1) {
    const long long tile = at / nkb_all;
    kb0 = (int)(at - tile * nkb_all);
    kb1 = kb0 + (int)min((long long)(nkb_all - kb0), run_end - at);
    tq = (int)(tile % prm.sk_qtiles);
    const long long rest = tile / prm.sk_qtiles;
    tp = (int)(rest % prm.sk_ptiles);
    tz = (int)(rest / prm.sk_ptiles);
  };
  // ---- this thread's share of the V tile: 4 rows (p) x one group of 4 k ------
  // A warp's 128-bit gather covers 8 rows x 64 contiguous bytes (the four k groups of a stage):
  // half as many cache lines per request as 16 rows x 32 bytes.  The L1 data stage spends its
  // cycles per line touched, and shares them with the table lookups: with 16 lines per request
  // the gathers took a tenth of the data pipe (24 cycles per request, where the filter
  // gradient's contiguous requests take 5); this layout made the 3x3 forward and input-gradient
  // kernels 3-5 % faster.  In shared memory the rows of k groups 2 and 3 are stored with
  // bit 3 of the column flipped, so that the four groups' stores fall into different banks;
  // the inner loop reads k rows 8..15 at its own column with the same bit flipped.
  constexpr int NPX = 4;
  int pl[NPX], r0[NPX], c0[NPX];
  long long nb[NPX];
  bool pv[NPX];
#pragma unroll
  for (int ip = 0; ip < NPX; ++ip) pl[ip] = (ip * 4 * WP + w) * 8 + (lane >> 2);
  // Points the staging at the segment that starts at run position run_at (balanced mode; advances
  // run_at past it) or at this CTA's tile (plain and cluster launches).
  auto next_segment = [&]() {
    if (BALANCED) {
      decode_tile(run_at, tile_p, tile_q, tile_z, kb_begin, nkb);
      run_at += nkb - kb_begin;
    } else {
      tile_p = blockIdx.x / ksplit;
      tile_q = blockIdx.y;
      tile_z = blockIdx.z;
      const int per = (nkb_all + ksplit - 1) / ksplit;
      kb_begin = krank * per;
      nkb = min(kb_begin + per, nkb_all);
    }
    p0 = tile_p * BP;
    q0 = tile_q * BQE;
    Vg = prm.V + (long long)tile_z * prm.v_bs;
    Ug = prm.U + (long long)tile_z * prm.u_bs;
#pragma unroll
    for (int ip = 0; ip < NPX; ++ip) {
      const uint32_t pg = (uint32_t)(p0 + pl[ip]);
      pv[ip] = pg < (uint32_t)prm.P;
      const uint32_t n = fdiv(pg, g.d_img);
      const uint32_t rem = pg - n * (uint32_t)(g.PH * g.PW);
      const uint32_t a = fdiv(rem, g.d_pw);
      const uint32_t b = rem - a * (uint32_t)g.PW;
      r0[ip] = (int)a * g.ps_h - g.off_t;
      c0[ip] = (int)b * g.ps_w - g.off_l;
      nb[ip] = (long long)n * ((long long)g.SH * g.SW * g.SC);
    }
  };
  const int kg = lane & 3;  // this thread's group of four reduction steps of a stage

  float4 vraw[NPX];
  float uraw[NU];
  const bool u_kmajor = prm.u_sk == 1 && prm.u_sq != 1;

  auto load_tile = [&](int kb) {
    {
      const int kglob = kb * BK + 4 * kg;
      if (VEC) {
        const uint32_t tap = fdiv((uint32_t)kglob, g.d_sc);
        const int ch = kglob - (int)tap * g.SC;
        const int kh = (int)fdiv(tap, g.d_kw);
        const int kw = (int)tap - kh * g.KW;
#pragma unroll
        for (int ip = 0; ip < NPX; ++ip) {
          float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
          const int u = r0[ip] + kh, v = c0[ip] + kw;
          if (pv[ip] && kglob < prm.K && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w) {
            // only the deterministic input gradient gathers a stride-dilated tensor (fast mode runs
            // one sub-convolution per stride phase instead)
            const int row = EXACT ? (int)fdiv((uint32_t)u, g.d_dh) : u, col = EXACT ? (int)fdiv((uint32_t)v, g.d_dw) : v;
            const float* src = Vg + nb[ip] + ((long long)(row * g.SW + col) * g.SC + ch);
            if ((!EXACT || (row * g.dil_h == u && col * g.dil_w == v)) && AMSIM_IN(prm, BUF_V, src, float4))
              val = __ldg(reinterpret_cast<const float4*>(src));
          }
          vraw[ip] = val;
        }
      } else {
        float tmp[NPX][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kj = kglob + j;
          const uint32_t tap = fdiv((uint32_t)kj, g.d_sc);
          const int ch = kj - (int)tap * g.SC;
          const int kh = (int)fdiv(tap, g.d_kw);
          const int kw = (int)tap - kh * g.KW;
#pragma unroll
          for (int ip = 0; ip < NPX; ++ip) {
            float val = 0.f;
            const int u = r0[ip] + kh, v = c0[ip] + kw;
            if (prm.v_trans) {
              if (pv[ip] && kj < prm.K && AMSIM_IN(prm, BUF_V, Vg + (long long)kj * prm.v_ld + (p0 + pl[ip]), float))
                val = __ldg(Vg + (long long)kj * prm.v_ld + (p0 + pl[ip]));
            } else if (pv[ip] && kj < prm.K && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w) {
              const int row = EXACT ? (int)fdiv((uint32_t)u, g.d_dh) : u, col = EXACT ? (int)fdiv((uint32_t)v, g.d_dw) : v;
              const float* src = Vg + nb[ip] + ((long long)(row * g.SW + col) * g.SC + ch);
              if ((!EXACT || (row * g.dil_h == u && col * g.dil_w == v)) && AMSIM_IN(prm, BUF_V, src, float)) val = __ldg(src);
            }
            tmp[ip][j] = val;
          }
        }
#pragma unroll
        for (int ip = 0; ip < NPX; ++ip) vraw[ip] = make_float4(tmp[ip][0], tmp[ip][1], tmp[ip][2], tmp[ip][3]);
      }
    }
    if (prm.u_vec) {
      // 128-bit loads along the contiguous index (q: u_vec 1, k: u_vec 2); the host has checked
      // alignment and that a group of four never straddles a tap or the end of the tensor
#pragma unroll
      for (int j = 0; j < NU / 4; ++j) {
        const int f = j * NT + t;
        const int kl = prm.u_vec == 2 ? (f & 3) * 4 : (f >> 4);
        const int ql = prm.u_vec == 2 ? (f >> 2) : (f & 15) * 4;
        const int kglob = kb * BK + kl, qg = q0 + ql;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kglob < prm.K && qg < prm.Q && ql < BQE) {
          const uint32_t tap = fdiv((uint32_t)kglob, g.d_sc);
          const int kk = kglob - (int)tap * g.SC;
          const int tj = (int)fdiv(tap, g.d_kw);
          const int tp = prm.u_t0 + tj * prm.u_tj + ((int)tap - tj * g.KW) * prm.u_ti;
          const float* src = Ug + (long long)tp * prm.u_tap + (long long)kk * prm.u_sk + (long long)qg * prm.u_sq;
          if (AMSIM_IN(prm, BUF_U, src, float4)) val = __ldg(reinterpret_cast<const float4*>(src));
        }
        uraw[4 * j] = val.x; uraw[4 * j + 1] = val.y; uraw[4 * j + 2] = val.z; uraw[4 * j + 3] = val.w;
      }
    } else {
#pragma unroll
    for (int j = 0; j < NU; ++j) {
      const int e = j * NT + t;
      // lanes run along whichever index is contiguous in memory
      const int kl = u_kmajor ? (e & (BK - 1)) : (e >> 6);
      const int ql = u_kmajor ? (e >> 4) : (e & 63);
      const int kglob = kb * BK + kl, qg = q0 + ql;
      float val = 0.f;
      if (kglob < prm.K && qg < prm.Q && ql < BQE) {
        const uint32_t tap = fdiv((uint32_t)kglob, g.d_sc);
        const int kk = kglob - (int)tap * g.SC;
        const int tj = (int)fdiv(tap, g.d_kw);
        const int tp = prm.u_t0 + tj * prm.u_tj + ((int)tap - tj * g.KW) * prm.u_ti;
        const float* src = Ug + (long long)tp * prm.u_tap + (long long)kk * prm.u_sk + (long long)qg * prm.u_sq;
        if (AMSIM_IN(prm, BUF_U, src, float)) val = __ldg(src);
      }
      uraw[j] = val;
    }
    }
  };

  auto store_tile = [&](int buf) {
    uint32_t* vs = Vs + buf * BK * VS;
    uint32_t hz = 0;
    {
      const int krow = 4 * kg, flip = (kg >> 1) << 3;
#pragma unroll
      for (int ip = 0; ip < NPX; ++ip) {
        const float4 f = vraw[ip];
        const int col = pl[ip] ^ flip;
        vs[(krow + 0) * VS + col] = enc_v<EXACT, LM>(__float_as_uint(f.x), prm.m);
        vs[(krow + 1) * VS + col] = enc_v<EXACT, LM>(__float_as_uint(f.y), prm.m);
        vs[(krow + 2) * VS + col] = enc_v<EXACT, LM>(__float_as_uint(f.z), prm.m);
        vs[(krow + 3) * VS + col] = enc_v<EXACT, LM>(__float_as_uint(f.w), prm.m);
        if (HAZARD_CHECK)
          hz |= hazard_bits(__float_as_uint(f.x), false) | hazard_bits(__float_as_uint(f.y), false) |
                hazard_bits(__float_as_uint(f.z), false) | hazard_bits(__float_as_uint(f.w), false);
      }
    }
    if (prm.u_vec) {
#pragma unroll
      for (int j = 0; j < NU / 4; ++j) {
        const int f = j * NT + t;
        if (prm.u_vec == 2) {  // four reduction rows of one column
          uint32_t* dst = Us + buf * BK * US + (f & 3) * 4 * US + (f >> 2);
#pragma unroll
          for (int i = 0; i < 4; ++i) store_u<LM>(dst + i * US, __float_as_uint(uraw[4 * j + i]), prm.m);
        } else {               // four columns of one reduction row
          const float f4[4] = {uraw[4 * j], uraw[4 * j + 1], uraw[4 * j + 2], uraw[4 * j + 3]};
          store_u4<LM>(Us + buf * BK * US + (f >> 4) * US + (f & 15) * 4, f4, prm.m);
        }
      }
    } else {
#pragma unroll
    for (int j = 0; j < NU; ++j) {
      const int e = j * NT + t;
      const int kl = u_kmajor ? (e & (BK - 1)) : (e >> 6);
      const int ql = u_kmajor ? (e >> 4) : (e & 63);
      store_u<LM>(Us + buf * BK * US + kl * US + ql, __float_as_uint(uraw[j]), prm.m);
    }
    }
    if (HAZARD_CHECK) {
#pragma unroll
      for (int j = 0; j < NU; ++j) hz |= hazard_bits(__float_as_uint(uraw[j]), true);
    }
    if (HAZARD_CHECK) {
      hz = __reduce_or_sync(0xffffffffu, hz);
      if (lane == 0) Fs[buf * 4 * WP + w] = hz;
    }
  };

  float acc[TR][TC];
#pragma unroll
  for (int r = 0; r < TR; ++r)
#pragma unroll
    for (int c = 0; c < TC; ++c) acc[r][c] = 0.f;

  long long seg_at = run_at;  // balanced mode: run position where the segment being accumulated starts
  next_segment();
  if (kb_begin < nkb) load_tile(kb_begin);
  // the table is copied while the first stage's global loads are in flight
  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, NT);
  if (kb_begin < nkb) store_tile(0);
  __syncthreads();

  const int vcol = wp * 128 + 4 * lane;
  // broadcast from lane 0: tells the compiler the uniform operand's address is warp-uniform
  const int ucol = __shfl_sync(0xffffffffu, wq, 0) * TR;
  int buf = 0;
  for (;;) {  // segments of this CTA's run (one pass unless the launch is balanced)
  const int seg_end_kb = nkb;
  const bool more = BALANCED && run_at < run_end;
  for (int kb = kb_begin; kb < seg_end_kb; ++kb, buf ^= 1) {
    const bool last = kb + 1 == seg_end_kb;
    if (!last) {
      load_tile(kb + 1);
    } else if (more) {
      // the next segment's first stage is fetched under this segment's last stage, so that no
      // tile of the run starts with an exposed global-memory latency
      next_segment();
      load_tile(kb_begin);
    }
    const uint32_t* vs = Vs + buf * BK * VS;
    const uint32_t* us = Us + buf * BK * US + ucol;
    // k rows 8..15 sit at the column with bit 3 flipped (see the staging above)
#define AMSIM_K_HALVES(...)                                                   \
  _Pragma("unroll 1") for (int kh = 0; kh < BK; kh += 8) {                     \
    const uint32_t* vh = vs + kh * VS + (vcol ^ kh);                           \
    const uint32_t* uh = us + kh * US;                                         \
    AMSIM_UNROLL_K                                                             \
    for (int kk = 0; kk < 8; ++kk)                                             \
      mac_step<__VA_ARGS__>(acc, vh + kk * VS, uh + kk * US, lut_base, prm.rmask, prm.mult, prm.cmask, prm.cadj, \
                            prm.lut_raw);                                      \
  }
    static_assert(BK == 16, "two halves of eight reduction steps");
    if (HAZARD_CHECK) {
      uint32_t hz = 0;
#pragma unroll
      for (int i = 0; i < 4 * WP; ++i) hz |= Fs[buf * 4 * WP + i];
      if (hazard_free(hz) && !prm.exact_only) {
        AMSIM_K_HALVES(false, LM, true)
      } else {
        AMSIM_K_HALVES(true, LM)
      }
    } else if (QS > 1) {
AMSIM_UNROLL_K
      for (int kq = 0; kq < BK / QS; ++kq) {
        const int kk = kq * QS + ksub;
        mac_step<EXACT, LM>(acc, vs + kk * VS + (vcol ^ (kk & 8)), us + kk * US, lut_base, prm.rmask, prm.mult, prm.cmask,
                            prm.cadj, prm.lut_raw);
      }
    } else {
      AMSIM_K_HALVES(EXACT, LM)
    }
#undef AMSIM_K_HALVES
    if (!last || more) store_tile(buf ^ 1);
    __syncthreads();
  }

  // the tile just accumulated (the staging variables may already describe the next segment)
  int cur_p, cur_q, cur_z, cur_kb0, cur_kb1;
  if (BALANCED) {
    decode_tile(seg_at, cur_p, cur_q, cur_z, cur_kb0, cur_kb1);
    seg_at += cur_kb1 - cur_kb0;
  } else {
    cur_p = tile_p; cur_q = tile_q; cur_z = tile_z; cur_kb0 = kb_begin; cur_kb1 = nkb;
  }
  const int op0 = cur_p * BP, oq0 = cur_q * BQE;
  float* __restrict__ Og = prm.O + (long long)cur_z * prm.o_bs;

  // ---- warps that shared a column group: add their register tiles in warp order ----------
  if (QS > 1) {
    float* red = reinterpret_cast<float*>(smem);  // [QS - 1][TR*TC][32 * (4 / QS)], the operand tiles are dead now
    constexpr int GT = 32 * (4 / QS);             // threads per share
    const int gt = wq * 32 + lane;                // this thread's slot within its share
    if (ksub != 0) {
#pragma unroll
      for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int c = 0; c < TC; ++c) red[((ksub - 1) * TR * TC + r * TC + c) * GT + gt] = acc[r][c];
    }
    __syncthreads();
    if (ksub != 0) return;
    for (int src = 1; src < QS; ++src) {
#pragma unroll
      for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int c = 0; c < TC; ++c) acc[r][c] = __fadd_rn(acc[r][c], red[((src - 1) * TR * TC + r * TC + c) * GT + gt]);
    }
  }

  // ---- cluster reduction: ranks 1.. park their register tiles in their own shared
  // memory, rank 0 adds them in rank order through distributed shared memory ----------
  if (CLUSTER) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    float* red = reinterpret_cast<float*>(smem);  // [TR*TC][NT], the operand tiles are dead now
    if (krank != 0) {
#pragma unroll
      for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int c = 0; c < TC; ++c) red[(r * TC + c) * NT + t] = acc[r][c];
    }
    cluster.sync();
    if (krank == 0) {
      for (int src = 1; src < ksplit; ++src) {
        const float* remote = cluster.map_shared_rank(red, src);
#pragma unroll
        for (int r = 0; r < TR; ++r)
#pragma unroll
          for (int c = 0; c < TC; ++c) acc[r][c] = __fadd_rn(acc[r][c], remote[(r * TC + c) * NT + t]);
      }
    }
    cluster.sync();  // keep the senders' shared memory alive until it has been read
    if (krank != 0) return;
  }

  // ---- balanced mode: a tile whose reduction this CTA only shares parks its register tile in
  // the workspace (slot 0: the run started inside the tile, slot 1: it started the tile) and
  // counts itself in; the CTA that completes the count adds all parked tiles of the tile in
  // CTA order (whoever it is, the order is the same) and writes the output.  Nobody waits.
  if (BALANCED && (cur_kb0 != 0 || cur_kb1 != nkb_all)) {
    float* slot = prm.ws + ((long long)blockIdx.x * 2 + (cur_kb0 == 0 ? 1 : 0)) * (TR * TC * NT);
#pragma unroll
    for (int r = 0; r < TR; ++r)
#pragma unroll
      for (int c = 0; c < TC; ++c)
        if (AMSIM_IN(prm, BUF_WS, slot + (r * TC + c) * NT + t, float)) __stcg(slot + (r * TC + c) * NT + t, acc[r][c]);
    __threadfence();  // this thread's part of the tile is visible device-wide before the count
    __syncthreads();
    const long long tile = ((long long)cur_z * prm.sk_ptiles + cur_p) * prm.sk_qtiles + cur_q;
    const long long first = tile * nkb_all, last = first + nkb_all;
    long long c0 = first * prm.sk_grid / prm.sk_iters;   // CTA whose run holds the tile's first block
    while (c0 > 0 && balanced_begin(c0, prm.sk_iters, prm.sk_grid) > first) --c0;
    while (balanced_begin(c0 + 1, prm.sk_iters, prm.sk_grid) <= first) ++c0;
    long long c1 = (last - 1) * prm.sk_grid / prm.sk_iters;  // ... and its last block
    while (c1 > 0 && balanced_begin(c1, prm.sk_iters, prm.sk_grid) > last - 1) --c1;
    while (balanced_begin(c1 + 1, prm.sk_iters, prm.sk_grid) <= last - 1) ++c1;
    if (t == 0) {
      const int arrived = AMSIM_IN(prm, BUF_WS, prm.sk_count + tile, int) ? atomicAdd(prm.sk_count + tile, 1) : 0;
      *flag_s = arrived == (int)(c1 - c0);  // c1 - c0 + 1 sharers
      // the last sharer leaves the counter at zero for the next launch that uses this buffer
      if (arrived == (int)(c1 - c0) && AMSIM_IN(prm, BUF_WS, prm.sk_count + tile, int)) prm.sk_count[tile] = 0;
    }
    __syncthreads();
    const bool completes = *flag_s != 0;
    __syncthreads();  // flag_s may be rewritten by the next segment
    if (completes) {
      __threadfence();
#pragma unroll
      for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int c = 0; c < TC; ++c) acc[r][c] = 0.f;
      for (long long cta = c0; cta <= c1; ++cta) {
        const long long b = balanced_begin(cta, prm.sk_iters, prm.sk_grid);
        const float* src = prm.ws + (cta * 2 + (b <= first ? 1 : 0)) * (TR * TC * NT);
#pragma unroll
        for (int r = 0; r < TR; ++r)
#pragma unroll
          for (int c = 0; c < TC; ++c)
            if (AMSIM_IN(prm, BUF_WS, src + (r * TC + c) * NT + t, float)) acc[r][c] = __fadd_rn(acc[r][c], __ldcg(src + (r * TC + c) * NT + t));
      }
      store_out_tile(prm, acc, Og, op0 + vcol, oq0 + ucol);
    }
  } else {
    store_out_tile(prm, acc, Og, op0 + vcol, oq0 + ucol);
  }
  if (!more) break;
#pragma unroll
  for (int r = 0; r < TR; ++r)
#pragma unroll
    for (int c = 0; c < TC; ++c) acc[r][c] = 0.f;
  }
}

// -----------------------------------------------------------------------------
// fgrad_gemm: p = (tap, channel) gathered along p, q = output channel, the
// reduction index k runs over grid positions (n, oh, ow).
// grid = (ceil(P/BP), ceil(Q/64), splits); split s reduces
// k in [s * k_chunk, min((s+1) * k_chunk, K)) and writes ws[s] (or O if there
// is only one split).
// -----------------------------------------------------------------------------
template <int WP, bool EXACT, bool VEC, int LM>
__global__ void __launch_bounds__(WP * 128, WP == 1 ? AMSIM_CTAS1 : 2) fgrad_gemm(const Params prm) {
  using L = SmemLayout<WP>;
  constexpr int NT = L::NT, BP = L::BP, VS = L::VS;
  constexpr int NU = BK * BQ / NT;
  constexpr int GPR = BP / 4;        // 4-wide p groups per k row
  constexpr int RPP = NT / GPR;      // k rows covered per pass (= 4)
  constexpr int NV = BK / RPP;       // passes (= 4)

  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* Vs = reinterpret_cast<uint32_t*>(smem);
  uint32_t* Us = Vs + L::V_WORDS;
  uint32_t* Fs = Us + L::U_WORDS;  // per stage and warp: hazard bits of the staged operands
  constexpr bool HAZARD_CHECK = EXACT && !lm_direct(LM);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t lut_base = (smem_base + L::TILE_BYTES + prm.lut_align - 1) & ~(prm.lut_align - 1);
  uint8_t* lut_s = smem + (lut_base - smem_base);

  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int wp = w % WP, wq = w / WP;
  const int p0 = blockIdx.x * BP, q0 = blockIdx.y * BQ;
  const int kbeg = blockIdx.z * prm.k_chunk;
  const int kend = min(kbeg + prm.k_chunk, prm.K);
  const Gather& g = prm.g;
  const float* __restrict__ Vg = prm.V;
  const float* __restrict__ Ug = prm.U;


  // ---- this thread's 4 consecutive p (same for every k row it stages) ---------
  const int pl = 4 * (t % GPR);
  const int krow0 = t / GPR;
  int kh[4], kw[4], ch[4];
  bool pv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t pg = (uint32_t)(p0 + pl + j);
    pv[j] = pg < (uint32_t)prm.P;
    const uint32_t tap = fdiv(pg, g.d_sc);
    ch[j] = (int)(pg - tap * (uint32_t)g.SC);
    kh[j] = (int)fdiv(tap, g.d_kw);
    kw[j] = (int)tap - kh[j] * g.KW;
  }

  float4 vraw[NV];
  float uraw[NU];

  auto load_tile = [&](int kb) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int pix = kbeg + kb * BK + i * RPP + krow0;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (pix < kend) {
        const uint32_t n = fdiv((uint32_t)pix, g.d_img);
        const uint32_t rem = (uint32_t)pix - n * (uint32_t)(g.PH * g.PW);
        const uint32_t a = fdiv(rem, g.d_pw);
        const uint32_t b = rem - a * (uint32_t)g.PW;
        const int r0 = (int)a * g.ps_h - g.off_t, c0 = (int)b * g.ps_w - g.off_l;
        const float* src = Vg + (long long)n * ((long long)g.SH * g.SW * g.SC);
        if (VEC) {
          const int u = r0 + kh[0], v = c0 + kw[0];
          if (pv[0] && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w &&
              AMSIM_IN(prm, BUF_V, src + ((long long)(u * g.SW + v) * g.SC + ch[0]), float4))
            val = __ldg(reinterpret_cast<const float4*>(src + ((long long)(u * g.SW + v) * g.SC + ch[0])));
        } else {
          float tmp[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int u = r0 + kh[j], v = c0 + kw[j];
            tmp[j] = 0.f;
            if (pv[j] && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w &&
                AMSIM_IN(prm, BUF_V, src + ((long long)(u * g.SW + v) * g.SC + ch[j]), float))
              tmp[j] = __ldg(src + ((long long)(u * g.SW + v) * g.SC + ch[j]));
          }
          val = make_float4(tmp[0], tmp[1], tmp[2], tmp[3]);
        }
      }
      vraw[i] = val;
    }
    if (prm.u_vec) {  // q contiguous, rows and base 16-byte aligned, Q a multiple of 4 (checked by the host)
#pragma unroll
      for (int j = 0; j < NU / 4; ++j) {
        const int f = j * NT + t;
        const int pix = kbeg + kb * BK + (f >> 4), qg = q0 + (f & 15) * 4;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (pix < kend && qg < prm.Q && AMSIM_IN(prm, BUF_U, Ug + (long long)pix * prm.u_sk + qg, float4))
          val = __ldg(reinterpret_cast<const float4*>(Ug + (long long)pix * prm.u_sk + qg));
        uraw[4 * j] = val.x; uraw[4 * j + 1] = val.y; uraw[4 * j + 2] = val.z; uraw[4 * j + 3] = val.w;
      }
    } else {
#pragma unroll
    for (int j = 0; j < NU; ++j) {
      const int e = j * NT + t;
      const int pix = kbeg + kb * BK + (e >> 6), qg = q0 + (e & 63);
      const float* src = Ug + (long long)pix * prm.u_sk + (long long)qg * prm.u_sq;
      uraw[j] = (pix < kend && qg < prm.Q && AMSIM_IN(prm, BUF_U, src, float)) ? __ldg(src) : 0.f;
    }
    }
  };

  auto store_tile = [&](int buf) {
    uint32_t* vs = Vs + buf * BK * VS;
    uint32_t hz = 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float4 f = vraw[i];
      uint4 wv;
      wv.x = enc_v<EXACT, LM>(__float_as_uint(f.x), prm.m);
      wv.y = enc_v<EXACT, LM>(__float_as_uint(f.y), prm.m);
      wv.z = enc_v<EXACT, LM>(__float_as_uint(f.z), prm.m);
      wv.w = enc_v<EXACT, LM>(__float_as_uint(f.w), prm.m);
      *reinterpret_cast<uint4*>(vs + (i * RPP + krow0) * VS + pl) = wv;
      if (HAZARD_CHECK)
        hz |= hazard_bits(__float_as_uint(f.x), false) | hazard_bits(__float_as_uint(f.y), false) |
              hazard_bits(__float_as_uint(f.z), false) | hazard_bits(__float_as_uint(f.w), false);
    }
    if (prm.u_vec) {
#pragma unroll
      for (int j = 0; j < NU / 4; ++j) {
        const int f = j * NT + t;
        const float f4[4] = {uraw[4 * j], uraw[4 * j + 1], uraw[4 * j + 2], uraw[4 * j + 3]};
        store_u4<LM>(Us + buf * BK * US + (f >> 4) * US + (f & 15) * 4, f4, prm.m);
      }
    } else {
#pragma unroll
    for (int j = 0; j < NU; ++j) {
      const int e = j * NT + t;
      store_u<LM>(Us + buf * BK * US + (e >> 6) * US + (e & 63), __float_as_uint(uraw[j]), prm.m);
    }
    }
    if (HAZARD_CHECK) {
#pragma unroll
      for (int j = 0; j < NU; ++j) hz |= hazard_bits(__float_as_uint(uraw[j]), true);
    }
    if (HAZARD_CHECK) {
      hz = __reduce_or_sync(0xffffffffu, hz);
      if (lane == 0) Fs[buf * 4 * WP + w] = hz;
    }
  };

  float acc[TR][TC];
#pragma unroll
  for (int r = 0; r < TR; ++r)
#pragma unroll
    for (int c = 0; c < TC; ++c) acc[r][c] = 0.f;

  const int nkb = (kend - kbeg + BK - 1) / BK;
  const int vcol = wp * 128 + 4 * lane;
  const int ucol = wq * TR;
  if (nkb > 0) load_tile(0);
  // the table is copied while the first stage's global loads are in flight
  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, NT);
  if (nkb > 0) store_tile(0);
  __syncthreads();
  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nkb) load_tile(kb + 1);
    const uint32_t* vs = Vs + buf * BK * VS + vcol;
    const uint32_t* us = Us + buf * BK * US + ucol;
    if (HAZARD_CHECK) {
      uint32_t hz = 0;
#pragma unroll
      for (int i = 0; i < 4 * WP; ++i) hz |= Fs[buf * 4 * WP + i];
      if (hazard_free(hz) && !prm.exact_only) {
AMSIM_UNROLL_K
        for (int kk = 0; kk < BK; ++kk)
          mac_step<false, LM, true>(acc, vs + kk * VS, us + kk * US, lut_base, prm.rmask, prm.mult, prm.cmask,
                                    prm.cadj, prm.lut_raw);
      } else {
AMSIM_UNROLL_K
        for (int kk = 0; kk < BK; ++kk)
          mac_step<true, LM>(acc, vs + kk * VS, us + kk * US, lut_base, prm.rmask, prm.mult, prm.cmask, prm.cadj,
                             prm.lut_raw);
      }
    } else {
AMSIM_UNROLL_K
      for (int kk = 0; kk < BK; ++kk)
        mac_step<EXACT, LM>(acc, vs + kk * VS, us + kk * US, lut_base, prm.rmask, prm.mult, prm.cmask, prm.cadj,
                            prm.lut_raw);
    }
    if (kb + 1 < nkb) store_tile(buf ^ 1);
    __syncthreads();
  }

  // partial sums go to ws[split][P][Q]; a single split writes Out[p * o_sp + q * o_sq] itself
  const bool to_ws = prm.splits > 1;
  float* __restrict__ Og = to_ws ? prm.ws + (long long)blockIdx.z * ((long long)prm.P * prm.Q) : prm.O;
  const long long sp = to_ws ? prm.Q : prm.o_sp, sq = to_ws ? 1 : prm.o_sq;
  const bool vec_out = sq == 1 && (sp & 3) == 0 && ((reinterpret_cast<uintptr_t>(Og) & 15) == 0);
#pragma unroll
  for (int c = 0; c < TC; ++c) {
    const int pg = p0 + vcol + c;
    if (pg >= prm.P) continue;
    float* orow = Og + (long long)pg * sp;
#pragma unroll
    for (int g4 = 0; g4 < TR / 4; ++g4) {
      const int qg = q0 + ucol + 4 * g4;
      if (vec_out && qg + 3 < prm.Q) {
        if (AMSIM_IN(prm, to_ws ? BUF_WS : BUF_O, orow + qg, float4))
          *reinterpret_cast<float4*>(orow + qg) =
              make_float4(acc[4 * g4][c], acc[4 * g4 + 1][c], acc[4 * g4 + 2][c], acc[4 * g4 + 3][c]);
      } else {
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if (qg + r < prm.Q && AMSIM_IN(prm, to_ws ? BUF_WS : BUF_O, orow + (long long)(qg + r) * sq, float))
            orow[(long long)(qg + r) * sq] = acc[4 * g4 + r][c];
      }
    }
  }
}

// -----------------------------------------------------------------------------
// fgrad_exact_thin: deterministic filter / weight gradient when the output is small.
// Every output is one serial FP32 chain over the whole reduction (the reference's order),
// so the only parallelism is the number of outputs: with 64 chains per thread (fgrad_gemm)
// a 576 x 64 gradient occupies five CTAs.  Here a thread owns TQ chains (one p, TQ
// consecutive q), a CTA of NW warps covers 32 p x NW*TQ q.  grid = (ceil(P/32), ceil(Q/(NW*TQ))).
// -----------------------------------------------------------------------------
constexpr int THIN_BK = 16;

// FLUSH: fast mode (an operand with exponent field 0 gives a zero product, as in the tiled fast kernels).
template <int TQ, int NW, int LM, bool FLUSH>
__global__ void __launch_bounds__(32 * NW) fgrad_exact_thin(const Params prm) {
  constexpr int NT = 32 * NW, BPT = 32, BQT = NW * TQ;  // NW warps share one staged V tile
  constexpr int BK = THIN_BK;
  constexpr int NV = BK / NW;                     // V rows staged per thread
  constexpr int NUQ = (BK * BQT + NT - 1) / NT;   // U elements staged per thread
  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* Vs = reinterpret_cast<uint32_t*>(smem);  // [2][BK][32]
  uint32_t* Us = Vs + 2 * BK * BPT;                  // [2][BK][BQT]
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t lut_base = (smem_base + prm.tile_bytes + prm.lut_align - 1) & ~(prm.lut_align - 1);
  uint8_t* lut_s = smem + (lut_base - smem_base);

  const int t = threadIdx.x, lane = t & 31;
  const int w = __shfl_sync(0xffffffffu, t >> 5, 0);
  const int p0 = blockIdx.x * BPT, q0 = blockIdx.y * BQT;
  const Gather& g = prm.g;
  // this CTA's slice of the reduction (the whole of it unless fast mode asked for splits)
  const int kbeg = blockIdx.z * prm.k_chunk;
  const int kend = min(kbeg + prm.k_chunk, prm.K);
  const float* __restrict__ Vg = prm.V;
  const float* __restrict__ Ug = prm.U;
  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, NT);

  const uint32_t pg = (uint32_t)(p0 + lane);
  const bool pv = pg < (uint32_t)prm.P;
  const uint32_t tap = fdiv(pg, g.d_sc);
  const int ch = (int)(pg - tap * (uint32_t)g.SC);
  const int kh = (int)fdiv(tap, g.d_kw);
  const int kw = (int)tap - kh * g.KW;

  float vraw[NV], uraw[NUQ];
  auto load_tile = [&](int kb) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int pix = kbeg + kb * BK + w + NW * i;
      float val = 0.f;
      if (pv && pix < kend) {
        const uint32_t n = fdiv((uint32_t)pix, g.d_img);
        const uint32_t rem = (uint32_t)pix - n * (uint32_t)(g.PH * g.PW);
        const uint32_t a = fdiv(rem, g.d_pw);
        const uint32_t b = rem - a * (uint32_t)g.PW;
        const int u = (int)a * g.ps_h - g.off_t + kh, v = (int)b * g.ps_w - g.off_l + kw;
        const float* src = Vg + (long long)n * ((long long)g.SH * g.SW * g.SC) + ((long long)(u * g.SW + v) * g.SC + ch);
        if ((unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w && AMSIM_IN(prm, BUF_V, src, float)) val = __ldg(src);
      }
      vraw[i] = val;
    }
#pragma unroll
    for (int j = 0; j < NUQ; ++j) {
      const int e = j * NT + t;
      const int pix = kbeg + kb * BK + e / BQT, qg = q0 + e % BQT;
      const float* src = Ug + (long long)pix * prm.u_sk + (long long)qg * prm.u_sq;
      uraw[j] = (e < BK * BQT && pix < kend && qg < prm.Q && AMSIM_IN(prm, BUF_U, src, float)) ? __ldg(src) : 0.f;
    }
  };
  auto store_tile = [&](int buf) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      Vs[(buf * BK + w + NW * i) * BPT + lane] = enc_v<true, LM>(__float_as_uint(vraw[i]), prm.m);
#pragma unroll
    for (int j = 0; j < NUQ; ++j) {
      const int e = j * NT + t;
      if (e < BK * BQT) Us[(buf * BK + e / BQT) * BQT + e % BQT] = enc_u<LM>(__float_as_uint(uraw[j]), prm.m);
    }
  };

  float acc[TQ];
#pragma unroll
  for (int r = 0; r < TQ; ++r) acc[r] = 0.f;
  const int nkb = (kend - kbeg + BK - 1) / BK;
  if (nkb > 0) {
    load_tile(0);
    store_tile(0);
  }
  __syncthreads();
  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nkb) load_tile(kb + 1);
    const uint32_t* vs = Vs + buf * BK * BPT + lane;
    const uint32_t* us = Us + buf * BK * BQT + w * TQ;
#pragma unroll 16
    for (int kk = 0; kk < BK; ++kk) {
      const uint32_t wv = vs[kk * BPT];
      // same arithmetic as the deterministic branch of mac_step
      const uint32_t ci = lm_global(LM) ? (wv & prm.cmask) : ((wv & 0xFFu) | lut_base);
      const uint32_t cs = (LM == LM_ADD ? wv : (wv & 0xFF800000u)) - 0x3F800000u;
      // fast mode treats zero / denormal operands as exact zeros (as the tiled fast kernels do): an
      // unreachable threshold switches the lane operand's products off
      const int cn = (FLUSH && !(wv & 0x7F800000u)) ? 0x7FFFFFFF : (int)(0x3F800000u - (wv & 0x7F800000u));
#pragma unroll
      for (int r = 0; r < TQ; ++r) {
        const uint32_t uu = us[kk * BQT + r];
        if (lm_direct(LM)) {
          acc[r] = __fadd_rn(acc[r], __uint_as_float(direct_mul_bits<LM == LM_DIRECT_MBM>(wv, uu)));
          continue;
        }
        const uint32_t pp = uu & 0xFF800000u;
        const int ee = (int)(uu & 0x7F800000u);
        uint32_t e;
        if (LM == LM_ADD) {
          e = uu & 0x007FFFFFu;
        } else if (lm_global(LM)) {
          e = global_entry<LM>(prm.lut_raw, (uu & prm.rmask) | ci, prm.mult, prm.cadj);
        } else {
          e = lds_u8((uu & prm.rmask) | ci) * prm.mult;
        }
        if (ee > cn && !(FLUSH && ee == 0)) acc[r] = __fadd_rn(acc[r], __uint_as_float(e + (pp + cs)));
      }
    }
    if (kb + 1 < nkb) store_tile(buf ^ 1);
    __syncthreads();
  }
  if (pv) {
#pragma unroll
    for (int r = 0; r < TQ; ++r) {
      const int qg = q0 + w * TQ + r;
      if (qg < prm.Q) {
        float* dst = prm.splits > 1 ? prm.ws + (((long long)blockIdx.z * prm.P + pg) * prm.Q + qg)
                                    : prm.O + ((long long)pg * prm.o_sp + (long long)qg * prm.o_sq);
        if (AMSIM_IN(prm, prm.splits > 1 ? BUF_WS : BUF_O, dst, float)) *dst = acc[r];
      }
    }
  }
}

// -----------------------------------------------------------------------------
// fgrad_exact_chain: deterministic filter / weight gradient for outputs with few chains and a
// long reduction (576 x 64 outputs over 200 704 pixels: 1152 warps' worth of chains).  The
// chains have to be added in order, but their products do not have to be computed in order:
// per 16-step stage 16 producer warps compute the stage's 16 x 8 x 32 products in parallel (warp w:
// reduction step w for all 8 columns, lane = row; the table row is warp-uniform as everywhere)
// into shared memory, and 8 consumer warps (warp = column, lane = row) add their own chain's 16
// products in ascending order while the producers work on the next stage.  A product the reference returns as 0
// is stored as +0.0, whose addition changes nothing (the accumulator is never -0.0).
// CTA tile: 32 rows x 8 columns, 768 threads.  grid = (ceil(P/32), ceil(Q/8)).
// -----------------------------------------------------------------------------
constexpr int CHAIN_Q = 8;

template <int LM>
__global__ void __launch_bounds__(768) fgrad_exact_chain(const Params prm) {
  // warps 0..15 produce (stage operands, compute one reduction step's products each), warps 16..23
  // consume (add their chains' products), so the additions of one stage overlap the products of the next
  constexpr int NT = 768, BPT = 32, BQT = CHAIN_Q, NPROD = 16;
  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* Vs = reinterpret_cast<uint32_t*>(smem);  // [2][BK][32]
  uint32_t* Us = Vs + 2 * BK * BPT;                  // [2][BK][8]
  float* Ps = reinterpret_cast<float*>(Us + 2 * BK * BQT);  // [2][BK][8][32] products of two stages
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t lut_base = (smem_base + prm.tile_bytes + prm.lut_align - 1) & ~(prm.lut_align - 1);
  uint8_t* lut_s = smem + (lut_base - smem_base);

  const int t = threadIdx.x, lane = t & 31;
  const int w = __shfl_sync(0xffffffffu, t >> 5, 0);
  const int p0 = blockIdx.x * BPT, q0 = blockIdx.y * BQT;
  const Gather& g = prm.g;
  const float* __restrict__ Vg = prm.V;
  const float* __restrict__ Ug = prm.U;
  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, NT);

  const uint32_t pg = (uint32_t)(p0 + lane);
  const bool pv = pg < (uint32_t)prm.P;
  const uint32_t tap = fdiv(pg, g.d_sc);
  const int ch = (int)(pg - tap * (uint32_t)g.SC);
  const int kh = (int)fdiv(tap, g.d_kw);
  const int kw = (int)tap - kh * g.KW;

  // Little arithmetic per staged element, so the global loads run PF stages ahead of their use:
  // register slots vq[slot], uq[slot], filled PF iterations before they are stored to shared memory.
  constexpr int PF = 4;
  float vq[PF][1], uq[PF];
  auto load_tile = [&](int kb, float (&vraw)[1], float& uraw) {
    {
      const int pix = kb * BK + w;
      float val = 0.f;
      if (pv && pix < prm.K) {
        const uint32_t n = fdiv((uint32_t)pix, g.d_img);
        const uint32_t rem = (uint32_t)pix - n * (uint32_t)(g.PH * g.PW);
        const uint32_t a = fdiv(rem, g.d_pw);
        const uint32_t b = rem - a * (uint32_t)g.PW;
        const int u = (int)a * g.ps_h - g.off_t + kh, v = (int)b * g.ps_w - g.off_l + kw;
        const float* src = Vg + (long long)n * ((long long)g.SH * g.SW * g.SC) + ((long long)(u * g.SW + v) * g.SC + ch);
        if ((unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w && AMSIM_IN(prm, BUF_V, src, float)) val = __ldg(src);
      }
      vraw[0] = val;
    }
    uraw = 0.f;
    if (t < BK * BQT) {
      const int pix = kb * BK + (t >> 3), qg = q0 + (t & 7);
      const float* src = Ug + (long long)pix * prm.u_sk + (long long)qg * prm.u_sq;
      if (pix < prm.K && qg < prm.Q && AMSIM_IN(prm, BUF_U, src, float)) uraw = __ldg(src);
    }
  };
  auto store_tile = [&](int buf, const float (&vraw)[1], float uraw) {
    Vs[(buf * BK + w) * BPT + lane] = enc_v<true, LM>(__float_as_uint(vraw[0]), prm.m);
    if (t < BK * BQT) Us[(buf * BK + (t >> 3)) * BQT + (t & 7)] = enc_u<LM>(__float_as_uint(uraw), prm.m);
  };

  float acc = 0.f;
  const int nkb = (prm.K + BK - 1) / BK;
  const bool producer = w < NPROD;
  const int wc = w - NPROD;  // consumer warp = column
  if (producer) {
#pragma unroll
    for (int j = 0; j < PF; ++j) load_tile(j, vq[j], uq[j]);  // tiles past the end load zeros
    store_tile(0, vq[0], uq[0]);
  }
  __syncthreads();
  for (int kb0 = 0; kb0 < nkb; kb0 += PF) {
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      const int kb = kb0 + j;
      if (kb >= nkb) break;
      const int buf = j & 1;                         // PF is even, so kb & 1 == j & 1
      // ---- products of this stage: producer warp w takes reduction step w ---------------------
      if (producer) {
        load_tile(kb + PF, vq[j], uq[j]);            // slot j is free: tile kb already sits in shared memory
        const int kk = w;
        const uint32_t wv = Vs[(buf * BK + kk) * BPT + lane];
        const uint32_t ci = lm_global(LM) ? (wv & prm.cmask) : ((wv & 0xFFu) | lut_base);
        const uint32_t cs = (LM == LM_ADD ? wv : (wv & 0xFF800000u)) - 0x3F800000u;
        const int cn = (int)(0x3F800000u - (wv & 0x7F800000u));
        const uint4 ua = *reinterpret_cast<const uint4*>(Us + (buf * BK + kk) * BQT);
        const uint4 ub = *reinterpret_cast<const uint4*>(Us + (buf * BK + kk) * BQT + 4);
        const uint32_t uq8[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
#pragma unroll
        for (int r = 0; r < BQT; ++r) {
          const uint32_t uu = uq8[r];
          uint32_t bits;
          if (lm_direct(LM)) {
            bits = direct_mul_bits<LM == LM_DIRECT_MBM>(wv, uu);
          } else {
            const uint32_t pp = uu & 0xFF800000u;
            const int ee = (int)(uu & 0x7F800000u);
            uint32_t e;
            if (LM == LM_ADD) {
              e = uu & 0x007FFFFFu;
            } else if (lm_global(LM)) {
              e = global_entry<LM>(prm.lut_raw, (uu & prm.rmask) | ci, prm.mult, prm.cadj);
            } else {
              e = lds_u8((uu & prm.rmask) | ci) * prm.mult;
            }
            bits = ee > cn ? e + (pp + cs) : 0u;  // AMsimulator.inl:28: exponent sum <= 127 gives +0
          }
          Ps[((buf * BK + kk) * BQT + r) * BPT + lane] = __uint_as_float(bits);
        }
        // next stage's operands (loaded PF - 1 stages ago) go to the other buffer, last read before the
        // previous barrier
        store_tile(buf ^ 1, vq[(j + 1) % PF], uq[(j + 1) % PF]);
      }
      // one barrier per stage; the products buffer alternates, so the producers' next stage does not
      // disturb the consumers' additions of this one
      __syncthreads();
      // ---- consumers: every thread adds its own chain's products in ascending order -------------
      if (!producer) {
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) acc = __fadd_rn(acc, Ps[((buf * BK + kk) * BQT + wc) * BPT + lane]);
      }
    }
  }
  const int qg = q0 + wc;
  if (!producer && pv && qg < prm.Q && AMSIM_IN(prm, BUF_O, prm.O + ((long long)pg * prm.o_sp + (long long)qg * prm.o_sq), float))
    prm.O[(long long)pg * prm.o_sp + (long long)qg * prm.o_sq] = acc;
}

// Sums the split-K partials in a fixed order (the result does not depend on scheduling).
// Partials are [split][n]; the sum of element i goes to out[(i / Q) * o_sp + (i % Q) * o_sq].
// `lanes` threads share one element: lane l adds the consecutive splits [l * per, (l + 1) * per)
// in ascending order, lane 0 then adds the lanes' sums in ascending order through shared memory
// (with hundreds of splits one thread per element is a chain of dependent loads: 45 us for 591
// partials of a bias gradient, 5 us with 32 lanes).  lanes = 1 is the plain ascending sum.
// Block of 256 threads = lanes x (256 / lanes) consecutive elements.
__global__ void __launch_bounds__(256) reduce_splits(const float* __restrict__ ws, float* __restrict__ out, long long n,
                                                     int splits, int Q, long long o_sp, long long o_sq, int lanes) {
  __shared__ float red[256];
  const int epb = 256 / lanes;
  const int l = threadIdx.x / epb, e = threadIdx.x - l * epb;
  const long long i = (long long)blockIdx.x * epb + e;
  const int per = (splits + lanes - 1) / lanes;
  const int k0 = l * per, k1 = min(splits, k0 + per);
  float s = 0.f;
  if (i < n && k0 < k1) {
    s = ws[(long long)k0 * n + i];
    for (int k = k0 + 1; k < k1; ++k) s = __fadd_rn(s, ws[(long long)k * n + i]);
  }
  if (lanes > 1) {
    red[threadIdx.x] = s;
    __syncthreads();
    if (l == 0) {
      for (int j = 1; j < lanes && j * per < splits; ++j) s = __fadd_rn(s, red[j * epb + e]);  // empty lanes are skipped
    }
  }
  if (l != 0 || i >= n) return;
  const long long p = i / Q, q = i - p * Q;
  out[p * o_sp + q * o_sq] = s;
}

// Lanes per element for reduce_splits: the smallest power of two that leaves at most 16 splits per lane.
inline int reduce_lanes(int splits) {
  int lanes = 1;
  while (lanes < 32 && (splits + lanes - 1) / lanes > 16) lanes <<= 1;
  return lanes;
}
inline unsigned reduce_blocks(long long n, int lanes) { return (unsigned)((n + (256 / lanes) - 1) / (256 / lanes)); }

// -----------------------------------------------------------------------------
// column_sums: part[chunk][c] = sum over the chunk's rows of g[row][c], exact FP32 adds.
// The bias gradient of a layer (sum of the output gradient over every pixel / sample) - an exact
// op that sits between the AM ops of a training step and is bound by one read of the gradient
// from HBM.  grid = (chunks, ceil(col groups / CG)); a block of 256 threads covers CG column
// groups (VEC: 4 columns each, 128-bit loads) x 256 / CG rows per pass; every thread adds the rows
// it visits in ascending order, the block's threads of one column group are then added in thread
// order through shared memory, and reduce_splits adds the chunks in ascending order: the result
// does not depend on scheduling.
// -----------------------------------------------------------------------------
template <bool VEC>
__global__ void __launch_bounds__(256) column_sums(const float* __restrict__ g, float* __restrict__ part, long long rows,
                                                   int cols, long long rows_per_chunk, int CG) {
  constexpr int W = VEC ? 4 : 1;
  __shared__ float red[256 * W];
  const int groups = (cols + W - 1) / W;
  const int cg = threadIdx.x % CG, rl = threadIdx.x / CG, RL = 256 / CG;
  const int grp = blockIdx.y * CG + cg;
  const long long r0 = (long long)blockIdx.x * rows_per_chunk;
  const long long r1 = min(rows, r0 + rows_per_chunk);
  float acc[W];
#pragma unroll
  for (int i = 0; i < W; ++i) acc[i] = 0.f;
  if (grp < groups) {
    for (long long r = r0 + rl; r < r1; r += RL) {
      if (VEC) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(g + r * cols) + grp);
        acc[0] = __fadd_rn(acc[0], v.x); acc[1 % W] = __fadd_rn(acc[1 % W], v.y);
        acc[2 % W] = __fadd_rn(acc[2 % W], v.z); acc[3 % W] = __fadd_rn(acc[3 % W], v.w);
      } else {
        acc[0] = __fadd_rn(acc[0], __ldg(g + r * cols + grp));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < W; ++i) red[(rl * CG + cg) * W + i] = acc[i];
  __syncthreads();
  if (rl == 0 && grp < groups) {
    for (int j = 1; j < RL; ++j)
#pragma unroll
      for (int i = 0; i < W; ++i) acc[i] = __fadd_rn(acc[i], red[(j * CG + cg) * W + i]);
#pragma unroll
    for (int i = 0; i < W; ++i)
      if (grp * W + i < cols) part[(long long)blockIdx.x * cols + grp * W + i] = acc[i];
  }
}

// The reference primitive on raw LUT bytes (cuda/AMsimulator.inl:13-36).
// `wide`: 16-bit entries (carry << 15 | top 15 mantissa bits of the product), a format extension.
__device__ __forceinline__ uint32_t am_mul_bits(uint32_t at, uint32_t bt, const uint8_t* __restrict__ lut, int m,
                                                bool wide = false) {
  const uint32_t mask = ((1u << m) - 1u) << (23 - m);
  const uint32_t idx = ((at & mask) >> (23 - 2 * m)) | ((bt & mask) >> (23 - m));
  const uint32_t e = ((at >> 23) & 0xFFu) + ((bt >> 23) & 0xFFu);
  if (e <= 127u) return 0u;
  if (wide) {
    const uint32_t v = __ldg(reinterpret_cast<const uint16_t*>(lut) + idx);
    return ((at ^ bt) & 0x80000000u) + ((e - 127u + (v >> 15)) << 23) + ((v & 0x7FFFu) << 8);
  }
  const uint32_t v = __ldg(lut + idx);
  return ((at ^ bt) & 0x80000000u) + ((e - 127u + (v >> 7)) << 23) + ((v & 0x7Fu) << (23 - m));
}

// ---- T = int32 ------------------------------------------------------------------
// The reference also instantiates its kernels for int32 (cuda/gemm.cu:64-67,
// cuda/denseam_kernel.cu:146-151): operands are converted to float for the
// multiplier and the accumulator is updated as acc = (int)((float)acc + product)
// at every step.  Kept for interface completeness: one thread per output, raw
// table in global memory, no tiling.  Same index maps as the FP32 kernels.
__device__ __forceinline__ int step_i32(int acc, int a, int b, bool a_first, const uint8_t* __restrict__ lut, int m) {
  const uint32_t at = __float_as_uint(__int2float_rn(a_first ? a : b));
  const uint32_t bt = __float_as_uint(__int2float_rn(a_first ? b : a));
  return __float2int_rz(__fadd_rn(__int2float_rn(acc), __uint_as_float(am_mul_bits(at, bt, lut, m))));
}

__global__ void naive_gather_i32(const Params prm) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)prm.P * prm.Q) return;
  const Gather& g = prm.g;
  const int* __restrict__ V = reinterpret_cast<const int*>(prm.V);
  const int* __restrict__ U = reinterpret_cast<const int*>(prm.U);
  const uint32_t p = (uint32_t)(idx / prm.Q);
  const int q = (int)(idx - (long long)p * prm.Q);
  const uint32_t n = fdiv(p, g.d_img);
  const uint32_t rem = p - n * (uint32_t)(g.PH * g.PW);
  const uint32_t a = fdiv(rem, g.d_pw), b = rem - a * (uint32_t)g.PW;
  const int r0 = (int)a * g.ps_h - g.off_t, c0 = (int)b * g.ps_w - g.off_l;
  const long long nb = (long long)n * ((long long)g.SH * g.SW * g.SC);
  int acc = 0;
  for (int k = 0; k < prm.K; ++k) {
    const uint32_t tap = fdiv((uint32_t)k, g.d_sc);
    const int ch = k - (int)tap * g.SC;
    const int kh = (int)fdiv(tap, g.d_kw), kw = (int)tap - kh * g.KW;
    const int u = r0 + kh, v = c0 + kw;
    int av = 0;
    if ((unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w) {
      const int row = (int)fdiv((uint32_t)u, g.d_dh), col = (int)fdiv((uint32_t)v, g.d_dw);
      if (row * g.dil_h == u && col * g.dil_w == v) av = V[nb + ((long long)(row * g.SW + col) * g.SC + ch)];
    }
    const int tp = prm.u_t0 + kh * prm.u_tj + kw * prm.u_ti;
    const int bv = U[(long long)tp * prm.u_tap + (long long)ch * prm.u_sk + (long long)q * prm.u_sq];
    acc = step_i32(acc, av, bv, prm.v_first != 0, prm.lut_raw, prm.m);
  }
  reinterpret_cast<int*>(prm.O)[(long long)p * prm.o_sp + (long long)q * prm.o_sq] = acc;
}

__global__ void naive_fgrad_i32(const Params prm) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)prm.P * prm.Q) return;
  const Gather& g = prm.g;
  const int* __restrict__ V = reinterpret_cast<const int*>(prm.V);
  const int* __restrict__ U = reinterpret_cast<const int*>(prm.U);
  const uint32_t p = (uint32_t)(idx / prm.Q);
  const int q = (int)(idx - (long long)p * prm.Q);
  const uint32_t tap = fdiv(p, g.d_sc);
  const int ch = (int)(p - tap * (uint32_t)g.SC);
  const int kh = (int)fdiv(tap, g.d_kw), kw = (int)tap - kh * g.KW;
  int acc = 0;
  for (int pix = 0; pix < prm.K; ++pix) {
    const uint32_t n = fdiv((uint32_t)pix, g.d_img);
    const uint32_t rem = (uint32_t)pix - n * (uint32_t)(g.PH * g.PW);
    const uint32_t a = fdiv(rem, g.d_pw), b = rem - a * (uint32_t)g.PW;
    const int u = (int)a * g.ps_h - g.off_t + kh, v = (int)b * g.ps_w - g.off_l + kw;
    int av = 0;
    if ((unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w)
      av = V[(long long)n * ((long long)g.SH * g.SW * g.SC) + ((long long)(u * g.SW + v) * g.SC + ch)];
    const int bv = U[(long long)pix * prm.u_sk + (long long)q * prm.u_sq];
    acc = step_i32(acc, av, bv, prm.v_first != 0, prm.lut_raw, prm.m);
  }
  reinterpret_cast<int*>(prm.O)[(long long)p * prm.Q + q] = acc;
}

__global__ void mul_elementwise(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                size_t n, const uint8_t* __restrict__ lut, int m, int lut_mode) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t at = __float_as_uint(a[i]), bt = __float_as_uint(b[i]);
    uint32_t r;
    if (lut_mode == LM_DIRECT_MBM) r = direct_mul_bits<true>(at, bt);
    else if (lut_mode == LM_DIRECT_MIT) r = direct_mul_bits<false>(at, bt);
    else r = am_mul_bits(at, bt, lut, m, lut_mode == LM_GLOBAL16);
    out[i] = __uint_as_float(r);
  }
}

}  // namespace amsim
