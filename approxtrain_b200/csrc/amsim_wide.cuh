// Wide-tile filter / weight gradient: the same abstract product as fgrad_gemm,
//     Out[p, q] = sum_k AM(V[p, k], U[k, q]),  p = (tap, channel), k = pixel,
// with a 16 (q) x 8 or 16 x 9 (p) register tile per thread instead of 16 x 4.
//
// What it buys.  (1) 288-row tiles (9 rows per lane) fit the 9 taps of a 3x3
// filter times a multiple of 32 channels exactly: a 576-row gradient (64
// channels) needs two tiles instead of five 128-row tiles with 10 % padding.
// (2) Per reduction step a warp fetches its 16 uniform-operand words once for
// twice as many products, so instructions per product drop from 4.8 to 4.65
// and shared-memory wavefronts from 1.35 to 1.19.  With an additive table
// (no lookups: two instructions per product, issue bound) that is worth
// 20-28 %; with a table in shared memory the kernel is bound by issue slots at
// about four instructions per product either way, 8 instead of 12 resident
// warps per multiprocessor hide less lookup latency, and it only pays where
// the taller tile removes padding.
//
// What makes 128-144 accumulators fit (255 registers, 2 CTAs of 4 warps per
// SM): the lane operand goes from global to shared memory with 16-byte
// cp.async (zero-filled where a tap falls into the padding) and is encoded on
// read (table column, sign+exponent word, zero test: four logic ops per word,
// each word used for 16 products), so no thread holds staged lane-operand
// values in registers across the product loop; the uniform operand (8
// elements per thread and stage) keeps the two-word register staging of the
// 16 x 4 kernels.  Products of one step are issued in groups of four rows so
// that only four "operand is zero" predicates are live at a time.
//
// Fast mode and tables in shared memory (or additive) only; 128-bit gathers, except for
// the 160-row variant (5 rows per lane), which stages element by element.
// A gather-side kernel of the same shape (forward / input gradient) was built
// in two layouts and measured 4-14 % slower than the 16 x 4 gather_gemm on the
// 3x3 microbenchmark shapes; it is not kept.
#pragma once
#include "amsim_kernels.cuh"

namespace amsim {

constexpr int WNT = 128;              // threads per CTA (4 warps, one 16-column group each)
__host__ __device__ constexpr int wide_fgrad_pitch(int np) { return 32 * np + 4; }  // wide_fgrad: V row [k][p], words

// words of the double-buffered V tile of wide_fgrad with np rows per lane
__host__ __device__ constexpr int wide_v_words(int np) { return 2 * BK * wide_fgrad_pitch(np); }
__host__ __device__ constexpr int wide_tile_bytes(int np) { return (wide_v_words(np) + 2 * U_TILE_WORDS + 8) * 4; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0 source bytes: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// One reduction step of a 16 (q) x 8 (p) register tile.
//   wv   : this lane's 8 lane-operand values, raw FP32 bits
//   urow : 16 uniform-operand sign+exponent words, their table-row (or mantissa-field)
//          words U_TILE_WORDS further on
template <int LM, int NP>
__device__ __forceinline__ void mac_wide(float (&acc)[TR][NP], const uint32_t (&wv)[NP],
                                         const uint32_t* __restrict__ urow, const uint32_t lut_base, const int sh,
                                         const uint32_t cmask, const uint32_t mult, const uint32_t keep) {
  uint32_t uu[TR], dd[TR];
#pragma unroll
  for (int g4 = 0; g4 < TR / 4; ++g4) {
    const uint4 a = *reinterpret_cast<const uint4*>(urow + 4 * g4);
    const uint4 b = *reinterpret_cast<const uint4*>(urow + U_TILE_WORDS + 4 * g4);
    uu[4 * g4] = a.x; uu[4 * g4 + 1] = a.y; uu[4 * g4 + 2] = a.z; uu[4 * g4 + 3] = a.w;
    dd[4 * g4] = b.x; dd[4 * g4 + 1] = b.y; dd[4 * g4 + 2] = b.z; dd[4 * g4 + 3] = b.w;
  }
  if (LM == LM_SMEM && NP == 9) {
    // The table-row offsets are the same in every lane.  A warp-wide OR says so to the compiler:
    // its result lives in a uniform register and rides in the lookup's address (lane register +
    // uniform register), which saves the address instruction of every product.  One such
    // reduction per column serves NP rows; with the four rows of the 16 x 4 kernels the reductions
    // cost more than the address instructions they save (measured: 7-13 % slower there, 3.7 %
    // faster here with nine rows, 7 % slower with eight).
#pragma unroll
    for (int r = 0; r < TR; ++r) dd[r] = __reduce_or_sync(0xffffffffu, dd[r]);
  }
#pragma unroll
  for (int h = 0; h < (NP + 3) / 4; ++h) {
    uint32_t ci[4], cs[4];
    bool nz[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (4 * h + t >= NP) continue;
      const uint32_t w = wv[4 * h + t];
      ci[t] = ((w >> sh) & cmask) | lut_base;
      cs[t] = LM == LM_ADD ? (w & keep) : (w & 0xFF800000u);
      nz[t] = (w & 0x7F800000u) != 0u;  // zero / denormal lane operand: the product is exactly 0
    }
#pragma unroll
    for (int r = 0; r < TR; ++r) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (4 * h + t >= NP) continue;
        const uint32_t e = LM == LM_ADD ? dd[r] : lds_u8(dd[r] + ci[t]) * mult;
        const float y = __uint_as_float(e + cs[t]);
        const float s = __fmaf_rn(__uint_as_float(uu[r]), y, acc[r][4 * h + t]);
        acc[r][4 * h + t] = nz[t] ? s : acc[r][4 * h + t];
      }
    }
  }
}

// -----------------------------------------------------------------------------
// wide_fgrad: p = (tap, channel), q = output channel, reduction over pixels.
// grid = (ceil(P / (32 NP)), ceil(Q/64), splits); split s reduces pixels
// [s * k_chunk, min((s+1) * k_chunk, K)) into ws[s] (or O if there is one split).
// NP rows per lane: 8 (256-row tiles) or 9 (288-row tiles: the 9 taps of a 3x3
// filter times a multiple of 32 channels tile without padding).  Lane l holds
// rows 4l..4l+3 of every full group of 128 rows, then row l of a last group of 32.
// NP = 5 with VEC = false (160-row tiles, 3 CTAs per SM, the lane operand staged
// element by element with 4-byte cp.async): channel counts that are no multiple
// of 4, whose rows would otherwise pad to the next multiple of 128 (a 7x7x3 first
// layer: 147 rows fill 92 % of one 160-row tile, 57 % of two 128-row tiles).
// -----------------------------------------------------------------------------
template <int NP>
__device__ __forceinline__ int wide_fgrad_row(int lane, int c) {
  return c < (NP / 4) * 4 ? (c >> 2) * 128 + 4 * lane + (c & 3) : (NP / 4) * 128 + (NP % 4) * lane + (c & 3);
}

template <int LM, int NP, bool VEC = true>
__global__ void __launch_bounds__(WNT, NP >= 8 ? 2 : 3) wide_fgrad(const Params prm) {
  static_assert(NP == 5 || NP == 8 || NP == 9, "rows per lane");
  static_assert(VEC == (NP != 5), "element-wise staging is written for the 128 + 32 columns of the 160-row tile");
  constexpr int NU = BK * BQ / WNT;
  constexpr int BPT = 32 * NP;            // rows of the CTA tile
  constexpr int FS = wide_fgrad_pitch(NP);
  constexpr int GPR = BPT / 4;            // 16-byte groups per k row (64 / 72)
  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* Vs = reinterpret_cast<uint32_t*>(smem);  // [2][BK][FS]
  uint32_t* Us = Vs + wide_v_words(NP);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t lut_base = (smem_base + prm.tile_bytes + prm.lut_align - 1) & ~(prm.lut_align - 1);
  uint8_t* lut_s = smem + (lut_base - smem_base);

  const int t = threadIdx.x, lane = t & 31;
  const int wq = __shfl_sync(0xffffffffu, t >> 5, 0);
  const int p0 = blockIdx.x * BPT, q0 = blockIdx.y * BQ;
  const int kbeg = blockIdx.z * prm.k_chunk;
  const int kend = min(kbeg + prm.k_chunk, prm.K);
  const Gather& g = prm.g;
  const float* __restrict__ Vg = prm.V;
  const float* __restrict__ Ug = prm.U;
  const int sh = 23 - prm.m;
  const uint32_t keep = ~((1u << sh) - 1u);


  // 16-byte group c = t + 128 i (i < NP) of the BK x GPR groups of a stage: k row c / GPR, rows
  // 4 (c % GPR) .. + 3 (one tap: the channel count is a multiple of 4)
  // Element-wise staging (VEC false): thread t fills column t of every k row and column 128 + lane
  // of k rows 4 (t / 32) .. + 3; the columns' taps are decoded once.
  int e_kh[2] = {0, 0}, e_kw[2] = {0, 0}, e_ch[2] = {0, 0};
  bool e_ok[2] = {false, false};
  if (!VEC) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t pg = (uint32_t)(p0 + (j == 0 ? t : 128 + lane));
      const uint32_t tap = fdiv(pg, g.d_sc);
      e_ch[j] = (int)(pg - tap * (uint32_t)g.SC);
      e_kh[j] = (int)fdiv(tap, g.d_kw);
      e_kw[j] = (int)tap - e_kh[j] * g.KW;
      e_ok[j] = pg < (uint32_t)prm.P;
    }
  }
  auto issue_v = [&](int kb, int buf) {
    if (!VEC) {
#pragma unroll 4
      for (int kr = 0; kr < BK; ++kr) {
        const int pix = kbeg + kb * BK + kr;
        const uint32_t n = fdiv((uint32_t)pix, g.d_img);
        const uint32_t rem = (uint32_t)pix - n * (uint32_t)(g.PH * g.PW);
        const uint32_t a = fdiv(rem, g.d_pw);
        const uint32_t b = rem - a * (uint32_t)g.PW;
        const int u0 = (int)a * g.ps_h - g.off_t, v0 = (int)b * g.ps_w - g.off_l;
        const float* img = Vg + (long long)n * ((long long)g.SH * g.SW * g.SC);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (j == 1 && (kr >> 2) != (t >> 5)) continue;
          const int u = u0 + e_kh[j], v = v0 + e_kw[j];
          bool ok = e_ok[j] && pix < kend && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w;
          const float* src = ok ? img + ((long long)(u * g.SW + v) * g.SC + e_ch[j]) : Vg;
          ok = ok && AMSIM_IN(prm, BUF_V, src, float);
          cp_async4(smem_base + (uint32_t)(((buf * BK + kr) * FS + (j == 0 ? t : 128 + lane)) * 4), src, ok);
        }
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int c = t + WNT * i;
      const int kr = c / GPR, pl = 4 * (c - kr * GPR);
      const uint32_t pg = (uint32_t)(p0 + pl);
      const uint32_t tap = fdiv(pg, g.d_sc);
      const int ch = (int)(pg - tap * (uint32_t)g.SC);
      const int kh = (int)fdiv(tap, g.d_kw);
      const int kw = (int)tap - kh * g.KW;
      const int pix = kbeg + kb * BK + kr;
      const uint32_t n = fdiv((uint32_t)pix, g.d_img);
      const uint32_t rem = (uint32_t)pix - n * (uint32_t)(g.PH * g.PW);
      const uint32_t a = fdiv(rem, g.d_pw);
      const uint32_t b = rem - a * (uint32_t)g.PW;
      const int u = (int)a * g.ps_h - g.off_t + kh, v = (int)b * g.ps_w - g.off_l + kw;
      bool ok = pg < (uint32_t)prm.P && pix < kend && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w;
      const float* src = ok ? Vg + ((long long)n * ((long long)g.SH * g.SW * g.SC) + ((long long)(u * g.SW + v) * g.SC + ch))
                            : Vg;
      ok = ok && AMSIM_IN(prm, BUF_V, src, float4);
      cp_async16(smem_base + (uint32_t)(((buf * BK + kr) * FS + pl) * 4), src, ok);
    }
  };

  float uraw[NU];
  auto load_u = [&](int kb) {
    if (prm.u_vec) {
#pragma unroll
      for (int j = 0; j < NU / 4; ++j) {
        const int f = j * WNT + t;
        const int pix = kbeg + kb * BK + (f >> 4), qg = q0 + (f & 15) * 4;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (pix < kend && qg < prm.Q && AMSIM_IN(prm, BUF_U, Ug + (long long)pix * prm.u_sk + qg, float4))
          val = __ldg(reinterpret_cast<const float4*>(Ug + (long long)pix * prm.u_sk + qg));
        uraw[4 * j] = val.x; uraw[4 * j + 1] = val.y; uraw[4 * j + 2] = val.z; uraw[4 * j + 3] = val.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NU; ++j) {
        const int e = j * WNT + t;
        const int pix = kbeg + kb * BK + (e >> 6), qg = q0 + (e & 63);
        const float* src = Ug + (long long)pix * prm.u_sk + (long long)qg * prm.u_sq;
        uraw[j] = (pix < kend && qg < prm.Q && AMSIM_IN(prm, BUF_U, src, float)) ? __ldg(src) : 0.f;
      }
    }
  };
  auto store_u_tile = [&](int buf) {
    if (prm.u_vec) {
#pragma unroll
      for (int j = 0; j < NU / 4; ++j) {
        const int f = j * WNT + t;
        const float f4[4] = {uraw[4 * j], uraw[4 * j + 1], uraw[4 * j + 2], uraw[4 * j + 3]};
        store_u4<LM>(Us + buf * BK * US + (f >> 4) * US + (f & 15) * 4, f4, prm.m);
      }
    } else {
#pragma unroll
      for (int j = 0; j < NU; ++j) {
        const int e = j * WNT + t;
        store_u<LM>(Us + buf * BK * US + (e >> 6) * US + (e & 63), __float_as_uint(uraw[j]), prm.m);
      }
    }
  };

  float acc[TR][NP];
#pragma unroll
  for (int r = 0; r < TR; ++r)
#pragma unroll
    for (int c = 0; c < NP; ++c) acc[r][c] = 0.f;

  const int nkb = (kend - kbeg + BK - 1) / BK;
  const int ucol = wq * TR;
  if (nkb > 0) {
    issue_v(0, 0);
    load_u(0);
  }
  // the table is copied while the first stage's copies and loads are in flight
  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, WNT);
  if (nkb > 0) store_u_tile(0);
  cp_async_wait_all();
  __syncthreads();
  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nkb) {
      issue_v(kb + 1, buf ^ 1);
      load_u(kb + 1);
    }
    const uint32_t* vs = Vs + buf * BK * FS;
    const uint32_t* us = Us + buf * BK * US + ucol;
#pragma unroll 1
    for (int kk = 0; kk < BK; ++kk) {
      uint32_t wv[NP];
      const uint4 lo = *reinterpret_cast<const uint4*>(vs + kk * FS + 4 * lane);
      wv[0] = lo.x; wv[1] = lo.y; wv[2] = lo.z; wv[3] = lo.w;
      if (NP >= 8) {
        const uint4 hi = *reinterpret_cast<const uint4*>(vs + kk * FS + 128 + 4 * lane);
        wv[4] = hi.x; wv[5] = hi.y; wv[6] = hi.z; wv[7] = hi.w;
      }
      if (NP % 4 == 1) wv[NP - 1] = vs[kk * FS + (NP / 4) * 128 + lane];
      mac_wide<LM, NP>(acc, wv, us + kk * US, lut_base, sh, prm.cmask, prm.mult, keep);
    }
    if (kb + 1 < nkb) store_u_tile(buf ^ 1);
    cp_async_wait_all();
    __syncthreads();
  }

  const bool to_ws = prm.splits > 1;
  float* __restrict__ Og = to_ws ? prm.ws + (long long)blockIdx.z * ((long long)prm.P * prm.Q) : prm.O;
  const long long sp = to_ws ? prm.Q : prm.o_sp, sq = to_ws ? 1 : prm.o_sq;
  const bool vec_out = sq == 1 && (sp & 3) == 0 && ((reinterpret_cast<uintptr_t>(Og) & 15) == 0);
#pragma unroll
  for (int c = 0; c < NP; ++c) {
    const int pg = p0 + wide_fgrad_row<NP>(lane, c);
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

}  // namespace amsim
