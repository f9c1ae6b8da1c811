// Wide-tile fast kernels: the same abstract product as amsim_kernels.cuh,
//     Out[p, q] = sum_k AM(V[p, k], U[k, q]),
// with a 16 (q) x 8 (p) register tile per thread instead of 16 x 4, for the
// large fast-mode launches that dominate a training step.
//
// Why.  In the 16 x 4 kernels the shared-memory data pipe is the busiest unit:
// per warp and reduction step 64 table lookups (one wavefront each, the bound),
// plus 16 wavefronts of uniform-operand words and 4 of lane-operand words,
// i.e. 1.31 wavefronts per warp-product before staging.  Both operand terms are
// per-step costs amortised over the register tile: 1/TC for the uniform
// operand, 1/TR for the lane operand.  With 8 rows per lane they drop to
// 16 + 8 wavefronts per 128 lookups (1.19), and the instructions spent on
// operand fetch and unpacking halve as well.
//
// What makes 128 accumulators fit (255 registers, 2 CTAs of 4 warps per SM):
// the lane operand goes from global to shared memory with cp.async and is
// encoded on read (table column, sign+exponent word, zero test: four logic ops
// per word, each word used for 16 products), so no thread holds staged operand
// values in registers across the product loop; the uniform operand (8 elements
// per thread and stage) keeps the two-word register staging of the 16 x 4
// kernels.  Products of one step are issued in two halves of four rows so that
// only four "operand is zero" predicates are live at a time.
//
//   wide_gather  V gathered along k (conv forward / input gradient, dense, 1x1
//                GEMMs).  Shared-memory tile [p][k], row pitch 17 words: the
//                four 4-byte cp.async of a 16-byte channel group land in one
//                row, and a warp's reads of one k (32 consecutive rows) fall
//                into 32 different banks.
//   wide_fgrad   V gathered along p (filter / weight gradients), tile [k][p]
//                filled by 16-byte cp.async, read with two 128-bit loads per
//                lane and step.
// Fast mode, 128-bit gathers and tables in shared memory (or additive) only;
// everything else stays on the 16 x 4 kernels.
#pragma once
#include "amsim_kernels.cuh"

namespace amsim {

constexpr int WT = 8;                 // p values per lane
constexpr int WBP = 32 * WT;          // rows of a CTA tile
constexpr int WNT = 128;              // threads per CTA (4 warps, one 16-column group each)
constexpr int WGP = BK + 1;           // wide_gather: pitch of a V row [p][k], words (odd: conflict-free column reads)
__host__ __device__ constexpr int wide_fgrad_pitch(int np) { return 32 * np + 4; }  // wide_fgrad: V row [k][p], words
constexpr int W_ACC = TR * WT * WNT;  // floats of one CTA's register tiles (balanced launch: one parked slot)

// words of the double-buffered V tile: np = 0 for wide_gather, else wide_fgrad with np rows per lane
__host__ __device__ constexpr int wide_v_words(int np) { return np ? 2 * BK * wide_fgrad_pitch(np) : 2 * WBP * WGP; }
__host__ __device__ constexpr int wide_tile_bytes(int np) { return (wide_v_words(np) + 2 * U_TILE_WORDS + 8) * 4; }

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 4 : 0;  // 0 source bytes: the word is zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
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
        const uint32_t e = LM == LM_ADD ? dd[r] : lds_u8(dd[r] | ci[t]) * mult;
        const float y = __uint_as_float(e + cs[t]);
        const float s = __fmaf_rn(__uint_as_float(uu[r]), y, acc[r][4 * h + t]);
        acc[r][4 * h + t] = nz[t] ? s : acc[r][4 * h + t];
      }
    }
  }
}

// -----------------------------------------------------------------------------
// wide_gather.  grid: plain = (ceil(P/256), ceil(Q/64), batch); balanced = sk_grid CTAs.
// -----------------------------------------------------------------------------
template <int LM, int MODE>
__global__ void __launch_bounds__(WNT, 2) wide_gather(const Params prm) {
  constexpr bool BALANCED = MODE == GM_BALANCED;
  constexpr int NU = BK * BQ / WNT;
  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* Vs = reinterpret_cast<uint32_t*>(smem);            // [2][WBP][WGP]
  uint32_t* Us = Vs + wide_v_words(0);                      // [2 words][2 stages][BK][US]
  uint32_t* flag_s = Us + 2 * U_TILE_WORDS;
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t lut_base = (smem_base + prm.tile_bytes + prm.lut_align - 1) & ~(prm.lut_align - 1);
  uint8_t* lut_s = smem + (lut_base - smem_base);

  const int t = threadIdx.x, lane = t & 31;
  const int wq = __shfl_sync(0xffffffffu, t >> 5, 0);  // warp index, known to be warp-uniform
  const Gather& g = prm.g;
  const int nkb_all = (prm.K + BK - 1) / BK;
  const int sh = 23 - prm.m;
  const uint32_t keep = ~((1u << sh) - 1u);

  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, WNT);

  long long run_at = 0, run_end = 0;
  if (BALANCED) {
    run_at = balanced_begin(blockIdx.x, prm.sk_iters, prm.sk_grid);
    run_end = balanced_begin((long long)blockIdx.x + 1, prm.sk_iters, prm.sk_grid);
    if (run_at >= run_end) return;
  }
  do {
    int tile_p, tile_q, tile_z, kb_begin, nkb;
    if (BALANCED) {
      const long long tile = run_at / nkb_all;
      kb_begin = (int)(run_at - tile * nkb_all);
      nkb = kb_begin + (int)min((long long)(nkb_all - kb_begin), run_end - run_at);
      run_at += nkb - kb_begin;
      tile_q = (int)(tile % prm.sk_qtiles);
      const long long rest = tile / prm.sk_qtiles;
      tile_p = (int)(rest % prm.sk_ptiles);
      tile_z = (int)(rest / prm.sk_ptiles);
    } else {
      tile_p = blockIdx.x;
      tile_q = blockIdx.y;
      tile_z = blockIdx.z;
      kb_begin = 0;
      nkb = nkb_all;
    }
    const int p0 = tile_p * WBP, q0 = tile_q * BQ;
    const float* __restrict__ Vg = prm.V + (long long)tile_z * prm.v_bs;
    const float* __restrict__ Ug = prm.U + (long long)tile_z * prm.u_bs;
    float* __restrict__ Og = prm.O + (long long)tile_z * prm.o_bs;

    // ---- V: thread t copies the 16-byte channel group (t & 3) of rows (t >> 2) + 32 i, i < 8 ----
    const int vrow = t >> 2, vgrp = t & 3;
    auto issue_v = [&](int kb, int buf) {
      const int kglob = kb * BK + 4 * vgrp;
      const uint32_t tap = fdiv((uint32_t)kglob, g.d_sc);
      const int ch = kglob - (int)tap * g.SC;
      const int kh = (int)fdiv(tap, g.d_kw);
      const int kw = (int)tap - kh * g.KW;
      const bool kok = kglob < prm.K;
      const uint32_t dst0 = smem_base + (uint32_t)((buf * WBP * WGP + vrow * WGP + 4 * vgrp) * 4);
#pragma unroll
      for (int i = 0; i < WT; ++i) {
        const uint32_t pg = (uint32_t)(p0 + vrow + 32 * i);
        const uint32_t n = fdiv(pg, g.d_img);
        const uint32_t rem = pg - n * (uint32_t)(g.PH * g.PW);
        const uint32_t a = fdiv(rem, g.d_pw);
        const uint32_t b = rem - a * (uint32_t)g.PW;
        const int u = (int)a * g.ps_h - g.off_t + kh, v = (int)b * g.ps_w - g.off_l + kw;
        const bool ok = kok && pg < (uint32_t)prm.P && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w;
        const float* src = ok ? Vg + ((long long)n * ((long long)g.SH * g.SW * g.SC) + ((long long)(u * g.SW + v) * g.SC + ch))
                              : Vg;
        const uint32_t dst = dst0 + (uint32_t)(32 * i * WGP * 4);
        cp_async4(dst, src, ok);
        cp_async4(dst + 4, src + 1, ok);
        cp_async4(dst + 8, src + 2, ok);
        cp_async4(dst + 12, src + 3, ok);
      }
    };

    // ---- U through registers, as in gather_gemm ------------------------------------------------
    float uraw[NU];
    const bool u_kmajor = prm.u_sk == 1 && prm.u_sq != 1;
    auto load_u = [&](int kb) {
      if (prm.u_vec) {
#pragma unroll
        for (int j = 0; j < NU / 4; ++j) {
          const int f = j * WNT + t;
          const int kl = prm.u_vec == 2 ? (f & 3) * 4 : (f >> 4);
          const int ql = prm.u_vec == 2 ? (f >> 2) : (f & 15) * 4;
          const int kglob = kb * BK + kl, qg = q0 + ql;
          float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
          if (kglob < prm.K && qg < prm.Q) {
            const uint32_t tap = fdiv((uint32_t)kglob, g.d_sc);
            const int kk = kglob - (int)tap * g.SC;
            const int tj = (int)fdiv(tap, g.d_kw);
            const int tp = prm.u_t0 + tj * prm.u_tj + ((int)tap - tj * g.KW) * prm.u_ti;
            val = __ldg(reinterpret_cast<const float4*>(Ug + (long long)tp * prm.u_tap + (long long)kk * prm.u_sk +
                                                        (long long)qg * prm.u_sq));
          }
          uraw[4 * j] = val.x; uraw[4 * j + 1] = val.y; uraw[4 * j + 2] = val.z; uraw[4 * j + 3] = val.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < NU; ++j) {
          const int e = j * WNT + t;
          const int kl = u_kmajor ? (e & (BK - 1)) : (e >> 6);
          const int ql = u_kmajor ? (e >> 4) : (e & 63);
          const int kglob = kb * BK + kl, qg = q0 + ql;
          float val = 0.f;
          if (kglob < prm.K && qg < prm.Q) {
            const uint32_t tap = fdiv((uint32_t)kglob, g.d_sc);
            const int kk = kglob - (int)tap * g.SC;
            const int tj = (int)fdiv(tap, g.d_kw);
            const int tp = prm.u_t0 + tj * prm.u_tj + ((int)tap - tj * g.KW) * prm.u_ti;
            val = __ldg(Ug + (long long)tp * prm.u_tap + (long long)kk * prm.u_sk + (long long)qg * prm.u_sq);
          }
          uraw[j] = val;
        }
      }
    };
    auto store_u_tile = [&](int buf) {
      if (prm.u_vec) {
#pragma unroll
        for (int j = 0; j < NU / 4; ++j) {
          const int f = j * WNT + t;
          if (prm.u_vec == 2) {
            uint32_t* dst = Us + buf * BK * US + (f & 3) * 4 * US + (f >> 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) store_u<LM>(dst + i * US, __float_as_uint(uraw[4 * j + i]), prm.m);
          } else {
            const float f4[4] = {uraw[4 * j], uraw[4 * j + 1], uraw[4 * j + 2], uraw[4 * j + 3]};
            store_u4<LM>(Us + buf * BK * US + (f >> 4) * US + (f & 15) * 4, f4, prm.m);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < NU; ++j) {
          const int e = j * WNT + t;
          const int kl = u_kmajor ? (e & (BK - 1)) : (e >> 6);
          const int ql = u_kmajor ? (e >> 4) : (e & 63);
          store_u<LM>(Us + buf * BK * US + kl * US + ql, __float_as_uint(uraw[j]), prm.m);
        }
      }
    };

    float acc[TR][WT];
#pragma unroll
    for (int r = 0; r < TR; ++r)
#pragma unroll
      for (int c = 0; c < WT; ++c) acc[r][c] = 0.f;

    if (kb_begin < nkb) {
      issue_v(kb_begin, 0);
      load_u(kb_begin);
      store_u_tile(0);
    }
    cp_async_wait_all();
    __syncthreads();

    const int ucol = wq * TR;
    for (int kb = kb_begin; kb < nkb; ++kb) {
      const int buf = (kb - kb_begin) & 1;
      if (kb + 1 < nkb) {
        issue_v(kb + 1, buf ^ 1);
        load_u(kb + 1);
      }
      const uint32_t* vs = Vs + buf * WBP * WGP + lane * WGP;
      const uint32_t* us = Us + buf * BK * US + ucol;
#pragma unroll 1
      for (int kk = 0; kk < BK; ++kk) {
        uint32_t wv[WT];
#pragma unroll
        for (int i = 0; i < WT; ++i) wv[i] = vs[32 * i * WGP + kk];
        mac_wide<LM, WT>(acc, wv, us + kk * US, lut_base, sh, prm.cmask, prm.mult, keep);
      }
      if (kb + 1 < nkb) store_u_tile(buf ^ 1);
      cp_async_wait_all();
      __syncthreads();
    }

    // ---- output: this thread holds rows p0 + lane + 32 i, columns q0 + ucol .. + 15 -------------
    auto store_rows = [&]() {
      const bool vec_out = prm.o_sq == 1 && (prm.o_sp & 3) == 0 && (prm.o_bs & 3) == 0 &&
                           ((reinterpret_cast<uintptr_t>(prm.O) & 15) == 0);
      const bool epi = prm.bias != nullptr || prm.relu || prm.scale != nullptr || prm.has_alpha;
#pragma unroll
      for (int i = 0; i < WT; ++i) {
        const int pg = p0 + lane + 32 * i;
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
          const int qg = q0 + ucol + 4 * g4;
          float o[4] = {acc[4 * g4][i], acc[4 * g4 + 1][i], acc[4 * g4 + 2][i], acc[4 * g4 + 3][i]};
          if (epi) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              if (prm.has_alpha) o[r] = __fmul_rn(o[r], prm.alpha);
              if (prm.scale != nullptr && qg + r < prm.Q) o[r] = __fmul_rn(o[r], __ldg(prm.scale + qg + r));
              if (prm.bias != nullptr && qg + r < prm.Q) o[r] = __fadd_rn(o[r], __ldg(prm.bias + qg + r));
              if (prm.relu) o[r] = o[r] < 0.f ? 0.f : o[r];
            }
          }
          if (vec_out && qg + 3 < prm.Q) {
            *reinterpret_cast<float4*>(orow + qg) = make_float4(o[0], o[1], o[2], o[3]);
          } else {
#pragma unroll
            for (int r = 0; r < 4; ++r)
              if (qg + r < prm.Q) orow[(long long)(qg + r) * prm.o_sq] = o[r];
          }
        }
      }
    };

    // Balanced launch: a tile shared between CTAs parks its register tile (slot 0: the run started
    // inside the tile, slot 1: it started the tile) and counts itself in; the CTA that completes
    // the count adds the parked tiles in CTA order and writes the output.  Nobody waits.
    if (BALANCED && (kb_begin != 0 || nkb != nkb_all)) {
      float* slot = prm.ws + ((long long)blockIdx.x * 2 + (kb_begin == 0 ? 1 : 0)) * W_ACC;
#pragma unroll
      for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int c = 0; c < WT; ++c) __stcg(slot + (r * WT + c) * WNT + t, acc[r][c]);
      __threadfence();
      __syncthreads();
      const long long tile = ((long long)tile_z * prm.sk_ptiles + tile_p) * prm.sk_qtiles + tile_q;
      const long long first = tile * nkb_all, last = first + nkb_all;
      long long c0 = first * prm.sk_grid / prm.sk_iters;
      while (c0 > 0 && balanced_begin(c0, prm.sk_iters, prm.sk_grid) > first) --c0;
      while (balanced_begin(c0 + 1, prm.sk_iters, prm.sk_grid) <= first) ++c0;
      long long c1 = (last - 1) * prm.sk_grid / prm.sk_iters;
      while (c1 > 0 && balanced_begin(c1, prm.sk_iters, prm.sk_grid) > last - 1) --c1;
      while (balanced_begin(c1 + 1, prm.sk_iters, prm.sk_grid) <= last - 1) ++c1;
      if (t == 0) {
        const int arrived = atomicAdd(prm.sk_count + tile, 1);
        *flag_s = arrived == (int)(c1 - c0);
      }
      __syncthreads();
      const bool completes = *flag_s != 0;
      __syncthreads();
      if (completes) {
        __threadfence();
#pragma unroll
        for (int r = 0; r < TR; ++r)
#pragma unroll
          for (int c = 0; c < WT; ++c) acc[r][c] = 0.f;
        for (long long cta = c0; cta <= c1; ++cta) {
          const long long b = balanced_begin(cta, prm.sk_iters, prm.sk_grid);
          const float* src = prm.ws + (cta * 2 + (b <= first ? 1 : 0)) * W_ACC;
#pragma unroll
          for (int r = 0; r < TR; ++r)
#pragma unroll
            for (int c = 0; c < WT; ++c) acc[r][c] = __fadd_rn(acc[r][c], __ldcg(src + (r * WT + c) * WNT + t));
        }
        store_rows();
      }
    } else {
      store_rows();
    }
  } while (BALANCED && run_at < run_end);
}

// -----------------------------------------------------------------------------
// wide_fgrad: p = (tap, channel), q = output channel, reduction over pixels.
// grid = (ceil(P / (32 NP)), ceil(Q/64), splits); split s reduces pixels
// [s * k_chunk, min((s+1) * k_chunk, K)) into ws[s] (or O if there is one split).
// NP rows per lane: 8 (256-row tiles) or 9 (288-row tiles: the 9 taps of a 3x3
// filter times a multiple of 32 channels tile without padding).  Lane l holds
// rows 4l..4l+3 of every full group of 128 rows, then row l of a last group of 32.
// -----------------------------------------------------------------------------
template <int NP>
__device__ __forceinline__ int wide_fgrad_row(int lane, int c) {
  return c < (NP / 4) * 4 ? (c >> 2) * 128 + 4 * lane + (c & 3) : (NP / 4) * 128 + (NP % 4) * lane + (c & 3);
}

template <int LM, int NP>
__global__ void __launch_bounds__(WNT, 2) wide_fgrad(const Params prm) {
  static_assert(NP == 8 || NP == 9, "rows per lane");
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

  if (LM == LM_SMEM) copy_lut_to_smem(lut_s, prm.lut, prm.lut_bytes, t, WNT);

  // 16-byte group c = t + 128 i (i < NP) of the BK x GPR groups of a stage: k row c / GPR, rows
  // 4 (c % GPR) .. + 3 (one tap: the channel count is a multiple of 4)
  auto issue_v = [&](int kb, int buf) {
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
      const bool ok = pg < (uint32_t)prm.P && pix < kend && (unsigned)u < (unsigned)g.lim_h && (unsigned)v < (unsigned)g.lim_w;
      const float* src = ok ? Vg + ((long long)n * ((long long)g.SH * g.SW * g.SC) + ((long long)(u * g.SW + v) * g.SC + ch))
                            : Vg;
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
        if (pix < kend && qg < prm.Q) val = __ldg(reinterpret_cast<const float4*>(Ug + (long long)pix * prm.u_sk + qg));
        uraw[4 * j] = val.x; uraw[4 * j + 1] = val.y; uraw[4 * j + 2] = val.z; uraw[4 * j + 3] = val.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NU; ++j) {
        const int e = j * WNT + t;
        const int pix = kbeg + kb * BK + (e >> 6), qg = q0 + (e & 63);
        uraw[j] = (pix < kend && qg < prm.Q) ? __ldg(Ug + (long long)pix * prm.u_sk + (long long)qg * prm.u_sq) : 0.f;
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
    store_u_tile(0);
  }
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
      const uint4 hi = *reinterpret_cast<const uint4*>(vs + kk * FS + 128 + 4 * lane);
      wv[0] = lo.x; wv[1] = lo.y; wv[2] = lo.z; wv[3] = lo.w;
      wv[4] = hi.x; wv[5] = hi.y; wv[6] = hi.z; wv[7] = hi.w;
      if (NP == 9) wv[NP - 1] = vs[kk * FS + 256 + lane];
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
        *reinterpret_cast<float4*>(orow + qg) =
            make_float4(acc[4 * g4][c], acc[4 * g4 + 1][c], acc[4 * g4 + 2][c], acc[4 * g4 + 3][c]);
      } else {
#pragma unroll
        for (int r = 0; r < 4; ++r)
          if (qg + r < prm.Q) orow[(long long)(qg + r) * sq] = acc[4 * g4 + r][c];
      }
    }
  }
}

}  // namespace amsim
