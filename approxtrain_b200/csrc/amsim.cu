// C ABI of the AM-Simulator kernels (declared in include/amsim.h): LUT handles,
// argument checking, launch configuration.  Device code is in
// amsim_kernels.cuh.  Nothing here synchronises the device or exits.
#include "../../include/amsim.h"

#include <cuda_runtime.h>
#include <limits.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#ifndef AMSIM_CTAS1
#define AMSIM_CTAS1 3
#endif
#include "amsim_kernels.cuh"
#include "amsim_wide.cuh"

#include <atomic>

// Kernels launched by this library since it was loaded (amsim_debug_launch_count).
static std::atomic<unsigned long long> g_launches{0};
#define AMSIM_COUNT_LAUNCH() g_launches.fetch_add(1, std::memory_order_relaxed)

using namespace amsim;

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define CUDA_TRY(expr)                                                                          \
  do {                                                                                          \
    cudaError_t e_ = (expr);                                                                    \
    if (e_ != cudaSuccess) return fail(AMSIM_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

// Debug switches.  The environment is read ONCE, when the first entry point needs a switch (or when
// amsim_debug_reload_env is called), never on the launch path: a *_workspace query and the launch
// that follows it always see the same plan.  -1 = not set (the library chooses per shape).
struct Switches {
  int balanced = -1;        // AMSIM_BALANCED=0/1        balanced launch of the gather kernels
  int force_ksplit = -1;    // AMSIM_FORCE_KSPLIT=n      cluster size of the cluster-split launch
  int no_qsplit = 0;        // AMSIM_NO_QSPLIT=1         narrow outputs on plain 64-column tiles
  int no_uvec = 0;          // AMSIM_NO_UVEC=1           scalar staging of the uniform operand
  int no_wgrad_swap = 0;    // AMSIM_NO_WGRAD_SWAP=1     GEMM-shaped weight gradients keep their operand roles
  int thin_fgrad = -1;      // AMSIM_THIN_FGRAD=0/1      deterministic filter gradient: tiled / thin kernel
  int thin_tq = -1;         // AMSIM_THIN_TQ=1/2/4       chains per thread of the thin kernel
  int thin_narrow = 0;      // AMSIM_THIN_NARROW=1       4 instead of 16 warps per CTA in the thin kernel
  int chain_fgrad = -1;     // AMSIM_CHAIN_FGRAD=0/1     deterministic filter gradient: products-in-parallel kernel
  int thin_fast = -1;       // AMSIM_THIN_FAST=0/1       fast filter gradient of tiny outputs
  int exact_only = 0;       // AMSIM_EXACT_ONLY=1        deterministic kernels never use the fast arithmetic
  int no_additive = 0;      // AMSIM_NO_ADDITIVE=1       additive tables are looked up like any other (at lut_open)
  int wide = -1;            // AMSIM_WIDE=0/1            wide-tile filter gradient: never / whenever eligible
  int capture_cluster = -1; // AMSIM_CAPTURE_CLUSTER=0/1 small launches inside a graph capture: balanced / cluster split
  int balanced_waves = -1;  // AMSIM_BALANCED_WAVES=n    CTAs of a balanced launch: n times the resident slots
  int bounds_shrink = 0;    // AMSIM_BOUNDS_SHRINK=n     bounds-checking build only: the output's recorded extent is n bytes
                            //                           short, so its last stores are caught (self-test of the checker)
};
Switches g_sw;
std::once_flag g_sw_once;

void load_switches() {
  Switches w;
  auto tri = [](const char* name, int& v) {
    if (const char* e = getenv(name)) v = atoi(e);
  };
  auto flag = [](const char* name, int& v) { v = getenv(name) != nullptr; };
  tri("AMSIM_BALANCED", w.balanced);
  tri("AMSIM_FORCE_KSPLIT", w.force_ksplit);
  flag("AMSIM_NO_QSPLIT", w.no_qsplit);
  flag("AMSIM_NO_UVEC", w.no_uvec);
  flag("AMSIM_NO_WGRAD_SWAP", w.no_wgrad_swap);
  tri("AMSIM_THIN_FGRAD", w.thin_fgrad);
  tri("AMSIM_THIN_TQ", w.thin_tq);
  flag("AMSIM_THIN_NARROW", w.thin_narrow);
  tri("AMSIM_CHAIN_FGRAD", w.chain_fgrad);
  tri("AMSIM_THIN_FAST", w.thin_fast);
  flag("AMSIM_EXACT_ONLY", w.exact_only);
  flag("AMSIM_NO_ADDITIVE", w.no_additive);
  tri("AMSIM_WIDE", w.wide);
  tri("AMSIM_CAPTURE_CLUSTER", w.capture_cluster);
  tri("AMSIM_BALANCED_WAVES", w.balanced_waves);
  tri("AMSIM_BOUNDS_SHRINK", w.bounds_shrink);
  g_sw = w;
}

const Switches& sw() {
  std::call_once(g_sw_once, load_switches);
  return g_sw;
}

// Multiprocessors of a device, looked up once per device.
int sm_count(int device) {
  static std::mutex mu;
  static std::map<int, int> known;
  std::lock_guard<std::mutex> lk(mu);
  auto it = known.find(device);
  if (it != known.end()) return it->second;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    (void)cudaGetLastError();
    return 148;  // B200; only reached when the attribute query itself fails
  }
  known[device] = sms;
  return sms;
}

#ifdef AMSIM_BOUNDS_CHECK
// Device word that records the first bad access of a bounds-checking build (one per device).
unsigned long long* bounds_word(int device) {
  static std::mutex mu;
  static std::map<int, unsigned long long*> words;
  std::lock_guard<std::mutex> lk(mu);
  auto it = words.find(device);
  if (it != words.end()) return it->second;
  unsigned long long* w = nullptr;
  if (cudaMalloc(&w, sizeof(*w)) != cudaSuccess || cudaMemset(w, 0, sizeof(*w)) != cudaSuccess) {
    (void)cudaGetLastError();
    w = nullptr;
  }
  words[device] = w;
  return w;
}
#endif

// Bounds-checking build: the extents the kernels' accesses are compared with.
void fill_bounds(amsim::Params& p, int device, const void* ws, size_t ws_bytes) {
#ifdef AMSIM_BOUNDS_CHECK
  const void* base[3] = {p.V, p.U, p.O};
  const long long elems[3] = {p.v_elems, p.u_elems, p.o_elems};
  for (int i = 0; i < 3; ++i) {
    p.bnd.lo[i] = static_cast<const char*>(base[i]);
    p.bnd.hi[i] = p.bnd.lo[i] + elems[i] * 4;
  }
  if (sw().bounds_shrink > 0) p.bnd.hi[amsim::BUF_O] -= sw().bounds_shrink;
  p.bnd.lo[amsim::BUF_WS] = static_cast<const char*>(ws);
  p.bnd.hi[amsim::BUF_WS] = static_cast<const char*>(ws) + ws_bytes;
  p.bnd.report = bounds_word(device);
#else
  (void)p; (void)device; (void)ws; (void)ws_bytes;
#endif
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) (void)cudaGetLastError();
  return dev;
}

}  // namespace

struct amsim_lut {
  int m = 0;
  int device = 0;
  int refs = 0;
  std::string key;
  uint8_t* d_raw = nullptr;    // 2^(2m) bytes as in the file (row = first operand)
  uint8_t* d_raw_t = nullptr;  // the same bytes transposed (row = second operand)  [m > 7]
  uint8_t* d_canon = nullptr;  // encoded, row = first operand (a)   [m <= 7]
  uint8_t* d_trans = nullptr;  // encoded, row = second operand (b)  [m <= 7]
  int enc_bytes = 0;           // size of each encoded copy, multiple of 16
  bool additive = false;       // encoded entry(i, j) == i + j for every pair: no lookups needed
  int direct = 0;              // LM_DIRECT_MBM / LM_DIRECT_MIT: no table at all, m = 23
  bool wide = false;           // 16-bit entries (d_raw / d_raw_t hold uint16), looked up in global memory
};

namespace {

std::mutex g_lut_mu;
std::map<std::string, amsim_lut*> g_lut_cache;

// approx_mul_lut.h:22-25
int parse_mant_width(const char* path) {
  const char* us = strrchr(path, '_');
  const char* dot = strrchr(path, '.');
  if (!us || !dot || dot <= us + 1) return -1;
  int m = 0;
  for (const char* p = us + 1; p < dot; ++p) {
    if (*p < '0' || *p > '9') return -1;
    m = m * 10 + (*p - '0');
    if (m > 99) return -1;
  }
  return (m >= 1 && m <= 11) ? m : -1;
}

// Table byte as the kernels consume it: carry and mantissa merged into one
// number so that  entry << (23 - m)  is exactly what AMsimulator.inl:22-23,31-32
// add to the exponent/mantissa bits.
inline uint8_t encode_entry(uint8_t v, int m) { return (uint8_t)(((v >> 7) << m) + (v & 0x7f)); }

// 16-bit entries: both orientations as uint16 tables in global memory.
int upload_lut16(const uint16_t* entries, int m, int device, amsim_lut** out) {
  int prev = 0;
  CUDA_TRY(cudaGetDevice(&prev));
  CUDA_TRY(cudaSetDevice(device));
  amsim_lut* h = new amsim_lut();
  h->m = m;
  h->device = device;
  h->refs = 1;
  h->wide = true;
  const size_t side = (size_t)1 << m, n = side * side;
  std::vector<uint16_t> tr(n);
  for (size_t a = 0; a < side; ++a)
    for (size_t b = 0; b < side; ++b) tr[b * side + a] = entries[a * side + b];
  cudaError_t e = cudaMalloc(&h->d_raw, n * 2);
  if (e == cudaSuccess) e = cudaMalloc(&h->d_raw_t, n * 2);
  if (e == cudaSuccess) e = cudaMemcpy(h->d_raw, entries, n * 2, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(h->d_raw_t, tr.data(), n * 2, cudaMemcpyHostToDevice);
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    cudaFree(h->d_raw_t);
    cudaFree(h->d_raw);
    delete h;
    return fail(AMSIM_ERR_CUDA, "upload of 16-bit lut: %s", cudaGetErrorString(e));
  }
  *out = h;
  return AMSIM_OK;
}

int upload_lut(const uint8_t* bytes, int m, int device, amsim_lut** out) {
  int prev = 0;
  CUDA_TRY(cudaGetDevice(&prev));
  CUDA_TRY(cudaSetDevice(device));
  amsim_lut* h = new amsim_lut();
  h->m = m;
  h->device = device;
  h->refs = 1;
  const size_t n = (size_t)1 << (2 * m);
  int rc = AMSIM_OK;
  auto bail = [&](cudaError_t e, const char* what) {
    rc = fail(AMSIM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  };
  cudaError_t e = cudaMalloc(&h->d_raw, n);
  if (e != cudaSuccess) bail(e, "cudaMalloc(lut)");
  if (rc == AMSIM_OK) {
    e = cudaMemcpy(h->d_raw, bytes, n, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) bail(e, "cudaMemcpy(lut)");
  }
  if (rc == AMSIM_OK && m <= 7) {
    const int side = 1 << m, stride = side;
    h->enc_bytes = (side * stride + 15) / 16 * 16;
    std::vector<uint8_t> canon(h->enc_bytes, 0), trans(h->enc_bytes, 0);
    bool additive = true;
    for (int a = 0; a < side; ++a)
      for (int b = 0; b < side; ++b) {
        const uint8_t v = encode_entry(bytes[a * side + b], m);
        canon[a * stride + b] = v;
        trans[b * stride + a] = v;
        additive = additive && (int)v == a + b;
      }
    // Mitchell-type tables: (carry << m) + mantissa == i + j everywhere, i.e. the multiplier adds the
    // operands' truncated mantissa fields.  The kernels then skip the table (bit-identical result).
    h->additive = additive && !sw().no_additive;
    e = cudaMalloc(&h->d_canon, h->enc_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_trans, h->enc_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(h->d_canon, canon.data(), h->enc_bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(h->d_trans, trans.data(), h->enc_bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) bail(e, "upload of encoded lut");
  }
  if (rc == AMSIM_OK && m > 7) {
    const size_t side = (size_t)1 << m;
    std::vector<uint8_t> tr(n);
    for (size_t a = 0; a < side; ++a)
      for (size_t b = 0; b < side; ++b) tr[b * side + a] = bytes[a * side + b];
    e = cudaMalloc(&h->d_raw_t, n);
    if (e == cudaSuccess) e = cudaMemcpy(h->d_raw_t, tr.data(), n, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) bail(e, "upload of transposed lut");
  }
  cudaSetDevice(prev);
  if (rc != AMSIM_OK) {
    cudaFree(h->d_raw_t);
    cudaFree(h->d_raw);
    cudaFree(h->d_canon);
    cudaFree(h->d_trans);
    delete h;
    return rc;
  }
  *out = h;
  return AMSIM_OK;
}

int check_common(const amsim_lut* lut, unsigned flags, bool need_gemm) {
  if (!lut) return fail(AMSIM_ERR_INVALID, "lut handle is NULL");
  if (flags & ~(AMSIM_DETERMINISTIC | AMSIM_INT32)) return fail(AMSIM_ERR_INVALID, "unknown flag bits 0x%x", flags);
  (void)need_gemm;
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev != lut->device)
    return fail(AMSIM_ERR_INVALID, "current device %d differs from the LUT's device %d", dev, lut->device);
  return AMSIM_OK;
}

template <typename K>
int ensure_smem(K kernel, size_t bytes, int device) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> done;
  std::lock_guard<std::mutex> lk(mu);
  auto key = std::make_pair((const void*)kernel, device);
  auto it = done.find(key);
  if (it != done.end() && it->second >= bytes) return AMSIM_OK;
  CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  done[key] = bytes;
  return AMSIM_OK;
}

void fill_lut(Params& p, const amsim_lut* lut, bool v_is_first_operand) {
  // The table row is selected by the warp-uniform operand U.  When the lane
  // operand V is the multiplier's first operand (a), U is b: rows indexed by b.
  p.lut = v_is_first_operand ? lut->d_trans : lut->d_canon;
  p.lut_bytes = lut->enc_bytes;
  p.m = lut->m;
  p.mult = 1u << (23 - lut->m);
  p.rowstride = 1u << lut->m;
  p.rmask = ((1u << lut->m) - 1u) << lut->m;
  p.cmask = (1u << lut->m) - 1u;
  p.cadj = (1u << 23) - 128u * p.mult;
  p.lut_mode = lut->direct ? lut->direct
               : lut->wide ? LM_GLOBAL16
               : lut->m > 7 ? LM_GLOBAL : (lut->additive ? LM_ADD : LM_SMEM);
  p.lut_raw = v_is_first_operand ? lut->d_raw_t : lut->d_raw;
  p.v_first = v_is_first_operand ? 1 : 0;
  p.exact_only = sw().exact_only;
  uint32_t al = 16;
  while (al < (uint32_t)lut->enc_bytes) al <<= 1;
  p.lut_align = al;  // m > 7: no table in shared memory (enc_bytes = 0)
}

void fill_gather_divs(Gather& g) {
  g.d_img = make_fastdiv((uint32_t)(g.PH * g.PW));
  g.d_pw = make_fastdiv((uint32_t)g.PW);
  g.d_sc = make_fastdiv((uint32_t)g.SC);
  g.d_kw = make_fastdiv((uint32_t)g.KW);
  g.d_dh = make_fastdiv((uint32_t)g.dil_h);
  g.d_dw = make_fastdiv((uint32_t)g.dil_w);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Resident CTA slots of a 128-thread kernel on the whole device (occupancy x multiprocessors);
// looked up once per kernel, device and shared-memory size.
template <typename Kern>
int resident_slots(Kern kern, size_t smem, int device, int* out) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, int, size_t>, int> known;
  std::lock_guard<std::mutex> lk(mu);
  auto key = std::make_tuple((const void*)kern, device, smem);
  auto it = known.find(key);
  if (it == known.end()) {
    int per_sm = 0, sms = 0;
    CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 128, smem));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    it = known.emplace(key, per_sm * sms).first;
  }
  *out = it->second;
  return AMSIM_OK;
}

// Stream-ordered scratch for the balanced launch, from a memory pool this library creates per
// device (the process-wide default pool is left as the host framework configured it).  The pool
// keeps its freed blocks, so after the first call this neither synchronises nor reaches the
// driver's allocator.
int scratch_alloc(cudaStream_t st, int device, size_t bytes, float** out) {
  static std::mutex mu;
  static std::map<int, cudaMemPool_t> pools;
  cudaMemPool_t pool = nullptr;
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = pools.find(device);
    if (it == pools.end()) {
      cudaMemPoolProps props;
      memset(&props, 0, sizeof(props));
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = device;
      CUDA_TRY(cudaMemPoolCreate(&pool, &props));
      uint64_t keep = ~0ull;
      CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
      pools[device] = pool;
    } else {
      pool = it->second;
    }
  }
  CUDA_TRY(cudaMallocFromPoolAsync(reinterpret_cast<void**>(out), bytes, pool, st));
  return AMSIM_OK;
}

// Scratch of a balanced launch.  Outside a graph capture it is a stream-ordered allocation (safe for
// launches on several streams at once).  While the stream is being captured nothing may be
// allocated, so a capture uses one persistent buffer per device: every eager balanced launch makes
// sure that buffer is at least as large as its own scratch (growing it is the one place where this
// library calls cudaMalloc after a LUT is open; it happens a handful of times, on the first eager
// steps), so a capture that follows a few warm-up steps of the same shapes finds room; a capture that
// does not takes the plain / cluster launch instead.  The nodes of one captured stream run in order,
// so they can share the buffer; graphs that are replayed concurrently on several streams must not
// both contain balanced launches.
struct BalancedScratch {
  float* ws = nullptr;
  bool pooled = false;
};
// The persistent buffer starts with room for the per-tile counters of a launch.  They are zeroed when
// the buffer is created and the CTA that completes a tile puts its counter back to zero, so launches
// inside a captured graph need no memset node.
constexpr size_t kPersistentCounters = 1u << 16;
constexpr size_t kPersistentCounterBytes = kPersistentCounters * sizeof(int);

int balanced_scratch_acquire(cudaStream_t st, int device, size_t bytes, bool capturing, BalancedScratch* out) {
  static std::mutex mu;
  static std::map<int, std::pair<void*, size_t>> persistent;
  out->ws = nullptr;
  out->pooled = false;
  {
    std::lock_guard<std::mutex> lk(mu);
    auto& slot = persistent[device];
    if (capturing) {
      if (slot.first && slot.second >= bytes) out->ws = static_cast<float*>(slot.first);
      return AMSIM_OK;  // ws stays null when there is no room: the caller launches without scratch
    }
    if (slot.second < bytes) {
      void* fresh = nullptr;
      if (cudaMalloc(&fresh, bytes) == cudaSuccess && cudaMemset(fresh, 0, kPersistentCounterBytes) == cudaSuccess) {
        // the old buffer may still be referenced by instantiated graphs: it is kept, not freed
        slot.first = fresh;
        slot.second = bytes;
      } else {
        (void)cudaGetLastError();
      }
    }
  }
  if (scratch_alloc(st, device, bytes, &out->ws) != AMSIM_OK) {
    (void)cudaGetLastError();
    out->ws = nullptr;
    return AMSIM_OK;
  }
  out->pooled = true;
  return AMSIM_OK;
}

cudaError_t balanced_scratch_release(cudaStream_t st, const BalancedScratch& b) {
  return b.pooled ? cudaFreeAsync(b.ws, st) : cudaSuccess;
}

// ---- 16 x 8 / 16 x 9 register-tile filter gradient (amsim_wide.cuh) ---------------------------------
// Measured rate of wide_fgrad relative to fgrad_gemm (time per padded product) on the 3x3
// microbenchmark shapes, used to weigh tile padding against operand-fetch cost.  With a table in
// shared memory it is about 3 % slower per padded product (8 instead of 12 warps per
// multiprocessor hide less lookup latency) and only pays where its 288-row tiles remove padding
// (576 rows: 1.40 -> 1.30 ms); with an additive table (no lookups, issue bound) it is 20-28 % faster.
// The 288-row tile, whose lookups take the table row from a uniform register, is 2 % faster than
// fgrad_gemm when its CTAs fill the device (3x3x256x256: 1.278 -> 1.252 ms) and slower when they
// do not (3x3x512x512, 256 CTAs on 296 slots: +5.6 %).
constexpr double kWideRateTable = 1.03, kWideRateTable9Full = 0.98, kWideRateAdditive = 0.80;

template <bool EXACT, bool VEC, int LM>
int launch_gather_t(cudaStream_t st, Params& p, int batch, int device) {
  using L = SmemLayout<1>;
  const int ptiles = (p.P + L::BP - 1) / L::BP, qtiles = (p.Q + BQ - 1) / BQ;
  const long long ctas = (long long)ptiles * qtiles * batch;
  const int nkb = (p.K + BK - 1) / BK;
  p.ksplit = 1;
  p.tile_bytes = L::TILE_BYTES;
  const size_t smem_plain = LM != LM_SMEM ? (size_t)p.tile_bytes + 16 : L::bytes(p.tile_bytes, p.lut_bytes, p.lut_align);

  // Fast mode, narrow outputs (at most 32 columns: first-layer input gradients, small heads, LeNet-5's
  // convolutions): 2 or 4 warps share each 16-column group and split the reduction steps.
  if constexpr (!EXACT && !lm_direct(LM)) {
    const int qs = p.Q <= 16 ? 4 : p.Q <= 32 ? 2 : 1;
    if (qs > 1 && nkb >= 2 && !sw().no_qsplit) {
      const int qt = (p.Q + BQ / qs - 1) / (BQ / qs);
      if (qs == 4) {
        int rc = ensure_smem(gather_gemm<1, EXACT, VEC, GM_PLAIN, LM, 4>, smem_plain, device);
        if (rc) return rc;
        AMSIM_COUNT_LAUNCH();
        gather_gemm<1, EXACT, VEC, GM_PLAIN, LM, 4><<<dim3(ptiles, qt, batch), L::NT, smem_plain, st>>>(p);
      } else {
        int rc = ensure_smem(gather_gemm<1, EXACT, VEC, GM_PLAIN, LM, 2>, smem_plain, device);
        if (rc) return rc;
        AMSIM_COUNT_LAUNCH();
        gather_gemm<1, EXACT, VEC, GM_PLAIN, LM, 2><<<dim3(ptiles, qt, batch), L::NT, smem_plain, st>>>(p);
      }
      CUDA_TRY(cudaGetLastError());
      return AMSIM_OK;
    }
  }

  // Fast mode, balanced launch: the plain grid would leave the last wave of resident CTA slots
  // partly empty (or never fill them), so the (tile, reduction block) pairs are dealt out in
  // equal runs to exactly as many CTAs as the device holds.  While the stream is being
  // captured into a graph the scratch is a persistent buffer (see balanced_scratch_acquire).
  // (not for tables in global memory: those launches are bound by L2 gathers, and lock-step CTAs
  // measured 50 % slower there)
  if constexpr (!EXACT && !lm_global(LM)) {
    int rc = ensure_smem(gather_gemm<1, EXACT, VEC, GM_BALANCED, LM>, smem_plain, device);
    if (rc) return rc;
    int slots = 0;
    rc = resident_slots(gather_gemm<1, EXACT, VEC, GM_BALANCED, LM>, smem_plain, device, &slots);
    if (rc) return rc;
    const long long iters = ctas * nkb;
    const long long waves = (ctas + slots - 1) / slots;
    const double fill = (double)ctas / (double)(waves * slots);
    // one CTA per resident slot; shorter runs in several waves measured slower (2 waves: +1.5 % on a
    // ResNet-50 step, 6 waves: +4 %): every run parks up to two partial tiles
    long long grid = (long long)slots * (sw().balanced_waves > 0 ? sw().balanced_waves : 1);
    // small problems are latency bound (a lone warp needs ~5 us per reduction block): spread them
    // down to 2 reduction blocks per CTA
    if (iters / grid < 2) grid = iters / 2;
    // measured: pays when the plain grid is at most two waves with a last wave under ~93 % full
    // (one wave at 88 %: -7 %); with more waves the plain grid's tail is already short
    // with long reductions (shape A of the 3x3 microbenchmark: 3.5 waves of 36 blocks) it also pays on
    // larger grids (-2.5 %); with short ones (1x1 layers of 4-8 blocks) the parked partial tiles cost
    // more than the tail (+3-4 %), and so they do with an additive table, whose kernels run 1.5 times
    // as fast (shape A: +6 %)
    int mode = ((waves <= 2 && fill < 0.93) || (LM == LM_SMEM && nkb >= 16 && fill < 0.95)) && grid >= 2 && nkb >= 2;
    if (sw().balanced >= 0) mode = sw().balanced != 0 && grid >= 1;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CUDA_TRY(cudaStreamIsCapturing(st, &cap));
    // Inside a graph capture the tiniest launches (LeNet-5's dense layers: two tiles of 8-16 reduction
    // blocks) take the cluster split below instead, which adds partial tiles through distributed
    // shared memory rather than through parked tiles in global memory: the replayed LeNet-5 step
    // measured 4 % faster that way; anything larger is faster balanced (ResNet-50 +2 %,
    // LeNet-300-100 +3 %; the persistent scratch needs no memset node).
    const bool capturing = cap != cudaStreamCaptureStatusNone;
    bool tiny = ctas * 2 <= slots && nkb >= 4 && iters <= 64;
    if (sw().capture_cluster >= 0) tiny = sw().capture_cluster != 0 && ctas * 2 <= slots && nkb >= 4;
    if (capturing && sw().balanced < 0 && tiny) mode = 0;
    if (mode && slots > 0) {
      p.sk_iters = iters;
      p.sk_ptiles = ptiles;
      p.sk_qtiles = qtiles;
      p.sk_grid = (int)grid;
      const size_t slot_bytes = (size_t)grid * 2 * TR * TC * L::NT * sizeof(float);
      // [counters kept at zero between launches][parked tiles][counters of a launch with more tiles than that]
      const size_t bytes = kPersistentCounterBytes + slot_bytes + (size_t)ctas * sizeof(int);
      BalancedScratch sc;
      rc = balanced_scratch_acquire(st, device, bytes, capturing, &sc);
      if (rc) return rc;
      if (sc.ws) {
        char* base = reinterpret_cast<char*>(sc.ws);
        p.ws = reinterpret_cast<float*>(base + kPersistentCounterBytes);
        const bool clean = !sc.pooled && (size_t)ctas <= kPersistentCounters;  // persistent buffer: zero already
        p.sk_count = reinterpret_cast<int*>(clean ? base : base + kPersistentCounterBytes + slot_bytes);
        fill_bounds(p, device, base, bytes);
        cudaError_t e1 = clean ? cudaSuccess : cudaMemsetAsync(p.sk_count, 0, (size_t)ctas * sizeof(int), st);
        if (e1 == cudaSuccess) {
          AMSIM_COUNT_LAUNCH();
          gather_gemm<1, EXACT, VEC, GM_BALANCED, LM><<<dim3((unsigned)grid), L::NT, smem_plain, st>>>(p);
          e1 = cudaGetLastError();
        }
        cudaError_t e2 = balanced_scratch_release(st, sc);
        p.ws = nullptr;
        p.sk_count = nullptr;
        CUDA_TRY(e1);
        CUDA_TRY(e2);
        return AMSIM_OK;
      }
      // no scratch to be had (pool exhausted, or a capture without a warm-up): the plain grid needs none
      p.ws = nullptr;
    }
  }

  // Fast mode, small launches inside a graph capture: a thread-block cluster of `ksplit` CTAs
  // shares each tile's reduction when the tiles alone cannot fill the resident CTA slots.
  int ksplit = 1;
  if (!EXACT && !lm_global(LM)) {
    const int slots = sm_count(device) * AMSIM_CTAS1;
    while (ksplit < 8 && ctas * (ksplit * 2) <= slots && nkb / (ksplit * 2) >= 2) ksplit *= 2;
    if (sw().force_ksplit >= 0) ksplit = sw().force_ksplit > 0 ? sw().force_ksplit : 1;
  }
  p.ksplit = ksplit;
  if (ksplit > 1 && L::EXCHANGE_BYTES > p.tile_bytes) p.tile_bytes = L::EXCHANGE_BYTES;
  const size_t smem = LM != LM_SMEM ? (size_t)p.tile_bytes + 16 : L::bytes(p.tile_bytes, p.lut_bytes, p.lut_align);
  if (ksplit == 1) {
    int rc = ensure_smem(gather_gemm<1, EXACT, VEC, GM_PLAIN, LM>, smem, device);
    if (rc) return rc;
    AMSIM_COUNT_LAUNCH();
    gather_gemm<1, EXACT, VEC, GM_PLAIN, LM><<<dim3(ptiles, qtiles, batch), L::NT, smem, st>>>(p);
    CUDA_TRY(cudaGetLastError());
    return AMSIM_OK;
  }
  constexpr int kClusterMode = (!EXACT && !lm_global(LM)) ? GM_CLUSTER : GM_PLAIN;
  int rc = ensure_smem(gather_gemm<1, EXACT, VEC, kClusterMode, LM>, smem, device);
  if (rc) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(ptiles * ksplit, qtiles, batch);
  cfg.blockDim = dim3(L::NT, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = ksplit;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  AMSIM_COUNT_LAUNCH();
  CUDA_TRY(cudaLaunchKernelEx(&cfg, gather_gemm<1, EXACT, VEC, kClusterMode, LM>, p));
  return AMSIM_OK;
}
int launch_gather(cudaStream_t st, Params& p, int batch, bool exact, int device) {
  if (p.P <= 0 || p.Q <= 0 || batch <= 0) return AMSIM_OK;  // nothing to compute
  fill_bounds(p, device, nullptr, 0);
  if ((long long)p.P >= (1ll << 31) - 256) return fail(AMSIM_ERR_UNSUPPORTED, "more than 2^31 output rows");
  const bool vec = !p.v_trans && (p.g.SC % 4 == 0) && aligned16(p.V) && (p.v_bs % 4 == 0);
  // U by 128-bit loads along its contiguous index when four elements are always one aligned
  // group inside one tap: along q (weights of a forward convolution / dense layer / matmul B),
  // or along k (flipped filter of an input gradient, transposed matmul B)
  p.u_vec = 0;
  if (aligned16(p.U) && p.u_bs % 4 == 0 && p.u_tap % 4 == 0 && !sw().no_uvec) {
    if (p.u_sq == 1 && p.u_sk % 4 == 0 && p.Q % 4 == 0) p.u_vec = 1;
    else if (p.u_sk == 1 && p.u_sq % 4 == 0 && p.g.SC % 4 == 0) p.u_vec = 2;
  }
#define AMSIM_GO(EX_, VEC_, LM_) return launch_gather_t<EX_, VEC_, LM_>(st, p, batch, device)
#define AMSIM_GO_LM(LM_)                                                                        \
  do {                                                                                          \
    if (exact) { if (vec) AMSIM_GO(true, true, LM_); else AMSIM_GO(true, false, LM_); }         \
    else       { if (vec) AMSIM_GO(false, true, LM_); else AMSIM_GO(false, false, LM_); }       \
  } while (0)
  // direct models: per-product arithmetic dominates; one kernel flavour (ordered chains) serves both modes
  if (p.lut_mode == LM_DIRECT_MBM) { if (vec) AMSIM_GO(true, true, LM_DIRECT_MBM); else AMSIM_GO(true, false, LM_DIRECT_MBM); }
  if (p.lut_mode == LM_DIRECT_MIT) { if (vec) AMSIM_GO(true, true, LM_DIRECT_MIT); else AMSIM_GO(true, false, LM_DIRECT_MIT); }
  if (p.lut_mode == LM_ADD) AMSIM_GO_LM(LM_ADD);
  if (p.lut_mode == LM_GLOBAL) AMSIM_GO_LM(LM_GLOBAL);
  if (p.lut_mode == LM_GLOBAL16) AMSIM_GO_LM(LM_GLOBAL16);
  AMSIM_GO_LM(LM_SMEM);
#undef AMSIM_GO_LM
#undef AMSIM_GO
}

struct FgradPlan {
  int np;  // rows per lane of the tile: 0 = the 128-row kernels, 8 / 9 = wide_fgrad
  int splits, k_chunk;
  int thin, tq;  // one-to-four-chains-per-thread kernel instead of the 128 x 64 tiles
  size_t ws_bytes;
};

// Rows per lane a fast-mode filter gradient of P x Q outputs takes if its operands allow the wide
// kernel (128-bit gathers; `additive`: the table is additive, else it sits in shared memory): the
// tile height with the least padded work, weighted by the kernels' measured rates.  0 = the
// 128-row kernel.
FgradPlan plan_fgrad(int P, int Q, int K, bool exact, int np, int sms);

int pick_fgrad_rows(int P, int Q, int K, int sms, bool additive, bool vec) {
  if (sw().wide == 0) return 0;
  auto padded = [&](int bp) { return (double)(((long long)P + bp - 1) / bp) * bp; };
  if (!vec) {
    // no 128-bit gathers (channel count no multiple of 4): the 160-row tile with element-wise staging,
    // where it has clearly less padded work than the 128-row tiles and the reduction is long
    if (sw().wide < 0 && padded(160) > 0.85 * padded(128)) return 0;
    const long long tiles5 = (((long long)P + 159) / 160) * (((long long)Q + BQ - 1) / BQ);
    if (sw().wide < 0 && tiles5 * (((long long)K + BK - 1) / BK) < 8ll * 3 * sms) return 0;
    return 5;
  }
  int best = 8;
  double cost = padded(256);
  if (padded(288) <= cost) { best = 9; cost = padded(288); }
  if (sw().wide > 0) return best;
  const long long tiles = (((long long)P + 32 * best - 1) / (32 * best)) * (((long long)Q + BQ - 1) / BQ);
  double rate = additive ? kWideRateAdditive : kWideRateTable;
  if (!additive && best == 9 && (double)tiles * plan_fgrad(P, Q, K, false, 9, sms).splits >= 0.95 * 2 * sms)
    rate = kWideRateTable9Full;
  if (cost * rate >= padded(128)) return 0;
  if (tiles * (((long long)K + BK - 1) / BK) < 8ll * 2 * sms) return 0;  // too small to fill the device a few times over
  return best;
}

// How a filter / weight gradient of P x Q outputs over a reduction of K runs.  Depends on the
// dimensions, the mode, the device's multiprocessor count and the debug switches (read once) only,
// so the *_workspace functions and the launch agree.
FgradPlan plan_fgrad(int P, int Q, int K, bool exact, int np, int sms) {
  FgradPlan f;
  f.np = exact ? 0 : np;
  const int bp = f.np ? 32 * f.np : 128;
  const int slots = sms * (f.np >= 8 ? 2 : AMSIM_CTAS1);  // resident CTAs on the whole GPU (launch bounds of the kernels)
  const long long tiles = (((long long)P + bp - 1) / bp) * (((long long)Q + BQ - 1) / BQ);
  const long long chains = (long long)P * Q;
  f.thin = 0;
  f.tq = 1;
  int splits = 1;
  if (exact) {
    // Deterministic mode cannot split a reduction; when the 128 x 64 tiles would fill less than
    // half of the resident CTA slots, threads take fewer chains each so the whole device works.
    f.thin = tiles * 2 < slots;
    if (sw().thin_fgrad >= 0) f.thin = sw().thin_fgrad != 0;
    f.tq = chains >= 4ll * 32 * 4 * sms * 2 ? 4 : chains >= 2ll * 32 * 4 * sms * 2 ? 2 : 1;
    if (sw().thin_tq > 0) f.tq = sw().thin_tq;
  } else if (tiles > 0) {
    // Fast mode, tiny outputs (LeNet-5's 5x5x1x6 filter: 150 of a tile's 8192 outputs): one chain per
    // thread over a slice of the reduction wastes nothing on padding; many slices, summed in order.
    f.thin = !f.np && (double)chains < 0.2 * (double)(tiles * bp * BQ);
    if (sw().thin_fast >= 0 && !f.np) f.thin = sw().thin_fast != 0;
    if (f.thin) {
      const int nw = ((long long)Q + f.tq - 1) / f.tq > 4 ? 16 : 4;
      const long long ctas = (((long long)P + 31) / 32) * (((long long)Q + nw * f.tq - 1) / (nw * f.tq));
      splits = (int)(4 * sms / ctas);
      const int max_splits = (int)(((long long)K + 2 * BK - 1) / (2 * BK));  // at least 2 stages per split
      if (splits > max_splits) splits = max_splits;
    } else {
      // one balanced wave: as many splits as fit in the resident slots
      splits = (int)(slots / tiles);
      const int max_splits = (int)(((long long)K + 4 * BK - 1) / (4 * BK));  // at least 4 stages per split
      if (splits > max_splits) splits = max_splits;
    }
    if (splits < 1) splits = 1;
  }
  long long chunk = ((long long)K + splits - 1) / splits;
  chunk = (chunk + BK - 1) / BK * BK;
  if (chunk < BK) chunk = BK;
  f.k_chunk = (int)chunk;
  f.splits = K > 0 ? (int)(((long long)K + chunk - 1) / chunk) : 1;
  f.ws_bytes = f.splits > 1 ? (size_t)f.splits * P * Q * sizeof(float) : 0;
  return f;
}

// Workspace that covers whichever plan the launch takes (the wide kernel needs operands the
// query cannot see: 16-byte aligned tensors, a table in shared memory).
size_t fgrad_workspace(int P, int Q, int K, bool exact, int sms) {
  size_t need = plan_fgrad(P, Q, K, exact, 0, sms).ws_bytes;
  if (!exact) {
    for (int additive = 0; additive < 2; ++additive) {
      for (int vec = 0; vec < 2; ++vec) {
        const int np = pick_fgrad_rows(P, Q, K, sms, additive != 0, vec != 0);
        if (np) need = std::max(need, plan_fgrad(P, Q, K, false, np, sms).ws_bytes);
      }
    }
  }
  return need;
}

template <int LM, int NP>
int launch_wide_fgrad_t(cudaStream_t st, Params& p, int device) {
  constexpr bool VEC = NP != 5;
  p.tile_bytes = wide_tile_bytes(NP);
  const size_t smem = LM != LM_SMEM ? (size_t)p.tile_bytes + 16 : (size_t)p.tile_bytes + p.lut_align + p.lut_bytes;
  int rc = ensure_smem(wide_fgrad<LM, NP, VEC>, smem, device);
  if (rc) return rc;
  dim3 grid((p.P + 32 * NP - 1) / (32 * NP), (p.Q + BQ - 1) / BQ, p.splits);
  AMSIM_COUNT_LAUNCH();
  wide_fgrad<LM, NP, VEC><<<grid, WNT, smem, st>>>(p);
  CUDA_TRY(cudaGetLastError());
  if (p.splits > 1) {
    const long long n = (long long)p.P * p.Q;
    const int lanes = reduce_lanes(p.splits);
    AMSIM_COUNT_LAUNCH();
    reduce_splits<<<reduce_blocks(n, lanes), 256, 0, st>>>(p.ws, p.O, n, p.splits, p.Q, p.o_sp, p.o_sq, lanes);
    CUDA_TRY(cudaGetLastError());
  }
  return AMSIM_OK;
}

template <bool EXACT, bool VEC, int LM>
int launch_fgrad_t(cudaStream_t st, const Params& p, int device) {
  using L = SmemLayout<1>;
  const size_t smem = LM != LM_SMEM ? (size_t)L::TILE_BYTES + 16 : L::bytes(L::TILE_BYTES, p.lut_bytes, p.lut_align);
  int rc = ensure_smem(fgrad_gemm<1, EXACT, VEC, LM>, smem, device);
  if (rc) return rc;
  dim3 grid((p.P + L::BP - 1) / L::BP, (p.Q + BQ - 1) / BQ, p.splits);
  AMSIM_COUNT_LAUNCH();
  fgrad_gemm<1, EXACT, VEC, LM><<<grid, L::NT, smem, st>>>(p);
  CUDA_TRY(cudaGetLastError());
  if (p.splits > 1) {
    const long long n = (long long)p.P * p.Q;
    const int lanes = reduce_lanes(p.splits);
    AMSIM_COUNT_LAUNCH();
    reduce_splits<<<reduce_blocks(n, lanes), 256, 0, st>>>(p.ws, p.O, n, p.splits, p.Q, p.o_sp, p.o_sq, lanes);
    CUDA_TRY(cudaGetLastError());
  }
  return AMSIM_OK;
}

template <int TQ, int NW, int LM, bool FLUSH>
int launch_fgrad_thin_t(cudaStream_t st, Params& p, int device) {
  p.tile_bytes = (2 * THIN_BK * 32 + 2 * THIN_BK * NW * TQ) * 4;
  const size_t smem = LM != LM_SMEM ? (size_t)p.tile_bytes + 16 : (size_t)p.tile_bytes + p.lut_align + p.lut_bytes;
  int rc = ensure_smem(fgrad_exact_thin<TQ, NW, LM, FLUSH>, smem, device);
  if (rc) return rc;
  dim3 grid((p.P + 31) / 32, (p.Q + NW * TQ - 1) / (NW * TQ), p.splits);
  AMSIM_COUNT_LAUNCH();
  fgrad_exact_thin<TQ, NW, LM, FLUSH><<<grid, 32 * NW, smem, st>>>(p);
  CUDA_TRY(cudaGetLastError());
  if (p.splits > 1) {
    const long long n = (long long)p.P * p.Q;
    const int lanes = reduce_lanes(p.splits);
    AMSIM_COUNT_LAUNCH();
    reduce_splits<<<reduce_blocks(n, lanes), 256, 0, st>>>(p.ws, p.O, n, p.splits, p.Q, p.o_sp, p.o_sq, lanes);
    CUDA_TRY(cudaGetLastError());
  }
  return AMSIM_OK;
}
template <int LM>
int launch_fgrad_chain(cudaStream_t st, Params& p, int device) {
  p.tile_bytes = (2 * BK * 32 + 2 * BK * CHAIN_Q) * 4 + 2 * BK * CHAIN_Q * 32 * 4;
  const size_t smem = LM != LM_SMEM ? (size_t)p.tile_bytes + 16 : (size_t)p.tile_bytes + p.lut_align + p.lut_bytes;
  int rc = ensure_smem(fgrad_exact_chain<LM>, smem, device);
  if (rc) return rc;
  dim3 grid((p.P + 31) / 32, (p.Q + CHAIN_Q - 1) / CHAIN_Q, 1);
  AMSIM_COUNT_LAUNCH();
  fgrad_exact_chain<LM><<<grid, 768, smem, st>>>(p);
  CUDA_TRY(cudaGetLastError());
  return AMSIM_OK;
}

template <int LM>
int launch_fgrad_thin(cudaStream_t st, Params& p, int tq, bool flush, int device) {
  // 16 warps per CTA share one staged V tile when the output is wide enough to use them
  const bool wide = (p.Q + tq - 1) / tq > 4 && !sw().thin_narrow;
  if (flush) {  // fast mode: tiny outputs only, one chain per thread
    if constexpr (lm_direct(LM)) return fail(AMSIM_ERR_UNSUPPORTED, "direct models run in ordered mode");
    else return wide ? launch_fgrad_thin_t<1, 16, LM, true>(st, p, device) : launch_fgrad_thin_t<1, 4, LM, true>(st, p, device);
  }
  if (tq == 4) return wide ? launch_fgrad_thin_t<4, 16, LM, false>(st, p, device) : launch_fgrad_thin_t<4, 4, LM, false>(st, p, device);
  if (tq == 2) return wide ? launch_fgrad_thin_t<2, 16, LM, false>(st, p, device) : launch_fgrad_thin_t<2, 4, LM, false>(st, p, device);
  return wide ? launch_fgrad_thin_t<1, 16, LM, false>(st, p, device) : launch_fgrad_thin_t<1, 4, LM, false>(st, p, device);
}

int launch_fgrad(cudaStream_t st, Params& p, bool exact, void* ws, size_t ws_bytes, int device) {
  if (p.P <= 0 || p.Q <= 0) return AMSIM_OK;
  if (lm_direct(p.lut_mode)) exact = true;  // one kernel flavour for the direct models: ordered chains
  const int sms = sm_count(device);
  const bool vec = (p.g.SC % 4 == 0) && aligned16(p.V);
  FgradPlan f = plan_fgrad(p.P, p.Q, p.K, exact, 0, sms);
  if (!exact && !f.thin && (p.lut_mode == LM_SMEM || p.lut_mode == LM_ADD)) {
    const int np = pick_fgrad_rows(p.P, p.Q, p.K, sms, p.lut_mode == LM_ADD, vec);
    if (np) f = plan_fgrad(p.P, p.Q, p.K, false, np, sms);
  }
  if (f.ws_bytes > 0) {
    if (!ws || ws_bytes < f.ws_bytes)
      return fail(AMSIM_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", f.ws_bytes, ws ? ws_bytes : (size_t)0);
    if (!aligned16(ws)) return fail(AMSIM_ERR_WORKSPACE, "workspace must be 16-byte aligned");
  }
  p.splits = f.splits;
  p.k_chunk = f.k_chunk;
  p.ws = static_cast<float*>(ws);
  fill_bounds(p, device, ws, f.ws_bytes);
  if (f.np) {
    p.u_vec = aligned16(p.U) && p.u_sq == 1 && p.u_sk % 4 == 0 && p.Q % 4 == 0 && !sw().no_uvec;
    if (p.lut_mode == LM_ADD)
      return f.np == 9   ? launch_wide_fgrad_t<LM_ADD, 9>(st, p, device)
             : f.np == 8 ? launch_wide_fgrad_t<LM_ADD, 8>(st, p, device)
                         : launch_wide_fgrad_t<LM_ADD, 5>(st, p, device);
    return f.np == 9   ? launch_wide_fgrad_t<LM_SMEM, 9>(st, p, device)
           : f.np == 8 ? launch_wide_fgrad_t<LM_SMEM, 8>(st, p, device)
                       : launch_wide_fgrad_t<LM_SMEM, 5>(st, p, device);
  }
  if (f.thin) {
    {
      const int tq = f.tq;
      const bool flush = !exact;
      // deterministic, few chains and a long reduction: products in parallel, additions in order
      int chain = exact && (long long)p.P * p.Q <= 2ll * sms * 256 && p.K >= 64 * BK;
      if (sw().chain_fgrad >= 0) chain = exact && sw().chain_fgrad != 0;
      if (chain) {
        if (p.lut_mode == LM_DIRECT_MBM) return launch_fgrad_chain<LM_DIRECT_MBM>(st, p, device);
        if (p.lut_mode == LM_DIRECT_MIT) return launch_fgrad_chain<LM_DIRECT_MIT>(st, p, device);
        if (p.lut_mode == LM_ADD) return launch_fgrad_chain<LM_ADD>(st, p, device);
        if (p.lut_mode == LM_GLOBAL) return launch_fgrad_chain<LM_GLOBAL>(st, p, device);
        if (p.lut_mode == LM_GLOBAL16) return launch_fgrad_chain<LM_GLOBAL16>(st, p, device);
        return launch_fgrad_chain<LM_SMEM>(st, p, device);
      }
      if (p.lut_mode == LM_DIRECT_MBM) return launch_fgrad_thin<LM_DIRECT_MBM>(st, p, tq, flush, device);
      if (p.lut_mode == LM_DIRECT_MIT) return launch_fgrad_thin<LM_DIRECT_MIT>(st, p, tq, flush, device);
      if (p.lut_mode == LM_ADD) return launch_fgrad_thin<LM_ADD>(st, p, tq, flush, device);
      if (p.lut_mode == LM_GLOBAL) return launch_fgrad_thin<LM_GLOBAL>(st, p, tq, flush, device);
      if (p.lut_mode == LM_GLOBAL16) return launch_fgrad_thin<LM_GLOBAL16>(st, p, tq, flush, device);
      return launch_fgrad_thin<LM_SMEM>(st, p, tq, flush, device);
    }
  }
  p.u_vec = aligned16(p.U) && p.u_sq == 1 && p.u_sk % 4 == 0 && p.Q % 4 == 0 && !sw().no_uvec;
#define AMSIM_GO(EX_, VEC_, LM_) return launch_fgrad_t<EX_, VEC_, LM_>(st, p, device)
#define AMSIM_GO_LM(LM_)                                                                        \
  do {                                                                                          \
    if (exact) { if (vec) AMSIM_GO(true, true, LM_); else AMSIM_GO(true, false, LM_); }         \
    else       { if (vec) AMSIM_GO(false, true, LM_); else AMSIM_GO(false, false, LM_); }       \
  } while (0)
  if (p.lut_mode == LM_DIRECT_MBM) { if (vec) AMSIM_GO(true, true, LM_DIRECT_MBM); else AMSIM_GO(true, false, LM_DIRECT_MBM); }
  if (p.lut_mode == LM_DIRECT_MIT) { if (vec) AMSIM_GO(true, true, LM_DIRECT_MIT); else AMSIM_GO(true, false, LM_DIRECT_MIT); }
  if (p.lut_mode == LM_ADD) AMSIM_GO_LM(LM_ADD);
  if (p.lut_mode == LM_GLOBAL) AMSIM_GO_LM(LM_GLOBAL);
  if (p.lut_mode == LM_GLOBAL16) AMSIM_GO_LM(LM_GLOBAL16);
  AMSIM_GO_LM(LM_SMEM);
#undef AMSIM_GO_LM
#undef AMSIM_GO
}

// T = int32: one thread per output on the raw table (see naive_*_i32).
int launch_naive_i32(cudaStream_t st, Params& p, const amsim_lut* lut, bool fgrad) {
  if (p.P <= 0 || p.Q <= 0) return AMSIM_OK;
  if (lut->direct) return fail(AMSIM_ERR_UNSUPPORTED, "the direct 32-bit models are FP32 only");
  if (lut->wide) return fail(AMSIM_ERR_UNSUPPORTED, "tables of 16-bit entries are FP32 only");
  p.lut_raw = lut->d_raw;  // rows by the first operand; v_first tells the kernel which operand that is
  const long long n = (long long)p.P * p.Q;
  const unsigned blocks = (unsigned)((n + 127) / 128);
  AMSIM_COUNT_LAUNCH();
  if (fgrad)
    naive_fgrad_i32<<<blocks, 128, 0, st>>>(p);
  else
    naive_gather_i32<<<blocks, 128, 0, st>>>(p);
  CUDA_TRY(cudaGetLastError());
  return AMSIM_OK;
}

// a * b * c < lim for non-negative ints, without overflowing
inline bool prod3_below(long long a, long long b, long long c, long long lim) {
  if (a == 0 || b == 0 || c == 0) return lim > 0;
  if (a >= lim || b >= lim || c >= lim) return false;
  const long long ab = a * b;  // < lim^2 <= 2^62
  if (ab >= lim) return false;
  return ab * c < lim;         // < lim^2
}

int check_conv_dims(int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h, int out_w,
                    int stride_h, int stride_w, int pad_top, int pad_left) {
  if (batch < 0 || in_h <= 0 || in_w <= 0 || in_c <= 0 || f_h <= 0 || f_w <= 0 || out_c <= 0 || out_h < 0 ||
      out_w < 0 || stride_h <= 0 || stride_w <= 0 || pad_top < 0 || pad_left < 0)
    return fail(AMSIM_ERR_INVALID, "convolution dimensions must be positive (strides > 0, pads >= 0)");
  if (!prod3_below(f_h, f_w, in_c > out_c ? in_c : out_c, 1ll << 30))
    return fail(AMSIM_ERR_UNSUPPORTED, "reduction length exceeds 2^30");
  if (!prod3_below(batch, in_h, in_w, (1ll << 31) - 256) || !prod3_below(batch, out_h, out_w, (1ll << 31) - 256))
    return fail(AMSIM_ERR_UNSUPPORTED, "more than 2^31 pixels");
  return AMSIM_OK;
}

}  // namespace

extern "C" {

const char* amsim_last_error(void) { return g_err; }

const char* amsim_version(void) { return "amsim 0.1 (sm_100a)"; }

unsigned long long amsim_debug_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int amsim_debug_bounds_report(unsigned long long* word) {
  if (word) *word = 0;
#ifdef AMSIM_BOUNDS_CHECK
  unsigned long long* w = bounds_word(current_device());
  if (!w) return fail(AMSIM_ERR_CUDA, "no bounds-report word on this device");
  CUDA_TRY(cudaDeviceSynchronize());
  unsigned long long v = 0;
  CUDA_TRY(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaMemset(w, 0, sizeof(v)));
  if (word) *word = v;
  return AMSIM_OK;
#else
  return fail(AMSIM_ERR_UNSUPPORTED, "this library was built without -DAMSIM_BOUNDS_CHECK");
#endif
}

void amsim_debug_reload_env(void) {
  sw();  // make sure the one-time load has happened, then replace its result
  load_switches();
}

uint32_t amsim_debug_fastdiv(uint32_t n, uint32_t d) { return fdiv(n, make_fastdiv(d)); }

int amsim_lut_open_bytes(const uint8_t* bytes, int m, int device, amsim_lut** out) {
  if (!bytes || !out) return fail(AMSIM_ERR_INVALID, "NULL argument");
  if (m < 1 || m > 11) return fail(AMSIM_ERR_LUT_NAME, "mantissa width %d outside 1..11", m);
  return upload_lut(bytes, m, device, out);
}

int amsim_lut_open(const char* path, int device, amsim_lut** out) {
  if (!path || !out) return fail(AMSIM_ERR_INVALID, "NULL argument");
  if (!*path) return fail(AMSIM_ERR_LUT_NAME, "no mant lut file name given");
  if (strncmp(path, "direct:", 7) == 0) {
    // mantissa width 23: the reference's direct C simulation instead of a table (README.md:107)
    int kind = 0;
    if (strcmp(path + 7, "MBM32") == 0) kind = LM_DIRECT_MBM;
    else if (strcmp(path + 7, "MIT32") == 0) kind = LM_DIRECT_MIT;
    else return fail(AMSIM_ERR_LUT_NAME, "unknown direct multiplier '%s' (direct:MBM32, direct:MIT32)", path + 7);
    const std::string key = std::string(path) + "@" + std::to_string(device);
    std::lock_guard<std::mutex> lk(g_lut_mu);
    auto it = g_lut_cache.find(key);
    if (it != g_lut_cache.end()) {
      it->second->refs++;
      *out = it->second;
      return AMSIM_OK;
    }
    int ndev = 0;
    CUDA_TRY(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(AMSIM_ERR_INVALID, "device %d out of range", device);
    amsim_lut* h = new amsim_lut();
    h->m = 23;
    h->device = device;
    h->refs = 1;
    h->direct = kind;
    h->key = key;
    g_lut_cache[key] = h;
    *out = h;
    return AMSIM_OK;
  }
  const int m = parse_mant_width(path);
  if (m < 0) return fail(AMSIM_ERR_LUT_NAME, "cannot take a mantissa width in 1..11 from '%s' (expected <MODEL>_<m>.bin)", path);
  char real[PATH_MAX];
  if (!realpath(path, real)) return fail(AMSIM_ERR_LUT_IO, "lut file '%s' cannot be opened", path);
  const std::string key = std::string(real) + "@" + std::to_string(device);
  std::lock_guard<std::mutex> lk(g_lut_mu);
  auto it = g_lut_cache.find(key);
  if (it != g_lut_cache.end()) {
    it->second->refs++;
    *out = it->second;
    return AMSIM_OK;
  }
  FILE* f = fopen(real, "rb");
  if (!f) return fail(AMSIM_ERR_LUT_IO, "lut file '%s' cannot be opened", path);
  const size_t want = (size_t)1 << (2 * m);
  std::vector<uint8_t> buf(2 * want + 2);
  const size_t got = fread(buf.data(), 1, 2 * want + 1, f);
  fclose(f);
  // exactly 2^(2m) bytes: the reference's format; exactly twice that: 16-bit little-endian entries
  if (got != want && got != 2 * want)
    return fail(AMSIM_ERR_LUT_SIZE, "lut file '%s' holds %s%zu bytes, m = %d needs exactly %zu (or %zu for 16-bit entries)",
                path, got > 2 * want ? "more than " : "", got > 2 * want ? 2 * want : got, m, want, 2 * want);
  amsim_lut* h = nullptr;
  int rc;
  if (got == 2 * want) {
    std::vector<uint16_t> wide(want);
    for (size_t i = 0; i < want; ++i) wide[i] = (uint16_t)(buf[2 * i] | (buf[2 * i + 1] << 8));
    rc = upload_lut16(wide.data(), m, device, &h);
  } else {
    rc = upload_lut(buf.data(), m, device, &h);
  }
  if (rc) return rc;
  h->key = key;
  g_lut_cache[key] = h;
  *out = h;
  return AMSIM_OK;
}

int amsim_lut_close(amsim_lut* lut) {
  if (!lut) return AMSIM_OK;
  std::lock_guard<std::mutex> lk(g_lut_mu);
  if (--lut->refs > 0) return AMSIM_OK;
  if (!lut->key.empty()) g_lut_cache.erase(lut->key);
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(lut->device);
  cudaFree(lut->d_raw);
  cudaFree(lut->d_raw_t);
  cudaFree(lut->d_canon);
  cudaFree(lut->d_trans);
  cudaSetDevice(prev);
  delete lut;
  return AMSIM_OK;
}

int amsim_lut_info(const amsim_lut* lut, int* mant_width, uint32_t* mant_mask, int* a_shift, int* b_shift,
                   const uint8_t** device_bytes) {
  if (!lut) return fail(AMSIM_ERR_INVALID, "lut handle is NULL");
  if (mant_width) *mant_width = lut->m;
  if (mant_mask) *mant_mask = ((1u << lut->m) - 1u) << (23 - lut->m);  // approx_mul_lut.h:28
  if (a_shift) *a_shift = lut->direct ? 0 : 23 - 2 * lut->m;           // :26
  if (b_shift) *b_shift = 23 - lut->m;                                 // :27
  if (device_bytes) *device_bytes = lut->d_raw;
  return AMSIM_OK;
}

int amsim_mul(void* stream, const amsim_lut* lut, const float* a, const float* b, float* out, size_t n) {
  int rc = check_common(lut, 0, false);
  if (rc) return rc;
  if (n == 0) return AMSIM_OK;
  if (!a || !b || !out) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  size_t blocks = (n + 255) / 256;
  const size_t cap = (size_t)sm_count(lut->device) * 16;
  if (blocks > cap) blocks = cap;
  AMSIM_COUNT_LAUNCH();
  mul_elementwise<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a, b, out, n, lut->d_raw, lut->m, lut->direct ? lut->direct : lut->wide ? LM_GLOBAL16 : 0);
  CUDA_TRY(cudaGetLastError());
  return AMSIM_OK;
}

int amsim_conv2d_geometry(int in_h, int in_w, int f_h, int f_w, int stride_h, int stride_w, int same, int* out_h,
                          int* out_w, int* pad_top, int* pad_left) {
  if (in_h <= 0 || in_w <= 0 || f_h <= 0 || f_w <= 0 || stride_h <= 0 || stride_w <= 0)
    return fail(AMSIM_ERR_INVALID, "geometry arguments must be positive");
  auto one = [&](int in, int f, int s, int* o, int* pb) -> int {
    if (same) {
      *o = (in + s - 1) / s;
      int total = (*o - 1) * s + f - in;
      *pb = total > 0 ? total / 2 : 0;
    } else {
      if (in < f) return 1;
      *o = (in - f + s) / s;
      *pb = 0;
    }
    return 0;
  };
  int oh, ow, pt, pl;
  if (one(in_h, f_h, stride_h, &oh, &pt) || one(in_w, f_w, stride_w, &ow, &pl))
    return fail(AMSIM_ERR_INVALID, "VALID padding needs the filter to fit inside the input");
  if (out_h) *out_h = oh;
  if (out_w) *out_w = ow;
  if (pad_top) *pad_top = pt;
  if (pad_left) *pad_left = pl;
  return AMSIM_OK;
}

static void dense_gather(Gather& g, int width);

static int conv2d_fwd_impl(void* stream, const amsim_lut* lut, const float* x, const float* w, const float* scale,
                           const float* bias, float* y, int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h,
                           int out_w, int stride_h, int stride_w, int pad_top, int pad_left, int act, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  if (act != AMSIM_ACT_NONE && act != AMSIM_ACT_RELU) return fail(AMSIM_ERR_INVALID, "unknown activation %d", act);
  if ((bias || scale || act) && (flags & AMSIM_INT32)) return fail(AMSIM_ERR_UNSUPPORTED, "the fused epilogue is FP32 only");
  rc = check_conv_dims(batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w, stride_h, stride_w, pad_top, pad_left);
  if (rc) return rc;
  if (batch == 0 || out_h == 0 || out_w == 0) return AMSIM_OK;
  if (!x || !w || !y) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  Params p{};
  p.V = x; p.U = w; p.O = y;
  p.v_elems = (long long)batch * in_h * in_w * in_c; p.u_elems = (long long)f_h * f_w * in_c * out_c;
  p.o_elems = (long long)batch * out_h * out_w * out_c;
  p.P = batch * out_h * out_w; p.Q = out_c; p.K = f_h * f_w * in_c;
  Gather& g = p.g;
  g.PH = out_h; g.PW = out_w; g.ps_h = stride_h; g.ps_w = stride_w; g.off_t = pad_top; g.off_l = pad_left;
  g.lim_h = in_h; g.lim_w = in_w; g.dil_h = 1; g.dil_w = 1; g.SH = in_h; g.SW = in_w; g.SC = in_c; g.KW = f_w;
  fill_gather_divs(g);
  if (f_h == 1 && f_w == 1 && stride_h == 1 && stride_w == 1 && pad_top == 0 && pad_left == 0 && out_h == in_h &&
      out_w == in_w)
    dense_gather(g, in_c);  // a plain GEMM over the pixels: no pixel -> (image, row, column) arithmetic
  p.u_t0 = 0; p.u_tj = f_w; p.u_ti = 1; p.u_tap = (long long)in_c * out_c; p.u_sk = out_c; p.u_sq = 1;
  p.o_sp = out_c; p.o_sq = 1;
  fill_lut(p, lut, /*v_is_first_operand=*/true);
  p.bias = bias;
  p.scale = scale;
  p.relu = act == AMSIM_ACT_RELU;
  if (flags & AMSIM_INT32) return launch_naive_i32((cudaStream_t)stream, p, lut, false);
  return launch_gather((cudaStream_t)stream, p, 1, flags & AMSIM_DETERMINISTIC, lut->device);
}

int amsim_conv2d_fwd(void* stream, const amsim_lut* lut, const float* x, const float* w, float* y, int batch, int in_h,
                     int in_w, int in_c, int f_h, int f_w, int out_c, int out_h, int out_w, int stride_h, int stride_w,
                     int pad_top, int pad_left, unsigned flags) {
  return conv2d_fwd_impl(stream, lut, x, w, nullptr, nullptr, y, batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w,
                         stride_h, stride_w, pad_top, pad_left, AMSIM_ACT_NONE, flags);
}

int amsim_conv2d_fwd_bias_act(void* stream, const amsim_lut* lut, const float* x, const float* w, const float* bias,
                              float* y, int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h,
                              int out_w, int stride_h, int stride_w, int pad_top, int pad_left, int act,
                              unsigned flags) {
  return conv2d_fwd_impl(stream, lut, x, w, nullptr, bias, y, batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w,
                         stride_h, stride_w, pad_top, pad_left, act, flags);
}

int amsim_conv2d_fwd_scale_bias_act(void* stream, const amsim_lut* lut, const float* x, const float* w,
                                    const float* scale, const float* bias, float* y, int batch, int in_h, int in_w,
                                    int in_c, int f_h, int f_w, int out_c, int out_h, int out_w, int stride_h,
                                    int stride_w, int pad_top, int pad_left, int act, unsigned flags) {
  return conv2d_fwd_impl(stream, lut, x, w, scale, bias, y, batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w,
                         stride_h, stride_w, pad_top, pad_left, act, flags);
}

int amsim_conv2d_bwd_input(void* stream, const amsim_lut* lut, const float* w, const float* dy, float* dx, int batch,
                           int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h, int out_w,
                           int stride_h, int stride_w, int pad_top, int pad_left, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  rc = check_conv_dims(batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w, stride_h, stride_w, pad_top, pad_left);
  if (rc) return rc;
  if (batch == 0) return AMSIM_OK;
  if (!dy || !w || !dx) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  if (out_h == 0 || out_w == 0) return fail(AMSIM_ERR_INVALID, "empty output gradient");
  if (pad_top > f_h - 1 || pad_left > f_w - 1) return fail(AMSIM_ERR_INVALID, "forward padding exceeds filter size - 1");
  const bool i32 = flags & AMSIM_INT32;
  const bool exact = (flags & AMSIM_DETERMINISTIC) || i32;  // int32 uses the reference's dense formulation
  const int hole_h = (out_h - 1) * stride_h + 1, hole_w = (out_w - 1) * stride_w + 1;  // convam.cc:1066-1067
  const int bpt = f_h - 1 - pad_top, bpl = f_w - 1 - pad_left;                        // convam.cc:1083-1084
  Params p{};
  p.V = dy; p.U = w; p.O = dx;
  p.v_elems = (long long)batch * out_h * out_w * out_c; p.u_elems = (long long)f_h * f_w * in_c * out_c;
  p.o_elems = (long long)batch * in_h * in_w * in_c;
  p.Q = in_c;
  p.u_tap = (long long)in_c * out_c; p.u_sk = 1; p.u_sq = out_c;  // w[tap][c][ko]: element (ko; c)
  p.o_sp = in_c; p.o_sq = 1;
  fill_lut(p, lut, true);
  Gather& g = p.g;
  g.SH = out_h; g.SW = out_w; g.SC = out_c;
  if (exact || (stride_h == 1 && stride_w == 1)) {
    // The reference's formulation: every input position gathers KH x KW taps of the
    // stride-dilated, back-padded gradient; positions between the strides are zeros
    // that still go through the multiplier.
    p.P = batch * in_h * in_w; p.K = f_h * f_w * out_c;
    g.PH = in_h; g.PW = in_w; g.ps_h = 1; g.ps_w = 1; g.off_t = bpt; g.off_l = bpl;
    g.lim_h = hole_h; g.lim_w = hole_w; g.dil_h = stride_h; g.dil_w = stride_w; g.KW = f_w;
    fill_gather_divs(g);
    if (f_h == 1 && f_w == 1 && stride_h == 1 && stride_w == 1 && bpt == 0 && bpl == 0 && out_h == in_h && out_w == in_w)
      dense_gather(g, out_c);  // a plain GEMM over the pixels
    // flipped filter with in/out channels swapped
    p.u_t0 = f_h * f_w - 1; p.u_tj = -f_w; p.u_ti = -1;
    if (i32) return launch_naive_i32((cudaStream_t)stream, p, lut, false);
    return launch_gather((cudaStream_t)stream, p, 1, exact, lut->device);
  }
  // Fast mode, stride > 1: a product with a structural zero is exactly 0, so each
  // stride phase (y % sh, x % sw) is computed on its own from the taps that can hit
  // a gradient sample: kh = kh0 + j * sh.  Same products, same order, no zero work.
  bool any_empty = false;
  for (int a = 0; a < stride_h && a < in_h; ++a)
    for (int b = 0; b < stride_w && b < in_w; ++b) {
      const int kh0 = (((bpt - a) % stride_h) + stride_h) % stride_h, kw0 = (((bpl - b) % stride_w) + stride_w) % stride_w;
      if (kh0 >= f_h || kw0 >= f_w) any_empty = true;
    }
  if (any_empty || stride_h > in_h || stride_w > in_w)
    CUDA_TRY(cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)batch * in_h * in_w * in_c, (cudaStream_t)stream));
  for (int a = 0; a < stride_h && a < in_h; ++a)
    for (int b = 0; b < stride_w && b < in_w; ++b) {
      const int kh0 = (((bpt - a) % stride_h) + stride_h) % stride_h, kw0 = (((bpl - b) % stride_w) + stride_w) % stride_w;
      if (kh0 >= f_h || kw0 >= f_w) continue;  // no tap reaches this phase: stays zero
      const int nh = (f_h - kh0 + stride_h - 1) / stride_h, nw = (f_w - kw0 + stride_w - 1) / stride_w;
      const int ra = (a - bpt + kh0) / stride_h, rb = (b - bpl + kw0) / stride_w;  // exact divisions
      Params q = p;
      Gather& h = q.g;
      h.PH = (in_h - a + stride_h - 1) / stride_h; h.PW = (in_w - b + stride_w - 1) / stride_w;
      h.ps_h = 1; h.ps_w = 1; h.off_t = -ra; h.off_l = -rb; h.lim_h = out_h; h.lim_w = out_w;
      h.dil_h = 1; h.dil_w = 1; h.KW = nw;
      fill_gather_divs(h);
      q.P = batch * h.PH * h.PW; q.K = nh * nw * out_c;
      q.u_t0 = (f_h - 1 - kh0) * f_w + (f_w - 1 - kw0); q.u_tj = -stride_h * f_w; q.u_ti = -stride_w;
      q.o_strided = 1; q.o_h = in_h; q.o_w = in_w; q.o_sh = stride_h; q.o_sw = stride_w; q.o_a = a; q.o_b = b;
      rc = launch_gather((cudaStream_t)stream, q, 1, false, lut->device);
      if (rc) return rc;
    }
  return AMSIM_OK;
}

// A weight gradient that is a plain GEMM, dw[k,u] = sum_r AM(x[r,k], g[r,u]) (dense layers; 1x1 stride-1
// unpadded convolutions, r = pixel): either operand can be the lane operand.  The 128 x 64 tile is filled
// better with the larger of (in_w, units) along its 128 rows; e.g. 64 -> 256 channels: 64 rows would
// half-fill the tile, 256 rows fill two.  Swapped, the table is indexed the other way round and the
// output is written transposed, so every product and every chain is the same.
static bool wgrad_swap(int in_w, int units) {
  auto padded = [](long long p, long long q) { return ((p + 127) / 128 * 128) * ((q + BQ - 1) / BQ * BQ); };
  if (sw().no_wgrad_swap) return false;
  return padded(units, in_w) < padded(in_w, units);
}

static void setup_wgrad(Params& p, const amsim_lut* lut, const float* x, const float* g_, float* dw, long long rows,
                        int in_w, int units, bool swap) {
  p.V = swap ? g_ : x;
  p.U = swap ? x : g_;
  p.O = dw;
  p.v_elems = rows * (swap ? units : in_w); p.u_elems = rows * (swap ? in_w : units); p.o_elems = (long long)in_w * units;
  p.P = swap ? units : in_w;
  p.Q = swap ? in_w : units;
  p.K = (int)rows;
  Gather& g = p.g;
  g.PH = 1; g.PW = 1; g.ps_h = 1; g.ps_w = 1; g.off_t = 0; g.off_l = 0; g.lim_h = 1; g.lim_w = 1;
  g.dil_h = 1; g.dil_w = 1; g.SH = 1; g.SW = 1; g.SC = p.P; g.KW = 1;
  fill_gather_divs(g);
  p.u_sk = p.Q; p.u_sq = 1;
  p.o_sp = swap ? 1 : units;
  p.o_sq = swap ? units : 1;
  fill_lut(p, lut, /*v_is_first_operand=*/!swap);
}

// Split-K scratch of a filter gradient; 0 for shapes the op itself refuses (check_conv_dims).
static size_t conv_fgrad_workspace(int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h,
                                   int out_w, bool det, int sms) {
  if (batch <= 0 || in_c <= 0 || f_h <= 0 || f_w <= 0 || out_c <= 0 || out_h <= 0 || out_w <= 0) return 0;
  if (!prod3_below(f_h, f_w, in_c > out_c ? in_c : out_c, 1ll << 30) || !prod3_below(batch, out_h, out_w, (1ll << 31) - 256))
    return 0;
  const long long rows = (long long)f_h * f_w * in_c, npix = (long long)batch * out_h * out_w;
  size_t need = fgrad_workspace((int)rows, out_c, (int)npix, det, sms);
  // a 1x1 stride-1 convolution may run with the operand roles swapped (wgrad_swap): cover both plans
  if (f_h == 1 && f_w == 1 && out_h == in_h && out_w == in_w && wgrad_swap(in_c, out_c))
    need = std::max(need, fgrad_workspace(out_c, in_c, (int)npix, det, sms));
  return need;
}

size_t amsim_conv2d_bwd_filter_workspace(int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c,
                                         int out_h, int out_w, unsigned flags) {
  if (flags & AMSIM_INT32) return 0;
  return conv_fgrad_workspace(batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w, flags & AMSIM_DETERMINISTIC,
                              sm_count(current_device()));
}

int amsim_conv2d_bwd_filter(void* stream, const amsim_lut* lut, const float* x, const float* dy, float* dw, int batch,
                            int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h, int out_w,
                            int stride_h, int stride_w, int pad_top, int pad_left, void* workspace,
                            size_t workspace_bytes, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  rc = check_conv_dims(batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w, stride_h, stride_w, pad_top, pad_left);
  if (rc) return rc;
  if (!dw) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  const long long npix = (long long)batch * out_h * out_w;
  if (npix == 0) {  // empty reduction: the gradient is all zeros
    CUDA_TRY(cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)f_h * f_w * in_c * out_c, (cudaStream_t)stream));
    return AMSIM_OK;
  }
  if (!x || !dy) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  if (f_h == 1 && f_w == 1 && stride_h == 1 && stride_w == 1 && pad_top == 0 && pad_left == 0 && out_h == in_h &&
      out_w == in_w && !(flags & AMSIM_INT32)) {
    // 1x1, stride 1, no padding: dw[c,k] = sum_pixels AM(x[pix,c], dy[pix,k]) is a plain GEMM
    // (no pixel -> (image, row, column) arithmetic in the gather, and either operand role)
    Params q{};
    setup_wgrad(q, lut, x, dy, dw, npix, in_c, out_c, wgrad_swap(in_c, out_c));
    return launch_fgrad((cudaStream_t)stream, q, flags & AMSIM_DETERMINISTIC, workspace, workspace_bytes, lut->device);
  }
  Params p{};
  p.V = x; p.U = dy; p.O = dw;
  p.v_elems = (long long)batch * in_h * in_w * in_c; p.u_elems = npix * out_c; p.o_elems = (long long)f_h * f_w * in_c * out_c;
  p.P = f_h * f_w * in_c; p.Q = out_c; p.K = (int)npix;
  Gather& g = p.g;
  g.PH = out_h; g.PW = out_w; g.ps_h = stride_h; g.ps_w = stride_w; g.off_t = pad_top; g.off_l = pad_left;
  g.lim_h = in_h; g.lim_w = in_w; g.dil_h = 1; g.dil_w = 1; g.SH = in_h; g.SW = in_w; g.SC = in_c; g.KW = f_w;
  fill_gather_divs(g);
  p.u_sk = out_c; p.u_sq = 1;
  p.o_sp = out_c; p.o_sq = 1;
  fill_lut(p, lut, true);
  if (flags & AMSIM_INT32) return launch_naive_i32((cudaStream_t)stream, p, lut, true);
  return launch_fgrad((cudaStream_t)stream, p, flags & AMSIM_DETERMINISTIC, workspace, workspace_bytes, lut->device);
}

// ---- built-in scratch for amsim_conv2d_bwd_filter_static ----------------------
// Lives in the device image of this library; in host code the symbol's name is
// only a handle, the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[AMSIM_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the CURRENT device, looked up once per
// device (the first call on a device does the lookup).
static int static_scratch_address(int device, void** out) {
  static std::mutex mu;
  static std::map<int, void*> known;
  std::lock_guard<std::mutex> lk(mu);
  auto it = known.find(device);
  if (it != known.end()) {
    *out = it->second;
    return AMSIM_OK;
  }
  void* p = nullptr;
  CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
  if (!p) return fail(AMSIM_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the built-in scratch");
  known[device] = p;
  *out = p;
  return AMSIM_OK;
}

int amsim_conv2d_bwd_filter_static(void* stream, const amsim_lut* lut, const float* x, const float* dy, float* dw,
                                   int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h,
                                   int out_w, int stride_h, int stride_w, int pad_top, int pad_left, unsigned flags) {
  int rc = check_common(lut, flags, true);  // also checks that lut->device is the current device
  if (rc) return rc;
  rc = check_conv_dims(batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w, stride_h, stride_w, pad_top, pad_left);
  if (rc) return rc;
  // the plan the launch will take: direct models always run unsplit (ordered chains), as in launch_fgrad
  const bool det = (flags & AMSIM_DETERMINISTIC) || lut->direct;
  const size_t need = (flags & AMSIM_INT32) ? 0
                                            : conv_fgrad_workspace(batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w,
                                                                   det, sm_count(lut->device));
  if (need > (size_t)AMSIM_STATIC_SCRATCH_BYTES)
    return fail(AMSIM_ERR_WORKSPACE,
                "this shape needs %zu bytes of split-K scratch, the built-in buffer holds %u: "
                "use amsim_conv2d_bwd_filter with a caller-provided workspace",
                need, (unsigned)AMSIM_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if (need > 0 && (rc = static_scratch_address(lut->device, &scratch))) return rc;
  return amsim_conv2d_bwd_filter(stream, lut, x, dy, dw, batch, in_h, in_w, in_c, f_h, f_w, out_c, out_h, out_w,
                                 stride_h, stride_w, pad_top, pad_left, scratch, need, flags);
}

// ---- bias gradient ------------------------------------------------------------------------------
// How the rows of a rows x cols gradient are cut into chunks: enough blocks to fill the device
// about four times over, at least 64 rows per chunk.
static void bias_grad_plan(long long rows, int cols, int sms, bool vec, int* cg, int* col_tiles, long long* chunks,
                           long long* rows_per_chunk) {
  const int groups = vec ? cols / 4 : cols;
  int c = 1;
  while (c < 64 && c < groups) c <<= 1;   // column groups per block: a power of two, at most 64
  *cg = c;
  *col_tiles = (groups + c - 1) / c;
  long long want = (4ll * sms + *col_tiles - 1) / *col_tiles;
  const long long most = (rows + 63) / 64;
  if (want > most) want = most;
  if (rows * cols <= (1ll << 16)) want = 1;  // small gradients (launch-bound networks): one kernel, no second pass
  if (want < 1) want = 1;
  *rows_per_chunk = (rows + want - 1) / want;
  *chunks = (rows + *rows_per_chunk - 1) / *rows_per_chunk;
}

size_t amsim_bias_grad_workspace(long long rows, int cols) {
  if (rows <= 0 || cols <= 0) return 0;
  int cg, tiles;
  long long chunks, rpc;
  bias_grad_plan(rows, cols, sm_count(current_device()), cols % 4 == 0, &cg, &tiles, &chunks, &rpc);
  long long scalar_chunks;
  bias_grad_plan(rows, cols, sm_count(current_device()), false, &cg, &tiles, &scalar_chunks, &rpc);
  const long long most = chunks > scalar_chunks ? chunks : scalar_chunks;  // the launch may fall back to scalar loads
  return most > 1 ? (size_t)most * cols * sizeof(float) : 0;
}

int amsim_bias_grad(void* stream, const float* grad, float* dbias, long long rows, int cols, void* workspace,
                    size_t workspace_bytes) {
  if (rows < 0 || cols <= 0) return fail(AMSIM_ERR_INVALID, "bias gradient: rows >= 0 and cols > 0 expected");
  if (!dbias) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) {
    CUDA_TRY(cudaMemsetAsync(dbias, 0, sizeof(float) * (size_t)cols, st));
    return AMSIM_OK;
  }
  if (!grad) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  const bool vec = cols % 4 == 0 && aligned16(grad);
  int cg, tiles;
  long long chunks, rpc;
  bias_grad_plan(rows, cols, sm_count(current_device()), vec, &cg, &tiles, &chunks, &rpc);
  float* part = dbias;
  if (chunks > 1) {
    const size_t need = (size_t)chunks * cols * sizeof(float);
    if (!workspace || workspace_bytes < need)
      return fail(AMSIM_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    part = static_cast<float*>(workspace);
  }
  dim3 grid((unsigned)chunks, (unsigned)tiles);
  AMSIM_COUNT_LAUNCH();
  if (vec) column_sums<true><<<grid, 256, 0, st>>>(grad, part, rows, cols, rpc, cg);
  else column_sums<false><<<grid, 256, 0, st>>>(grad, part, rows, cols, rpc, cg);
  CUDA_TRY(cudaGetLastError());
  if (chunks > 1) {
    AMSIM_COUNT_LAUNCH();
    const int lanes = reduce_lanes((int)chunks);
    reduce_splits<<<reduce_blocks(cols, lanes), 256, 0, st>>>(part, dbias, cols, (int)chunks, cols, 0, 1, lanes);
    CUDA_TRY(cudaGetLastError());
  }
  return AMSIM_OK;
}

static void dense_gather(Gather& g, int width) {
  g.PH = 1; g.PW = 1; g.ps_h = 1; g.ps_w = 1; g.off_t = 0; g.off_l = 0; g.lim_h = 1; g.lim_w = 1;
  g.dil_h = 1; g.dil_w = 1; g.SH = 1; g.SW = 1; g.SC = width; g.KW = 1;
  fill_gather_divs(g);
}

static int check_dense(int batch, int units, int input_width) {
  if (batch < 0 || units <= 0 || input_width <= 0) return fail(AMSIM_ERR_INVALID, "dense dimensions must be positive");
  if (units >= (1 << 30) || input_width >= (1 << 30) || (long long)batch >= (1ll << 31) - 256)
    return fail(AMSIM_ERR_UNSUPPORTED, "dense dimensions exceed 2^30 columns or 2^31 rows");
  return AMSIM_OK;
}

static int dense_fwd_impl(void* stream, const amsim_lut* lut, const float* x, const float* w, const float* bias,
                          float* y, int batch, int units, int input_width, int act, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  if (act != AMSIM_ACT_NONE && act != AMSIM_ACT_RELU) return fail(AMSIM_ERR_INVALID, "unknown activation %d", act);
  if ((bias || act) && (flags & AMSIM_INT32)) return fail(AMSIM_ERR_UNSUPPORTED, "the fused epilogue is FP32 only");
  if ((rc = check_dense(batch, units, input_width))) return rc;
  if (batch == 0) return AMSIM_OK;
  if (!x || !w || !y) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  Params p{};
  p.V = x; p.U = w; p.O = y;
  p.v_elems = (long long)batch * input_width; p.u_elems = (long long)input_width * units; p.o_elems = (long long)batch * units;
  p.P = batch; p.Q = units; p.K = input_width;
  dense_gather(p.g, input_width);
  p.u_t0 = 0; p.u_tj = 0; p.u_ti = 0; p.u_tap = 0; p.u_sk = units; p.u_sq = 1;
  p.o_sp = units; p.o_sq = 1;
  fill_lut(p, lut, true);
  p.bias = bias;
  p.relu = act == AMSIM_ACT_RELU;
  if (flags & AMSIM_INT32) return launch_naive_i32((cudaStream_t)stream, p, lut, false);
  return launch_gather((cudaStream_t)stream, p, 1, flags & AMSIM_DETERMINISTIC, lut->device);
}

int amsim_dense_fwd(void* stream, const amsim_lut* lut, const float* x, const float* w, float* y, int batch, int units,
                    int input_width, unsigned flags) {
  return dense_fwd_impl(stream, lut, x, w, nullptr, y, batch, units, input_width, AMSIM_ACT_NONE, flags);
}

int amsim_dense_fwd_bias_act(void* stream, const amsim_lut* lut, const float* x, const float* w, const float* bias,
                             float* y, int batch, int units, int input_width, int act, unsigned flags) {
  return dense_fwd_impl(stream, lut, x, w, bias, y, batch, units, input_width, act, flags);
}

int amsim_dense_bwd_input(void* stream, const amsim_lut* lut, const float* w, const float* g_, float* dx, int batch,
                          int units, int input_width, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  if ((rc = check_dense(batch, units, input_width))) return rc;
  if (batch == 0) return AMSIM_OK;
  if (!w || !g_ || !dx) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  // dx[b,k] = sum_u AM(w[k,u], g[b,u]) — denseam_kernel.cu:84-94: the weight is
  // the multiplier's FIRST operand, the gradient (lane operand here) the second.
  Params p{};
  p.V = g_; p.U = w; p.O = dx;
  p.v_elems = (long long)batch * units; p.u_elems = (long long)input_width * units; p.o_elems = (long long)batch * input_width;
  p.P = batch; p.Q = input_width; p.K = units;
  dense_gather(p.g, units);
  p.u_t0 = 0; p.u_tj = 0; p.u_ti = 0; p.u_tap = 0; p.u_sk = 1; p.u_sq = units;
  p.o_sp = input_width; p.o_sq = 1;
  fill_lut(p, lut, /*v_is_first_operand=*/false);
  if (flags & AMSIM_INT32) return launch_naive_i32((cudaStream_t)stream, p, lut, false);
  return launch_gather((cudaStream_t)stream, p, 1, flags & AMSIM_DETERMINISTIC, lut->device);
}

size_t amsim_dense_bwd_weight_workspace(int batch, int units, int input_width, unsigned flags) {
  if (batch <= 0 || units <= 0 || input_width <= 0) return 0;
  if (units >= (1 << 30) || input_width >= (1 << 30) || (long long)batch >= (1ll << 31) - 256) return 0;  // refused by the op
  if (flags & AMSIM_INT32) return 0;
  const int sms = sm_count(current_device());
  if (wgrad_swap(input_width, units)) return fgrad_workspace(units, input_width, batch, flags & AMSIM_DETERMINISTIC, sms);
  return fgrad_workspace(input_width, units, batch, flags & AMSIM_DETERMINISTIC, sms);
}

int amsim_dense_bwd_weight(void* stream, const amsim_lut* lut, const float* x, const float* g_, float* dw, int batch,
                           int units, int input_width, void* workspace, size_t workspace_bytes, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  if ((rc = check_dense(batch, units, input_width))) return rc;
  if (!dw) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  if (batch == 0) {
    CUDA_TRY(cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)input_width * units, (cudaStream_t)stream));
    return AMSIM_OK;
  }
  if (!x || !g_) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  // dw[k,u] = sum_b AM(x[b,k], g[b,u]) — the filter gradient of a 1x1
  // convolution over a batch x 1 x 1 grid.
  Params p{};
  setup_wgrad(p, lut, x, g_, dw, batch, input_width, units, !(flags & AMSIM_INT32) && wgrad_swap(input_width, units));
  if (flags & AMSIM_INT32) return launch_naive_i32((cudaStream_t)stream, p, lut, true);
  return launch_fgrad((cudaStream_t)stream, p, flags & AMSIM_DETERMINISTIC, workspace, workspace_bytes, lut->device);
}

static int matmul_impl(void* stream, const amsim_lut* lut, const float* a, const float* b, float* c, int batch_a,
                       int batch_b, int row_a, int col_a, int row_b, int col_b, int trans_a, int trans_b, int has_alpha,
                       float alpha, unsigned flags) {
  int rc = check_common(lut, flags, true);
  if (rc) return rc;
  if (batch_a < 0 || batch_b < 0 || row_a < 0 || col_a < 0 || row_b < 0 || col_b < 0)
    return fail(AMSIM_ERR_INVALID, "negative matrix dimension");
  if (flags & AMSIM_INT32)
    return fail(AMSIM_ERR_UNSUPPORTED, "MatMulAM is registered for float only (matmulam.cc:269-274)");
  // logical shapes after the transposes: [M, K] x [K, N]
  const int M = trans_a ? col_a : row_a, Ka = trans_a ? row_a : col_a;
  const int Kb = trans_b ? col_b : row_b, N = trans_b ? row_b : col_b;
  if (Ka != Kb) return fail(AMSIM_ERR_INVALID, "Does not meet cols of mat a is equal rows of mat b");
  if (batch_a > 1 && batch_b > 1 && batch_a != batch_b)
    return fail(AMSIM_ERR_INVALID, "Does not meet batch of mat a is equal batch of matb");
  int nb = batch_a > batch_b ? batch_a : batch_b;
  if (nb == 0) nb = 1;
  if (M == 0 || N == 0) return AMSIM_OK;
  if (!c) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  if (Ka == 0) {  // [x,0] x [0,y]: zeros (matmulam.cc:156-161)
    CUDA_TRY(cudaMemsetAsync(c, 0, sizeof(float) * (size_t)nb * M * N, (cudaStream_t)stream));
    return AMSIM_OK;
  }
  if (!a || !b) return fail(AMSIM_ERR_INVALID, "NULL tensor pointer");
  Params p{};
  p.V = a; p.U = b; p.O = c;
  p.v_elems = (long long)(batch_a > 1 ? batch_a : 1) * row_a * col_a; p.u_elems = (long long)(batch_b > 1 ? batch_b : 1) * row_b * col_b;
  p.o_elems = (long long)nb * M * N;
  p.P = M; p.Q = N; p.K = Ka;
  dense_gather(p.g, Ka);
  if (trans_a) {
    // a is stored [K, M]: element (p, k) at a[k * M + p]; the scalar gather path reads it in place
    p.v_trans = 1;
    p.v_ld = M;
  }
  p.u_t0 = 0; p.u_tj = 0; p.u_ti = 0; p.u_tap = 0;
  if (trans_b) { p.u_sk = 1; p.u_sq = Ka; } else { p.u_sk = N; p.u_sq = 1; }
  p.o_sp = N; p.o_sq = 1;
  p.v_bs = batch_a > 1 ? (long long)row_a * col_a : 0;
  p.u_bs = batch_b > 1 ? (long long)row_b * col_b : 0;
  p.o_bs = (long long)M * N;
  p.has_alpha = has_alpha;
  p.alpha = alpha;
  fill_lut(p, lut, true);
  return launch_gather((cudaStream_t)stream, p, nb, flags & AMSIM_DETERMINISTIC, lut->device);
}

int amsim_matmul(void* stream, const amsim_lut* lut, const float* a, const float* b, float* c, int batch_a,
                 int batch_b, int row_a, int col_a, int row_b, int col_b, unsigned flags) {
  return matmul_impl(stream, lut, a, b, c, batch_a, batch_b, row_a, col_a, row_b, col_b, 0, 0, 0, 1.0f, flags);
}

int amsim_matmul_ex(void* stream, const amsim_lut* lut, const float* a, const float* b, float* c, int batch_a,
                    int batch_b, int row_a, int col_a, int row_b, int col_b, int transpose_a, int transpose_b,
                    const float* alpha, unsigned flags) {
  return matmul_impl(stream, lut, a, b, c, batch_a, batch_b, row_a, col_a, row_b, col_b, transpose_a != 0,
                     transpose_b != 0, alpha != nullptr, alpha ? *alpha : 1.0f, flags);
}

}  // extern "C"
