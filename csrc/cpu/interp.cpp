// CPU backend: packet reader/validator, counter-gated multi-threaded interpreter, golden f32 ops.
//
// The interpreter executes exactly the model every backend shares: a worker owns a set of
// compute-unit streams and, for the entry at the head of each, polls its wait counters, runs
// its slice range, publishes with a release increment of its instruction's counter.  Streams
// are in instruction order, so the globally earliest unfinished instruction always has all of
// its entries at stream heads and the walk cannot deadlock; a watchdog deadline turns a
// malformed program into an error code instead of a hang.
//
// All arithmetic is plain f32: this backend is the hermetic serving path for CPU-only boxes
// and the numeric oracle the GPU kernels are compared against.  Reference counterparts:
// crates/plowrt/src/exec/cpu/{interp,engine}.rs, runtime/cpu/dev/golden/*.c,
// crates/plowrt/src/exec/health.rs (counter monitor).
#include <algorithm>
#include <immintrin.h>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#if defined(__linux__)
#include <sys/syscall.h>
#include <unistd.h>
#endif

#include "plow_packet.h"

namespace {

struct Pkt {
  std::vector<uint8_t> raw;
  const PlowPktHeader* hdr = nullptr;
  const PlowTensorEnt* tensors = nullptr;
  const PlowProgramEnt* programs = nullptr;
  const PlowSectionEnt* sections = nullptr;
  const char* strtab = nullptr;
};

bool in_range(const Pkt& p, uint64_t ofs, uint64_t n) {
  return ofs >= sizeof(PlowPktHeader) && ofs + n <= p.raw.size() && ofs + n >= ofs;
}

std::string validate(Pkt& p) {
  if (p.raw.size() < sizeof(PlowPktHeader)) return "truncated header";
  p.hdr = reinterpret_cast<const PlowPktHeader*>(p.raw.data());
  const PlowPktHeader& h = *p.hdr;
  if (std::memcmp(h.magic, PLOW_PKT_MAGIC, 8) != 0) return "bad magic";
  if (h.version != PLOW_PKT_VERSION) return "unsupported packet version";
  if (h.header_bytes != sizeof(PlowPktHeader) || h.file_bytes != p.raw.size()) return "size mismatch";
  if (!in_range(p, h.tensor_ofs, uint64_t(h.n_tensor) * sizeof(PlowTensorEnt))) return "tensor table out of range";
  if (!in_range(p, h.program_ofs, uint64_t(h.n_program) * sizeof(PlowProgramEnt))) return "program table out of range";
  if (!in_range(p, h.section_ofs, uint64_t(h.n_section) * sizeof(PlowSectionEnt))) return "section table out of range";
  if (!in_range(p, h.strtab_ofs, h.strtab_bytes)) return "string table out of range";
  p.tensors = reinterpret_cast<const PlowTensorEnt*>(p.raw.data() + h.tensor_ofs);
  p.programs = reinterpret_cast<const PlowProgramEnt*>(p.raw.data() + h.program_ofs);
  p.sections = reinterpret_cast<const PlowSectionEnt*>(p.raw.data() + h.section_ofs);
  p.strtab = reinterpret_cast<const char*>(p.raw.data() + h.strtab_ofs);
  if (h.strtab_bytes == 0 || p.strtab[h.strtab_bytes - 1] != 0) return "string table not terminated";
  for (uint32_t i = 0; i < h.n_tensor; ++i) {
    if (p.tensors[i].name_ofs >= h.strtab_bytes) return "tensor name out of range";
    if (p.tensors[i].rank > 4) return "tensor rank > 4";
  }
  // the activation arena is allocated from this field: no program may need more than it says, and it may not say more
  // than any host could hold (a flipped high byte would otherwise turn into an allocation failure at engine creation)
  if (h.act_arena_bytes > (uint64_t(1) << 40)) return "activation arena size is not plausible";
  for (uint32_t k = 0; k < h.n_program; ++k) {
    const PlowProgramEnt& g = p.programs[k];
    if (g.arena_bytes > h.act_arena_bytes) return "a program's arena exceeds the packet's arena size";
    if (!in_range(p, g.inst_ofs, uint64_t(g.n_inst) * sizeof(PlowInst))) return "inst range";
    if (!in_range(p, g.stream_ofs, uint64_t(g.n_stream) * sizeof(PlowStreamEnt))) return "stream range";
    if (!in_range(p, g.cu_ofs, uint64_t(g.n_cu + 1) * 4)) return "cu_ofs range";
    if (!in_range(p, g.wait_ofs, uint64_t(g.n_wait) * sizeof(PlowWait)) && g.n_wait) return "wait range";
    if (!in_range(p, g.succ_ofs, uint64_t(g.n_succ) * 4) && g.n_succ) return "succ range";
    if (!in_range(p, g.actmap_ofs, uint64_t(h.n_tensor) * 8)) return "actmap range";
    const PlowInst* insts = reinterpret_cast<const PlowInst*>(p.raw.data() + g.inst_ofs);
    const PlowStreamEnt* st = reinterpret_cast<const PlowStreamEnt*>(p.raw.data() + g.stream_ofs);
    const uint32_t* cu = reinterpret_cast<const uint32_t*>(p.raw.data() + g.cu_ofs);
    const PlowWait* waits = reinterpret_cast<const PlowWait*>(p.raw.data() + g.wait_ofs);
    const uint32_t* succs = reinterpret_cast<const uint32_t*>(p.raw.data() + g.succ_ofs);
    if (cu[0] != 0 || cu[g.n_cu] != g.n_stream) return "cu_ofs does not cover the stream";
    for (uint32_t c = 0; c < g.n_cu; ++c)
      if (cu[c] > cu[c + 1]) return "cu_ofs not monotone";
    for (uint32_t i = 0; i < g.n_inst; ++i) {
      if (insts[i].op >= PLOW_OP__COUNT) return "unknown opcode";
      for (int j = 0; j < 8; ++j)
        if (insts[i].t[j] != PLOW_T_NONE && insts[i].t[j] >= h.n_tensor) return "tensor handle out of range";
    }
    for (uint32_t s = 0; s < g.n_stream; ++s) {
      if (st[s].inst >= g.n_inst) return "stream entry names a missing instruction";
      if (uint32_t(st[s].slice0) + st[s].nslice > insts[st[s].inst].nslice) return "slice range exceeds instruction";
      if (uint64_t(st[s].wait_ofs) + st[s].n_wait > g.n_wait) return "wait range out of bounds";
      if (uint64_t(st[s].succ_ofs) + st[s].n_succ > g.n_succ) return "succ range out of bounds";
    }
    // every activation the program places must lie inside its arena (sampled-row dims counted as one row: a lower bound
    // that still catches an offset or a dimension that points nowhere)
    const uint64_t* actmap = reinterpret_cast<const uint64_t*>(p.raw.data() + g.actmap_ofs);
    static const uint64_t kEs[] = {4, 2, 2, 1, 4, 1, 8};
    for (uint32_t t = 0; t < h.n_tensor; ++t) {
      const PlowTensorEnt& te = p.tensors[t];
      if (te.tclass != PLOW_TC_ACT || actmap[t] == UINT64_MAX) continue;
      if (te.dtype >= sizeof(kEs) / sizeof(kEs[0])) return "unknown dtype";
      unsigned __int128 nb = kEs[te.dtype];
      for (int d = 0; d < te.rank; ++d) {
        const int64_t v = te.dims[d];
        if (v == 0 || v < -4) return "tensor dimension out of range";
        nb *= v == -1 ? uint64_t(g.rows) : v < 0 ? uint64_t(1) : uint64_t(v);
        if (nb > (unsigned __int128)(uint64_t(1) << 42)) return "activation size is not plausible";
      }
      if (actmap[t] > g.arena_bytes || uint64_t(nb) > g.arena_bytes - actmap[t]) return "activation lies outside the arena";
    }
    for (uint32_t w = 0; w < g.n_wait; ++w)
      if (waits[w].ctr >= g.n_ctr) return "wait counter out of range";
    for (uint32_t s = 0; s < g.n_succ; ++s)
      if (succs[s] >= g.n_ctr) return "succ counter out of range";
  }
  return "";
}

// ---------------------------------------------------------------------------------------------
struct StepIO {
  int32_t rows;
  int32_t n_sample;
  const int32_t* page_table;  // [n_slots, max_pages]
  int32_t max_pages;
  const int32_t* kvlen;       // [n_slots] (unused by the causal path; pos drives the mask)
  int32_t n_slots;
  const int32_t* pos;         // [rows]
  const int32_t* seq;         // [rows]
};

struct Engine {
  Pkt* pkt;
  int n_threads;
  std::vector<void*> bound;          // per tensor handle
  std::vector<uint8_t> arena;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv_start, cv_done;
  uint64_t generation = 0;
  int pending = 0;
  bool quit = false;
  // per run
  const PlowProgramEnt* prog = nullptr;
  StepIO io{};
  std::vector<std::atomic<uint32_t>> counters;
  std::atomic<int> status{0};
  std::vector<PlowTraceRec> trace;
  bool trace_on = false;
  double watchdog_s = 30.0;
};

inline uint64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Ctx {
  Engine* e;
  const PlowInst* in;
  int s0, s1, ns;  // slice range [s0, s1) of ns
  void* T(int j) const {
    uint16_t h = in->t[j];
    if (h == PLOW_T_NONE) return nullptr;
    const PlowTensorEnt& te = e->pkt->tensors[h];
    if (te.tclass == PLOW_TC_ACT) {
      const uint64_t* actmap = reinterpret_cast<const uint64_t*>(e->pkt->raw.data() + e->prog->actmap_ofs);
      return e->arena.data() + actmap[h];
    }
    return e->bound[h];
  }
  // work range of this entry over W items
  void range(int64_t W, int64_t& a, int64_t& b) const {
    a = W * s0 / ns;
    b = W * s1 / ns;
  }
};

inline float dotf(const float* a, const float* b, int n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
  float s = 0.f;
  for (; i < n; ++i) s += a[i] * b[i];
  for (int j = 0; j < 8; ++j) s += acc[j];
  return s;
}

void op_embed(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* tab = (const float*)c.T(1);
  const int32_t* ids = (const int32_t*)c.T(2);
  const int H = c.in->i[0];
  const float scale = c.in->w[0].f;
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const float* src = tab + int64_t(ids[r]) * H;
    for (int j = 0; j < H; ++j) out[r * H + j] = scale == 1.0f ? src[j] : src[j] * scale;
  }
}

inline void rmsnorm_row(float* out, const float* x, const float* g, int W, float eps, int mode) {
  float ss = 0.f;
  for (int j = 0; j < W; ++j) ss += x[j] * x[j];
  const float r = 1.0f / std::sqrt(ss / W + eps);
  for (int j = 0; j < W; ++j) {
    const float gm = g ? (mode ? 1.0f + g[j] : g[j]) : 1.0f;
    out[j] = x[j] * r * gm;
  }
}

void op_rmsnorm(const Ctx& c, int64_t rows) {
  float* out = (float*)c.T(0);
  const float* x = (const float*)c.T(1);
  const float* g = (const float*)c.T(2);
  const int W = c.in->i[0], mode = c.in->i[1];
  const int co = c.in->i[6], pitch = c.in->i[7] ? c.in->i[7] : W;
  int64_t a, b;
  c.range(rows, a, b);
  for (int64_t r = a; r < b; ++r) rmsnorm_row(out + r * W, x + r * pitch + co, g, W, c.in->w[0].f, mode);
}

void op_add_norm(const Ctx& c) {
  float* h = (float*)c.T(0);
  const float* x = (const float*)c.T(1);
  const float* d = (const float*)c.T(2);
  const float* g = (const float*)c.T(3);
  float* xo = (float*)c.T(4);
  const int W = c.in->i[0];
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    for (int j = 0; j < W; ++j) xo[r * W + j] = x[r * W + j] + d[r * W + j];
    rmsnorm_row(h + r * W, xo + r * W, g, W, c.in->w[0].f, c.in->i[1]);
  }
}

void op_residual(const Ctx& c) {
  float* o = (float*)c.T(0);
  const float* x = (const float*)c.T(1);
  const float* d = (const float*)c.T(2);
  const int W = c.in->i[0];
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t k = a * W; k < b * W; ++k) o[k] = x[k] + d[k];
}

// ---- GEMM kernel tiers ---------------------------------------------------------------------------------------------
// y[m][n] = x[m] . w[n] (+ SiLU-gated pair).  Four bodies behind one op, picked once per process (PLOW_CPU_TIER =
// golden | avx2 | avx512 | amx | auto, or plow_cpu_set_tier):
//   golden  one output at a time: the numeric statement the others are held to;
//   avx2    eight rows share every weight row they read (the weight matrix is streamed rows / 8 times instead of rows
//           times) with 8-lane FMA accumulators, summed tail elements first, then lanes 0..7;
//   avx512  the same with 16 lanes;
//   amx     16x16 output tiles on the AMX unit (TDPBF16PS): inputs rounded to bf16, fp32 accumulation.  The product is
//           formed transposed, y^T = w . x^T, so weight rows load as A tiles straight after conversion and only the
//           activations (small) are repacked into the pair-interleaved B layout, once per op.  GEMMs of fewer than
//           16 rows take the avx512 body.  Never picked by `auto`: bf16 inputs move logits by ~1e-2 relative, the
//           same order as the GPU engine's bf16 path.
// The tiers order their sums differently from the compiler's own vectorisation of the golden loop, so they agree with it
// to rounding (1e-6 relative on a model's logits), not bit for bit.  `auto` takes avx2 when the CPU has it; avx512 is a
// choice (on a 250-row prefill of the 4-layer test model: golden 77 ms, avx2 56 ms, avx512 41 ms).
// Reference counterpart: runtime/cpu (scalar / AVX2 / AVX-512 / AMX kernel tiers behind one dispatch table).
enum { TIER_GOLDEN = 0, TIER_AVX2 = 1, TIER_AVX512 = 2, TIER_AMX = 3 };

// gate activation of a GLU: SiLU unless the flags ask for GELU (tanh or erf form)
static inline float glu_act(float v, uint32_t flags) {
  if (flags & PLOW_GEMM_ACT_GELU_TANH) return 0.5f * v * (1.0f + std::tanh(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  if (flags & PLOW_GEMM_ACT_GELU_ERF) return 0.5f * v * (1.0f + std::erf(v * 0.7071067811865476f));
  return v / (1.0f + std::exp(-v));
}

// The kernel hands out AMX tile state per process on request (arch_prctl ARCH_REQ_XCOMP_PERM, feature 18 = tile data).
static int amx_permitted() {
  static const int ok = [] {
#if defined(__linux__) && defined(__x86_64__)
    if (!__builtin_cpu_supports("amx-tile") || !__builtin_cpu_supports("amx-bf16") || !__builtin_cpu_supports("avx512bf16")) return 0;
    return syscall(SYS_arch_prctl, 0x1023, 18) == 0 ? 1 : 0;
#else
    return 0;
#endif
  }();
  return ok;
}

static int tier_supported(int t) {
  if (t == TIER_AVX2) return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  if (t == TIER_AVX512) return __builtin_cpu_supports("avx512f");
  if (t == TIER_AMX) return __builtin_cpu_supports("avx512f") && amx_permitted();
  return t == TIER_GOLDEN;
}

static int pick_tier() {
  const char* e = std::getenv("PLOW_CPU_TIER");
  const std::string v = e ? e : "auto";
  if (v == "golden") return TIER_GOLDEN;
  if (v == "amx" && tier_supported(TIER_AMX)) return TIER_AMX;
  if ((v == "avx512" || v == "amx") && tier_supported(TIER_AVX512)) return TIER_AVX512;
  if ((v == "avx2" || v == "auto" || v == "avx512" || v == "amx") && tier_supported(TIER_AVX2)) return TIER_AVX2;
  return TIER_GOLDEN;
}
static std::atomic<int> g_tier{-1};
static int cur_tier() {
  int t = g_tier.load(std::memory_order_relaxed);
  if (t < 0) { t = pick_tier(); g_tier.store(t, std::memory_order_relaxed); }
  return t;
}

constexpr int kRowBlock = 8;

// dots of up to 8 rows of x (row pitch `pitch`) with one weight row: out[r] = x[r] . w
__attribute__((target("avx2,fma"))) static void dots_avx2(const float* x, int64_t pitch, int nr, const float* w, int K, float* out) {
  __m256 acc[kRowBlock];
  for (int r = 0; r < kRowBlock; ++r) acc[r] = _mm256_setzero_ps();
  int i = 0;
  for (; i + 8 <= K; i += 8) {
    const __m256 wv = _mm256_loadu_ps(w + i);
    for (int r = 0; r < nr; ++r) acc[r] = _mm256_fmadd_ps(_mm256_loadu_ps(x + r * pitch + i), wv, acc[r]);
  }
  for (int r = 0; r < nr; ++r) {
    float s = 0.f;
    for (int k = i; k < K; ++k) s += x[r * pitch + k] * w[k];
    alignas(32) float lane[8];
    _mm256_store_ps(lane, acc[r]);
    for (int j = 0; j < 8; ++j) s += lane[j];
    out[r] = s;
  }
}

__attribute__((target("avx512f"))) static void dots_avx512(const float* x, int64_t pitch, int nr, const float* w, int K, float* out) {
  __m512 acc[kRowBlock];
  for (int r = 0; r < kRowBlock; ++r) acc[r] = _mm512_setzero_ps();
  int i = 0;
  for (; i + 16 <= K; i += 16) {
    const __m512 wv = _mm512_loadu_ps(w + i);
    for (int r = 0; r < nr; ++r) acc[r] = _mm512_fmadd_ps(_mm512_loadu_ps(x + r * pitch + i), wv, acc[r]);
  }
  for (int r = 0; r < nr; ++r) {
    float s = 0.f;
    for (int k = i; k < K; ++k) s += x[r * pitch + k] * w[k];
    alignas(64) float lane[16];
    _mm512_store_ps(lane, acc[r]);
    for (int j = 0; j < 16; ++j) s += lane[j];
    out[r] = s;
  }
}

// ---- AMX tier ----
struct alignas(64) AmxTileCfg {
  uint8_t palette, start_row, rsv[14];
  uint16_t colsb[16];
  uint8_t rows[16];
};
#define PLOW_AMX_TARGET __attribute__((target("amx-tile,amx-bf16,avx512f,avx512bf16,avx512bw")))

// 32 floats -> 32 bf16 (round to nearest even) as 16 dwords; dword j holds elements (2j, 2j+1)
PLOW_AMX_TARGET static inline __m512i cvt32(const float* p) {
  return (__m512i)_mm512_cvtne2ps_pbh(_mm512_loadu_ps(p + 16), _mm512_loadu_ps(p));
}
PLOW_AMX_TARGET static inline __m512i cvt32_tail(const float* p, int n) {   // n < 32 valid elements, the rest zero
  const __mmask16 lo = n >= 16 ? 0xffff : __mmask16((1u << n) - 1), hi = n > 16 ? __mmask16((1u << (n - 16)) - 1) : 0;
  return (__m512i)_mm512_cvtne2ps_pbh(_mm512_maskz_loadu_ps(hi, p + 16), _mm512_maskz_loadu_ps(lo, p));
}

// x rows -> B tiles: xt[(mb * KT + kt)][k2][m][2] = x[mb*16 + m][kt*32 + 2*k2 + {0,1}], zero beyond rows / K
PLOW_AMX_TARGET static void amx_pack_x(const float* x, int64_t pitch, int64_t rows, int K, int KT, uint32_t* xt) {
  const int64_t MB = (rows + 15) / 16;
  alignas(64) uint32_t v[16];
  for (int64_t mb = 0; mb < MB; ++mb)
    for (int kt = 0; kt < KT; ++kt) {
      uint32_t* tile = xt + (mb * KT + kt) * 256;
      const int kn = std::min(32, K - kt * 32);
      for (int m = 0; m < 16; ++m) {
        const int64_t r = mb * 16 + m;
        if (r < rows) {
          const float* src = x + r * pitch + kt * 32;
          _mm512_store_si512((void*)v, kn == 32 ? cvt32(src) : cvt32_tail(src, kn));
          for (int k2 = 0; k2 < 16; ++k2) tile[k2 * 16 + m] = v[k2];
        } else {
          for (int k2 = 0; k2 < 16; ++k2) tile[k2 * 16 + m] = 0;
        }
      }
    }
}

// 16 weight rows (nn valid) -> bf16 staging [16][KT*32], zero padded
PLOW_AMX_TARGET static void amx_stage_w(const float* w, int K, int KT, int nn, uint16_t* st) {
  const int Kp = KT * 32;
  for (int n = 0; n < 16; ++n) {
    uint16_t* d = st + int64_t(n) * Kp;
    if (n >= nn) { std::memset(d, 0, sizeof(uint16_t) * Kp); continue; }
    const float* src = w + int64_t(n) * K;
    int k = 0;
    for (; k + 32 <= K; k += 32) _mm512_storeu_si512((void*)(d + k), cvt32(src + k));
    if (k < K) _mm512_storeu_si512((void*)(d + k), cvt32_tail(src + k, K - k));
  }
}

// out[n][m] (pitch Mp floats) = staged weight rows . packed x, for all row blocks; two row blocks share each A tile
PLOW_AMX_TARGET static void amx_block(const uint16_t* st, const uint32_t* xt, int KT, int64_t MB, int64_t Mp, float* out) {
  const int Kp = KT * 32;
  int64_t mb = 0;
  for (; mb + 2 <= MB; mb += 2) {
    _tile_zero(0);
    _tile_zero(1);
    const uint32_t* b0 = xt + mb * KT * 256;
    const uint32_t* b1 = b0 + int64_t(KT) * 256;
    for (int kt = 0; kt < KT; ++kt) {
      _tile_loadd(2, st + kt * 32, Kp * 2);
      _tile_loadd(3, b0 + kt * 256, 64);
      _tile_loadd(4, b1 + kt * 256, 64);
      _tile_dpbf16ps(0, 2, 3);
      _tile_dpbf16ps(1, 2, 4);
    }
    _tile_stored(0, out + mb * 16, Mp * 4);
    _tile_stored(1, out + (mb + 1) * 16, Mp * 4);
  }
  if (mb < MB) {
    _tile_zero(0);
    const uint32_t* b0 = xt + mb * KT * 256;
    for (int kt = 0; kt < KT; ++kt) {
      _tile_loadd(2, st + kt * 32, Kp * 2);
      _tile_loadd(3, b0 + kt * 256, 64);
      _tile_dpbf16ps(0, 2, 3);
    }
    _tile_stored(0, out + mb * 16, Mp * 4);
  }
}

PLOW_AMX_TARGET static void gemm_amx(float* y, const float* x, const float* w, const float* bias, int64_t rows, int N, int K, int64_t pitch,
                                     uint32_t flags, int64_t a, int64_t b) {
  const bool dual = flags & PLOW_GEMM_DUAL_SILU;
  const int KT = (K + 31) / 32;
  const int64_t MB = (rows + 15) / 16, Mp = MB * 16;
  thread_local std::vector<uint32_t> xt;
  thread_local std::vector<uint16_t> st;
  thread_local std::vector<float> og, ou;
  xt.resize(size_t(MB) * KT * 256 + 16);
  st.resize(size_t(16) * KT * 32 + 32);
  og.resize(size_t(16) * Mp + 16);
  ou.resize(size_t(16) * Mp + 16);
  auto al = [](auto* p) { return (decltype(p))((uintptr_t(p) + 63) & ~uintptr_t(63)); };
  uint32_t* xtp = al(xt.data());
  uint16_t* stp = al(st.data());
  float *g = al(og.data()), *u = al(ou.data());
  amx_pack_x(x, pitch, rows, K, KT, xtp);
  AmxTileCfg cfg;
  std::memset(&cfg, 0, sizeof cfg);
  cfg.palette = 1;
  for (int t = 0; t < 5; ++t) { cfg.colsb[t] = 64; cfg.rows[t] = 16; }
  _tile_loadconfig(&cfg);
  for (int64_t n0 = a; n0 < b; n0 += 16) {
    const int nn = int(std::min<int64_t>(16, b - n0));
    amx_stage_w(w + n0 * K, K, KT, nn, stp);
    amx_block(stp, xtp, KT, MB, Mp, g);
    if (dual) {
      amx_stage_w(w + (n0 + N) * K, K, KT, nn, stp);
      amx_block(stp, xtp, KT, MB, Mp, u);
    }
    for (int n = 0; n < nn; ++n)
      for (int64_t m = 0; m < rows; ++m) {
        float v = g[n * Mp + m] + (bias ? bias[n0 + n] : 0.f);
        if (dual) v = glu_act(v, flags) * u[n * Mp + m];
        y[m * N + n0 + n] = v;
      }
  }
  _tile_release();
}

void op_gemm(const Ctx& c, int64_t rows) {
  float* y = (float*)c.T(0);
  const float* x = (const float*)c.T(1);
  const float* w = (const float*)c.T(2);
  const int N = c.in->i[0], K = c.in->i[1];
  const uint32_t flags = c.in->i[2];
  const int co = c.in->i[6], pitch = c.in->i[7] ? c.in->i[7] : K;
  const bool dual = flags & PLOW_GEMM_DUAL_SILU;
  const float* bias = (flags & PLOW_GEMM_BIAS) ? (const float*)c.T(7) : nullptr;   // never together with a gated pair
  int64_t a, b;
  c.range(N, a, b);
  const int tier = cur_tier();
  if (tier == TIER_GOLDEN) {
    for (int64_t m = 0; m < rows; ++m) {
      const float* xr = x + m * pitch + co;
      for (int64_t n = a; n < b; ++n) {
        float v = dotf(xr, w + n * K, K) + (bias ? bias[n] : 0.f);
        if (dual) {
          const float u = dotf(xr, w + (n + N) * K, K);
          v = glu_act(v, flags) * u;
        }
        y[m * N + n] = v;
      }
    }
    return;
  }
  if (tier == TIER_AMX && rows >= 16) {
    gemm_amx(y, x + co, w, bias, rows, N, K, pitch, flags, a, b);
    return;
  }
  auto dots = tier >= TIER_AVX512 ? dots_avx512 : dots_avx2;
  float g[kRowBlock], u[kRowBlock];
  for (int64_t m0 = 0; m0 < rows; m0 += kRowBlock) {
    const int nr = int(std::min<int64_t>(kRowBlock, rows - m0));
    const float* xb = x + m0 * pitch + co;
    for (int64_t n = a; n < b; ++n) {
      dots(xb, pitch, nr, w + n * K, K, g);
      if (dual) {
        dots(xb, pitch, nr, w + (n + N) * K, K, u);
        for (int r = 0; r < nr; ++r) g[r] = glu_act(g[r], flags) * u[r];
      }
      const float bn = bias ? bias[n] : 0.f;
      for (int r = 0; r < nr; ++r) y[(m0 + r) * N + n] = g[r] + bn;
    }
  }
}

inline void rope_head(float* out, const float* x, const float* tab, int hd, int rot, int pair) {
  // tab row: [cos(rot/2) | sin(rot/2)]
  const int half = rot / 2;
  const float* cs = tab;
  const float* sn = tab + half;
  if (pair == 0) {
    for (int i = 0; i < half; ++i) {
      const float a = x[i], b = x[i + half];
      out[i] = a * cs[i] - b * sn[i];
      out[i + half] = b * cs[i] + a * sn[i];
    }
  } else {
    for (int i = 0; i < half; ++i) {
      const float a = x[2 * i], b = x[2 * i + 1];
      out[2 * i] = a * cs[i] - b * sn[i];
      out[2 * i + 1] = b * cs[i] + a * sn[i];
    }
  }
  for (int i = rot; i < hd; ++i) out[i] = x[i];
}

void op_rope_kv(const Ctx& c) {
  float* qo = (float*)c.T(0);
  const float* qkv = (const float*)c.T(1);
  float* kc = (float*)c.T(2);
  float* vc = (float*)c.T(3);
  const float* qn = (const float*)c.T(4);
  const float* kn = (const float*)c.T(5);
  const float* rope = (const float*)c.T(6);
  const int nq = c.in->i[0], nkv = c.in->i[1], hd = c.in->i[2], rot = c.in->i[3], pair = c.in->i[4];
  const int gmode = c.in->i[6];
  const float eps = c.in->w[0].f;
  const StepIO& io = c.e->io;
  // gated attention: query heads arrive as [Q (hd) | gate (hd)] pairs and the gates are copied to t7 [rows][nq*hd]
  float* gate_out = c.in->i[7] ? (float*)c.T(7) : nullptr;
  const int qw = gate_out ? 2 * hd : hd;
  const int W = nq * qw + 2 * nkv * hd;
  std::vector<float> tmp(hd);
  int64_t a, b;
  c.range(io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const int pos = io.pos[r], slot = io.seq[r];
    const float* tab = rope + int64_t(pos) * rot;
    const int page = io.page_table[int64_t(slot) * io.max_pages + pos / PLOW_KV_PAGE];
    const int64_t cell = (int64_t(page) * PLOW_KV_PAGE + pos % PLOW_KV_PAGE) * nkv * hd;
    const float* row = qkv + r * W;
    for (int h = 0; h < nq; ++h) {
      const float* src = row + h * qw;
      if (gate_out) std::memcpy(gate_out + (r * nq + h) * hd, src + hd, sizeof(float) * hd);
      if (qn) { rmsnorm_row(tmp.data(), src, qn, hd, eps, gmode); src = tmp.data(); }
      rope_head(qo + (r * nq + h) * hd, src, tab, hd, rot, pair);
    }
    const float* kv_row = row + nq * qw;
    for (int h = 0; h < nkv; ++h) {
      const float* src = kv_row + h * hd;
      if (kn) { rmsnorm_row(tmp.data(), src, kn, hd, eps, gmode); src = tmp.data(); }
      rope_head(kc + cell + h * hd, src, tab, hd, rot, pair);
      std::memcpy(vc + cell + h * hd, kv_row + (nkv + h) * hd, sizeof(float) * hd);
    }
  }
}

void op_attn(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* q = (const float*)c.T(1);
  const float* kc = (const float*)c.T(2);
  const float* vc = (const float*)c.T(3);
  const int nq = c.in->i[0], nkv = c.in->i[1], hd = c.in->i[2], window = c.in->i[3];
  const float scale = c.in->w[0].f;
  const float* sinks = (const float*)c.T(5);      // optional: a logit per head that joins the softmax and carries no value
  const StepIO& io = c.e->io;
  const int group = nq / nkv;
  std::vector<float> sc;
  int64_t a, b;
  c.range(int64_t(io.rows) * nq, a, b);
  for (int64_t item = a; item < b; ++item) {
    const int64_t r = item / nq;
    const int h = int(item % nq), kvh = h / group;
    const int pos = io.pos[r], slot = io.seq[r];
    const int t0 = window > 0 ? std::max(0, pos - window + 1) : 0;
    const int n = pos - t0 + 1;
    sc.resize(n);
    const float* qr = q + (r * nq + h) * hd;
    float mx = -INFINITY;
    for (int t = t0; t <= pos; ++t) {
      const int page = io.page_table[int64_t(slot) * io.max_pages + t / PLOW_KV_PAGE];
      const float* kr = kc + ((int64_t(page) * PLOW_KV_PAGE + t % PLOW_KV_PAGE) * nkv + kvh) * hd;
      const float s = dotf(qr, kr, hd) * scale;
      sc[t - t0] = s;
      mx = std::max(mx, s);
    }
    if (sinks) mx = std::max(mx, sinks[h]);
    float den = sinks ? std::exp(sinks[h] - mx) : 0.f;
    for (int i = 0; i < n; ++i) { sc[i] = std::exp(sc[i] - mx); den += sc[i]; }
    float* o = out + (r * nq + h) * hd;
    for (int d = 0; d < hd; ++d) o[d] = 0.f;
    for (int t = t0; t <= pos; ++t) {
      const int page = io.page_table[int64_t(slot) * io.max_pages + t / PLOW_KV_PAGE];
      const float* vr = vc + ((int64_t(page) * PLOW_KV_PAGE + t % PLOW_KV_PAGE) * nkv + kvh) * hd;
      const float p = sc[t - t0] / den;
      for (int d = 0; d < hd; ++d) o[d] += p * vr[d];
    }
  }
}

void op_row_gather(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* x = (const float*)c.T(1);
  const int32_t* rows = (const int32_t*)c.T(2);
  const int W = c.in->i[0];
  int64_t a, b;
  c.range(c.e->io.n_sample, a, b);
  for (int64_t s = a; s < b; ++s) std::memcpy(out + s * W, x + int64_t(rows[s]) * W, sizeof(float) * W);
}

void op_argmax(const Ctx& c) {
  int32_t* out = (int32_t*)c.T(0);
  const float* lg = (const float*)c.T(1);
  const int V = c.in->i[0];
  int64_t a, b;
  c.range(c.e->io.n_sample, a, b);
  for (int64_t s = a; s < b; ++s) {
    const float* row = lg + s * V;
    int best = 0;
    for (int j = 1; j < V; ++j)
      if (row[j] > row[best]) best = j;  // strict: lowest index wins ties
    out[s] = best;
  }
}

void op_glu(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* g = (const float*)c.T(1);
  const float* u = (const float*)c.T(2);
  const PlowTensorEnt& te = c.e->pkt->tensors[c.in->t[0]];
  const int W = int(te.dims[1]);
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  const uint32_t act = c.in->i[0];
  for (int64_t k = a * W; k < b * W; ++k) out[k] = glu_act(g[k], act) * u[k];
}


// ---- gated delta rule (golden f32) ---------------------------------------------------------------------------------
// t0=out [rows][hv*d]  t1=conv state [slots][C][conv-1] (oldest input first)  t2=recurrent state [slots][hv][d(V)][d(K)]
// t3=qkvz [rows][(2hk+hv)d | hv*d]  t4=ba [rows][hv | hv]  t5=conv weight [C][conv]  t6=A_log [hv]  t7=dt_bias [hv]
// i0=hk i1=hv i2=d i3=conv.  Per token: causal depthwise conv + SiLU over the packed q|k|v channels, q and k L2-normalised,
// S <- alpha S; S += beta (v - S k) k^T; out = S q / sqrt(d).  A row at position 0 starts its slot from zero state.
// Work is split by slot (the state of a sequence is touched by one entry only); rows of a slot come in position order.
// Reference semantics: runtime/nvidia/op_qwen_gdn.cuh, runtime/common/dev_isa.h:1259-1280.
// Kimi Delta Attention step (GDN_STEP with i4 = 1): t3 = [q | k | v | beta_raw] rows ([3*H*D + H]), t4 = raw forget gate
// [H*D], t5 = conv weights [3*H*D][W], t6 = A_log [H], t7 = dt_bias [H*D]; f0 < 0 selects the bounded gate.
// Per head: S <- (I - beta k k^T) diag(exp(g)) S + beta k v^T, o = S^T q, with the state kept value-first [H][v][k].
static void op_kda(const Ctx& c) {
  float* out = (float*)c.T(0);
  float* conv_state = (float*)c.T(1);
  float* ssm = (float*)c.T(2);
  const float* qkvb = (const float*)c.T(3);
  const float* graw = (const float*)c.T(4);
  const float* cw = (const float*)c.T(5);
  const float* a_log = (const float*)c.T(6);
  const float* dt_bias = (const float*)c.T(7);
  const int H = c.in->i[0], d = c.in->i[2], conv = c.in->i[3];
  const float floor_g = c.in->w[0].f;
  const int C = 3 * H * d, Wr = C + H, hist = conv - 1;
  const StepIO& io = c.e->io;
  std::vector<float> x(C), dec(d), pred(d);
  for (int64_t r = 0; r < io.rows; ++r) {
    const int slot = io.seq[r], pos = io.pos[r];
    if (pos < 0 || slot % c.ns < c.s0 || slot % c.ns >= c.s1) continue;
    float* hs = conv_state + int64_t(slot) * C * hist;
    float* S = ssm + int64_t(slot) * H * d * d;
    if (pos == 0) {
      std::fill(hs, hs + int64_t(C) * hist, 0.f);
      std::fill(S, S + int64_t(H) * d * d, 0.f);
    }
    const float* row = qkvb + r * Wr;
    for (int ch = 0; ch < C; ++ch) {
      float* h = hs + int64_t(ch) * hist;
      float acc = cw[ch * conv + hist] * row[ch];
      for (int j = 0; j < hist; ++j) acc += cw[ch * conv + j] * h[j];
      for (int j = 0; j + 1 < hist; ++j) h[j] = h[j + 1];
      if (hist > 0) h[hist - 1] = row[ch];
      x[ch] = acc / (1.0f + std::exp(-acc));
    }
    for (int h = 0; h < 2 * H; ++h) {           // q heads, then k heads: x / sqrt(sum x^2 + 1e-6)
      float* v = x.data() + h * d;
      const float rs = 1.0f / std::sqrt(dotf(v, v, d) + 1e-6f);
      for (int i = 0; i < d; ++i) v[i] *= rs;
    }
    const float scale = 1.0f / std::sqrt(float(d));
    for (int h = 0; h < H; ++h) {
      const float* q = x.data() + h * d;
      const float* k = x.data() + (H + h) * d;
      const float* v = x.data() + (2 * H + h) * d;
      const float beta = 1.0f / (1.0f + std::exp(-row[C + h]));
      const float ea = std::exp(a_log[h]);
      for (int j = 0; j < d; ++j) {
        const float al = graw[(r * H + h) * d + j] + dt_bias[h * d + j];
        float g;
        if (floor_g < 0.f) {
          g = floor_g / (1.0f + std::exp(-ea * al));
        } else {
          const float sp = al > 20.f ? al : std::log1p(std::exp(al));
          g = -ea * sp;
        }
        dec[j] = std::exp(g);
      }
      float* Sh = S + int64_t(h) * d * d;
      for (int i = 0; i < d; ++i) {
        float* Sr = Sh + int64_t(i) * d;
        for (int j = 0; j < d; ++j) Sr[j] *= dec[j];
        pred[i] = dotf(Sr, k, d);
      }
      for (int i = 0; i < d; ++i) {
        float* Sr = Sh + int64_t(i) * d;
        const float u = beta * (v[i] - pred[i]);
        for (int j = 0; j < d; ++j) Sr[j] += u * k[j];
        out[(r * H + h) * d + i] = dotf(Sr, q, d) * scale;
      }
    }
  }
}

void op_gdn(const Ctx& c) {
  if (c.in->i[4] == 1) { op_kda(c); return; }
  float* out = (float*)c.T(0);
  float* conv_state = (float*)c.T(1);
  float* ssm = (float*)c.T(2);
  const float* qkvz = (const float*)c.T(3);
  const float* ba = (const float*)c.T(4);
  const float* cw = (const float*)c.T(5);
  const float* a_log = (const float*)c.T(6);
  const float* dt_bias = (const float*)c.T(7);
  const int hk = c.in->i[0], hv = c.in->i[1], d = c.in->i[2], conv = c.in->i[3];
  const int C = (2 * hk + hv) * d, Wq = C + hv * d, rep = hv / hk, hist = conv - 1;
  const StepIO& io = c.e->io;
  std::vector<float> x(C), pred(d);
  for (int64_t r = 0; r < io.rows; ++r) {
    const int slot = io.seq[r], pos = io.pos[r];
    if (pos < 0 || slot % c.ns < c.s0 || slot % c.ns >= c.s1) continue;
    float* hs = conv_state + int64_t(slot) * C * hist;
    float* S = ssm + int64_t(slot) * hv * d * d;
    if (pos == 0) {
      std::fill(hs, hs + int64_t(C) * hist, 0.f);
      std::fill(S, S + int64_t(hv) * d * d, 0.f);
    }
    const float* row = qkvz + r * Wq;
    for (int ch = 0; ch < C; ++ch) {
      float* h = hs + int64_t(ch) * hist;
      float acc = cw[ch * conv + hist] * row[ch];
      for (int j = 0; j < hist; ++j) acc += cw[ch * conv + j] * h[j];
      for (int j = 0; j + 1 < hist; ++j) h[j] = h[j + 1];
      if (hist > 0) h[hist - 1] = row[ch];
      x[ch] = acc / (1.0f + std::exp(-acc));
    }
    for (int h = 0; h < 2 * hk; ++h) {          // q heads, then k heads: x / sqrt(sum x^2 + 1e-6)
      float* v = x.data() + h * d;
      const float rs = 1.0f / std::sqrt(dotf(v, v, d) + 1e-6f);
      for (int i = 0; i < d; ++i) v[i] *= rs;
    }
    const float scale = 1.0f / std::sqrt(float(d));
    for (int h = 0; h < hv; ++h) {
      const float* q = x.data() + (h / rep) * d;
      const float* k = x.data() + (hk + h / rep) * d;
      const float* v = x.data() + 2 * hk * d + h * d;
      const float beta = 1.0f / (1.0f + std::exp(-ba[r * 2 * hv + h]));
      const float al = ba[r * 2 * hv + hv + h] + dt_bias[h];
      const float sp = al > 20.f ? al : std::log1p(std::exp(al));
      const float alpha = std::exp(-std::exp(a_log[h]) * sp);
      float* Sh = S + int64_t(h) * d * d;
      for (int i = 0; i < d; ++i) {
        float* Sr = Sh + int64_t(i) * d;
        for (int j = 0; j < d; ++j) Sr[j] *= alpha;
        pred[i] = dotf(Sr, k, d);
      }
      for (int i = 0; i < d; ++i) {
        float* Sr = Sh + int64_t(i) * d;
        const float u = beta * (v[i] - pred[i]);
        for (int j = 0; j < d; ++j) Sr[j] += u * k[j];
        out[(r * hv + h) * d + i] = dotf(Sr, q, d) * scale;
      }
    }
  }
}

// t0=out t1=o [rows][heads*hd] t2=z source (columns z_offset.. of its rows) t3=gamma [hd]; i0=heads i1=hd i2=z_offset
// i3=gate (0 silu, 1 sigmoid); f0=eps:  out = rmsnorm_per_head(o) * gamma * gate(z)
void op_gated_norm(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* o = (const float*)c.T(1);
  const float* zsrc = (const float*)c.T(2);
  const float* gamma = (const float*)c.T(3);
  const int heads = c.in->i[0], hd = c.in->i[1], zo = c.in->i[2];
  const bool sig = c.in->i[3] == 1;
  const float eps = c.in->w[0].f;
  const int zw = int(c.e->pkt->tensors[c.in->t[2]].dims[1]);
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t r = a; r < b; ++r)
    for (int h = 0; h < heads; ++h) {
      const float* x = o + (r * heads + h) * hd;
      const float* z = zsrc + r * zw + zo + h * hd;
      const float rs = 1.0f / std::sqrt(dotf(x, x, hd) / hd + eps);
      for (int i = 0; i < hd; ++i) out[(r * heads + h) * hd + i] = x[i] * rs * gamma[i] * ((sig ? 1.0f : z[i]) / (1.0f + std::exp(-z[i])));
    }
}

// t0=out t1=a t2=gate: out = a * sigmoid(gate)
void op_sigmoid_gate(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* x = (const float*)c.T(1);
  const float* g = (const float*)c.T(2);
  const int W = int(c.e->pkt->tensors[c.in->t[0]].dims[1]);
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t k = a * W; k < b * W; ++k) out[k] = x[k] / (1.0f + std::exp(-g[k]));
}

// ---- multi-head latent attention (golden f32; cache row = [c_kv (kv_lora) | k_rope (qk_rope)]) -----------------
// Reference semantics: runtime/nvidia/op_mla.cuh:23-42 (absorbed scores over the latent cache, W_uv folded once).
void op_mla_kv_write(const Ctx& c) {
  float* cache = (float*)c.T(0);
  const float* kva = (const float*)c.T(1);
  const float* gamma = (const float*)c.T(2);
  const float* rope = (const float*)c.T(3);
  const int L = c.in->i[0], R = c.in->i[1], pair = c.in->i[2], co = c.in->i[5];
  const StepIO& io = c.e->io;
  const int pitch = c.in->i[6] ? int(c.in->i[6]) : L + R;
  const float eps = c.in->w[0].f;
  int64_t a, b;
  c.range(io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const int pos = io.pos[r], slot = io.seq[r];
    const int page = io.page_table[int64_t(slot) * io.max_pages + pos / PLOW_KV_PAGE];
    float* dst = cache + (int64_t(page) * PLOW_KV_PAGE + pos % PLOW_KV_PAGE) * (L + R);
    const float* src = kva + r * pitch + co;
    rmsnorm_row(dst, src, gamma, L, eps, 0);
    rope_head(dst + L, src + L, rope + int64_t(pos) * R, R, R, pair);
  }
}

void op_mla_attn(const Ctx& c) {
  float* out = (float*)c.T(0);
  const float* q = (const float*)c.T(1);
  const float* rope = (const float*)c.T(2);
  const float* wkvb = (const float*)c.T(4);
  const float* cache = (const float*)c.T(5);
  const int H = c.in->i[0], L = c.in->i[1], NP = c.in->i[2], RP = c.in->i[3], V = c.in->i[4], pair = c.in->i[5];
  const float scale = c.in->w[0].f;
  const StepIO& io = c.e->io;
  const int qh = NP + RP, row = L + RP;
  // sparse attention: the indexer's selection [rows][top_k] (ascending positions, -1 padded) replaces "every position"
  // (operand 6 is the cache's scale tensor when the cache is e4m3 and the selection follows it; this backend's caches
  // are f32 and have no scale tensor, so the selection is operand 6)
  const int sel_op = c.in->t[7] != PLOW_T_NONE ? 7 : 6;
  const int32_t* sel = (c.in->i[6] != 0) ? (const int32_t*)c.T(sel_op) : nullptr;
  const int top_k = sel ? int(c.e->pkt->tensors[c.in->t[sel_op]].dims[1]) : 0;
  std::vector<int> keys;
  std::vector<float> qabs(L), qr(RP), olat(L), sc;
  int64_t a, b;
  c.range(int64_t(io.rows) * H, a, b);
  for (int64_t item = a; item < b; ++item) {
    const int64_t r = item / H;
    const int h = int(item % H);
    const int pos = io.pos[r], slot = io.seq[r];
    const float* qv = q + (r * H + h) * qh;
    const float* wuk = wkvb + int64_t(h) * (NP + V) * L;        // [NP][L]
    const float* wuv = wuk + int64_t(NP) * L;                   // [V][L]
    for (int j = 0; j < L; ++j) {
      float s = 0.f;
      for (int d = 0; d < NP; ++d) s += qv[d] * wuk[int64_t(d) * L + j];
      qabs[j] = s;
    }
    rope_head(qr.data(), qv + NP, rope + int64_t(pos) * RP, RP, RP, pair);
    keys.clear();
    if (sel) {
      for (int j = 0; j < top_k; ++j) {
        const int t = sel[r * top_k + j];
        if (t >= 0 && t <= pos) keys.push_back(t);
      }
    } else {
      for (int t = 0; t <= pos; ++t) keys.push_back(t);
    }
    sc.resize(keys.size());
    float mx = -INFINITY;
    for (size_t n = 0; n < keys.size(); ++n) {
      const int t = keys[n];
      const int page = io.page_table[int64_t(slot) * io.max_pages + t / PLOW_KV_PAGE];
      const float* kr = cache + (int64_t(page) * PLOW_KV_PAGE + t % PLOW_KV_PAGE) * row;
      sc[n] = (dotf(qabs.data(), kr, L) + dotf(qr.data(), kr + L, RP)) * scale;
      mx = std::max(mx, sc[n]);
    }
    float den = 0.f;
    std::fill(olat.begin(), olat.end(), 0.f);
    for (size_t n = 0; n < keys.size(); ++n) {
      const int t = keys[n];
      const float p = std::exp(sc[n] - mx);
      den += p;
      const int page = io.page_table[int64_t(slot) * io.max_pages + t / PLOW_KV_PAGE];
      const float* kr = cache + (int64_t(page) * PLOW_KV_PAGE + t % PLOW_KV_PAGE) * row;
      for (int j = 0; j < L; ++j) olat[j] += p * kr[j];
    }
    float* o = out + (r * H + h) * V;
    for (int d = 0; d < V; ++d) o[d] = dotf(wuv + int64_t(d) * L, olat.data(), L) / den;
  }
}

// ---- sparse-attention indexer (golden, f32; runtime/common/dev_isa.h:516-534, 1083-1115) ----------------------------
// Index key of every new row: LayerNorm (with bias) of the projected key, RoPE on the first `rot` dims (halves
// pairing), stored in the paged index-key cache (the scale tensor is 1 on this backend).
void op_dsa_index(const Ctx& c) {
  float* cache = (float*)c.T(0);
  float* cscale = (float*)c.T(1);
  const float* k = (const float*)c.T(2);
  const float* gamma = (const float*)c.T(3);
  const float* beta = (const float*)c.T(4);
  const float* rope = (const float*)c.T(5);
  const int D = c.in->i[0], rot = c.in->i[1];
  const StepIO& io = c.e->io;
  std::vector<float> y(D);
  int64_t a, b;
  c.range(io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const int pos = io.pos[r], slot = io.seq[r];
    const float* x = k + r * D;
    float mean = 0.f;
    for (int j = 0; j < D; ++j) mean += x[j];
    mean /= D;
    float var = 0.f;
    for (int j = 0; j < D; ++j) var += (x[j] - mean) * (x[j] - mean);
    const float rs = 1.0f / std::sqrt(var / D + 1e-6f);
    for (int j = 0; j < D; ++j) y[j] = (x[j] - mean) * rs * gamma[j] + beta[j];
    const int page = io.page_table[int64_t(slot) * io.max_pages + pos / PLOW_KV_PAGE];
    const int64_t cell = int64_t(page) * PLOW_KV_PAGE + pos % PLOW_KV_PAGE;
    rope_head(cache + cell * D, y.data(), rope + int64_t(pos) * rot, D, rot, 0);
    if (cscale) cscale[cell] = 1.0f;
  }
}

// Selection of every row: score[t] = sum_h w[h] relu(q_h . k_t) over the visible positions, the top_k best (ties to
// the lower position), written in ascending position order and padded with -1.
void op_dsa_topk(const Ctx& c) {
  int32_t* sel = (int32_t*)c.T(0);
  const float* q = (const float*)c.T(1);
  const float* w = (const float*)c.T(2);
  const float* cache = (const float*)c.T(3);
  const float* rope = (const float*)c.T(5);
  const int NH = c.in->i[0], D = c.in->i[1], K = c.in->i[2], rot = c.in->i[3];
  const StepIO& io = c.e->io;
  std::vector<float> qr(size_t(NH) * D), sc;
  std::vector<int> order;
  int64_t a, b;
  c.range(io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const int pos = io.pos[r], slot = io.seq[r];
    int32_t* out = sel + r * K;
    const int n = pos + 1;
    if (n <= K) {
      for (int j = 0; j < K; ++j) out[j] = j < n ? j : -1;
      continue;
    }
    for (int h = 0; h < NH; ++h) rope_head(qr.data() + size_t(h) * D, q + (r * NH + h) * D, rope + int64_t(pos) * rot, D, rot, 0);
    sc.assign(n, 0.f);
    for (int t = 0; t < n; ++t) {
      const int page = io.page_table[int64_t(slot) * io.max_pages + t / PLOW_KV_PAGE];
      const float* kt = cache + (int64_t(page) * PLOW_KV_PAGE + t % PLOW_KV_PAGE) * D;
      float s = 0.f;
      for (int h = 0; h < NH; ++h) s += w[r * NH + h] * std::max(0.f, dotf(qr.data() + size_t(h) * D, kt, D));
      sc[t] = s;
    }
    order.resize(n);
    for (int t = 0; t < n; ++t) order[t] = t;
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return sc[x] > sc[y]; });
    std::sort(order.begin(), order.begin() + K);
    for (int j = 0; j < K; ++j) out[j] = order[j];
  }
}

// ---- MoE router + experts (golden).  Selection key = score + bias, gate = unbiased score; group-limited: group score =
// sum of its two largest biased scores, lowest id wins ties (crates/packet/src/moe.rs:97-160).
void op_router_topk(const Ctx& c) {
  int32_t* table = (int32_t*)c.T(0);
  const float* logits = (const float*)c.T(1);
  const float* bias = (const float*)c.T(2);
  const int E = c.in->i[0], K = c.in->i[1], NG = std::max(1, int(c.in->i[2])), TG = std::max(1, int(c.in->i[3]));
  const bool sigmoid = c.in->i[4] != 0, norm = c.in->i[5] != 0;
  const float route_scale = c.in->w[0].f;
  std::vector<float> score(E), sel(E);
  std::vector<char> keep(NG);
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const float* lg = logits + r * E;
    if (sigmoid) {
      for (int e = 0; e < E; ++e) score[e] = 1.0f / (1.0f + std::exp(-lg[e]));
    } else {
      float mx = -INFINITY, den = 0.f;
      for (int e = 0; e < E; ++e) mx = std::max(mx, lg[e]);
      for (int e = 0; e < E; ++e) { score[e] = std::exp(lg[e] - mx); den += score[e]; }
      for (int e = 0; e < E; ++e) score[e] /= den;
    }
    for (int e = 0; e < E; ++e) sel[e] = score[e] + (bias ? bias[e] : 0.f);
    if (NG > 1) {
      const int per = E / NG;
      std::vector<float> gs(NG);
      for (int g = 0; g < NG; ++g) {
        float m1 = -INFINITY, m2 = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          if (sel[e] > m1) { m2 = m1; m1 = sel[e]; } else if (sel[e] > m2) { m2 = sel[e]; }
        }
        gs[g] = m1 + m2;
      }
      std::fill(keep.begin(), keep.end(), 0);
      for (int k = 0; k < TG; ++k) {
        int best = -1;
        for (int g = 0; g < NG; ++g) if (!keep[g] && (best < 0 || gs[g] > gs[best])) best = g;
        keep[best] = 1;
      }
      for (int e = 0; e < E; ++e) if (!keep[e / per]) sel[e] = -INFINITY;
    }
    float gsum = 0.f;
    int32_t* row = table + r * K * 2;
    std::vector<char> used(E, 0);
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int e = 0; e < E; ++e) if (!used[e] && (best < 0 || sel[e] > sel[best])) best = e;
      used[best] = 1;
      row[2 * k] = best;
      gsum += score[best];
    }
    for (int k = 0; k < K; ++k) {
      float g = score[row[2 * k]];
      if (norm) g /= std::max(gsum, 1e-20f);
      g *= route_scale;
      std::memcpy(&row[2 * k + 1], &g, 4);
    }
  }
}

void op_moe(const Ctx& c) {
  float* y = (float*)c.T(0);
  const float* h = (const float*)c.T(1);
  const int32_t* table = (const int32_t*)c.T(2);
  const float* w1 = (const float*)c.T(3);      // [E][2F][H]: gate rows then up rows per expert
  const float* w2 = (const float*)c.T(4);      // [E][H][F]
  const float* shared = (const float*)c.T(5);
  const float* b1 = (const float*)c.T(6);      // optional [E][2F]: gate biases then up biases per expert
  const float* b2 = (const float*)c.T(7);      // optional [E][H]
  const float limit = c.in->w[0].f, alpha = c.in->w[1].f;   // limit > 0: (up + 1) * g * sigmoid(alpha * g), clamped
  const int K = c.in->i[2], F = c.in->i[3];
  // i[6]: the shared expert is stacked behind the e_local routed ones and applies to every row with gate 1;
  // it is added first, where the separately computed shared output would have been
  const int shared_group = c.in->i[6] ? c.in->i[1] : -1;
  const PlowTensorEnt& te = c.e->pkt->tensors[c.in->t[0]];
  const int H = int(te.dims[1]);
  std::vector<float> glu(F), acc(H);
  int64_t a, b;
  c.range(c.e->io.rows, a, b);
  for (int64_t r = a; r < b; ++r) {
    const float* x = h + r * H;
    for (int j = 0; j < H; ++j) acc[j] = shared ? shared[r * H + j] : 0.f;
    for (int k = shared_group >= 0 ? -1 : 0; k < K; ++k) {                // fixed slot order
      int e = shared_group;
      float gate = 1.0f;
      if (k >= 0) {
        e = table[(r * K + k) * 2];
        std::memcpy(&gate, &table[(r * K + k) * 2 + 1], 4);
      }
      if (e < 0) continue;
      const float* wg = w1 + int64_t(e) * 2 * F * H;
      const float* wu = wg + int64_t(F) * H;
      for (int f = 0; f < F; ++f) {
        float gv = dotf(wg + int64_t(f) * H, x, H), uv = dotf(wu + int64_t(f) * H, x, H);
        if (b1) { gv += b1[int64_t(e) * 2 * F + f]; uv += b1[int64_t(e) * 2 * F + F + f]; }
        if (limit > 0.f) {
          gv = std::min(gv, limit);
          uv = std::max(-limit, std::min(uv, limit));
          glu[f] = (uv + 1.0f) * gv / (1.0f + std::exp(-alpha * gv));
        } else {
          glu[f] = gv / (1.0f + std::exp(-gv)) * uv;
        }
      }
      const float* wd = w2 + int64_t(e) * H * F;
      for (int j = 0; j < H; ++j) acc[j] += gate * (dotf(wd + int64_t(j) * F, glu.data(), F) + (b2 ? b2[int64_t(e) * H + j] : 0.f));
    }
    for (int j = 0; j < H; ++j) y[r * H + j] = acc[j];
  }
}

int exec_entry(Engine* e, const PlowInst* in, const PlowStreamEnt& se) {
  Ctx c{e, in, se.slice0, se.slice0 + se.nslice, in->nslice};
  switch (in->op) {
    case PLOW_OP_NOP: return 0;
    case PLOW_OP_EMBED: op_embed(c); return 0;
    case PLOW_OP_RMSNORM: {
      const PlowTensorEnt& te = e->pkt->tensors[in->t[0]];
      op_rmsnorm(c, te.dims[0] == -2 ? e->io.n_sample : e->io.rows);
      return 0;
    }
    case PLOW_OP_ADD_NORM: op_add_norm(c); return 0;
    case PLOW_OP_RESIDUAL: op_residual(c); return 0;
    case PLOW_OP_GEMM: {
      const PlowTensorEnt& te = e->pkt->tensors[in->t[0]];
      op_gemm(c, te.dims[0] == -2 ? e->io.n_sample : e->io.rows);
      return 0;
    }
    case PLOW_OP_ROPE_KV: op_rope_kv(c); return 0;
    case PLOW_OP_ATTN: op_attn(c); return 0;
    case PLOW_OP_ROW_GATHER: op_row_gather(c); return 0;
    case PLOW_OP_ARGMAX: op_argmax(c); return 0;
    case PLOW_OP_GLU: op_glu(c); return 0;
    case PLOW_OP_MLA_KV_WRITE: op_mla_kv_write(c); return 0;
    case PLOW_OP_MLA_DECODE:
    case PLOW_OP_MLA_PREFILL: op_mla_attn(c); return 0;
    case PLOW_OP_GDN_STEP: op_gdn(c); return 0;
    case PLOW_OP_GATED_NORM: op_gated_norm(c); return 0;
    case PLOW_OP_SIGMOID_GATE: op_sigmoid_gate(c); return 0;
    case PLOW_OP_DSA_INDEX: op_dsa_index(c); return 0;
    case PLOW_OP_DSA_TOPK: op_dsa_topk(c); return 0;
    case PLOW_OP_ROUTER_TOPK: op_router_topk(c); return 0;
    case PLOW_OP_MOE_GEMM: op_moe(c); return 0;
    default: return 100 + in->op;  // op not implemented on the CPU backend
  }
}

void run_worker_program(Engine* e, int tid) {
  const PlowProgramEnt& g = *e->prog;
  const uint8_t* base = e->pkt->raw.data();
  const PlowInst* insts = reinterpret_cast<const PlowInst*>(base + g.inst_ofs);
  const PlowStreamEnt* st = reinterpret_cast<const PlowStreamEnt*>(base + g.stream_ofs);
  const uint32_t* cu = reinterpret_cast<const uint32_t*>(base + g.cu_ofs);
  const PlowWait* waits = reinterpret_cast<const PlowWait*>(base + g.wait_ofs);
  const uint32_t* succs = reinterpret_cast<const uint32_t*>(base + g.succ_ofs);
  std::vector<uint32_t> pc, end, ids;
  for (uint32_t c = tid; c < g.n_cu; c += e->n_threads) { pc.push_back(cu[c]); end.push_back(cu[c + 1]); ids.push_back(c); }
  uint64_t last_progress = now_ns();
  size_t live = pc.size();
  while (live > 0 && e->status.load(std::memory_order_relaxed) == 0) {
    bool progressed = false;
    live = 0;
    for (size_t k = 0; k < pc.size(); ++k) {
      if (pc[k] >= end[k]) continue;
      ++live;
      const PlowStreamEnt& se = st[pc[k]];
      const uint64_t t_arrive = e->trace_on ? now_ns() : 0;
      bool ready = true;
      for (uint32_t w = 0; w < se.n_wait; ++w) {
        const PlowWait& pw = waits[se.wait_ofs + w];
        if (e->counters[size_t(pw.ctr) * PLOW_CTR_STRIDE_U32].load(std::memory_order_acquire) < pw.target) { ready = false; break; }
      }
      if (!ready) continue;
      const uint64_t t_ready = e->trace_on ? now_ns() : 0;
      const int rc = exec_entry(e, &insts[se.inst], se);
      if (rc) { e->status.store(rc); return; }
      for (uint32_t s = 0; s < se.n_succ; ++s)
        e->counters[size_t(succs[se.succ_ofs + s]) * PLOW_CTR_STRIDE_U32].fetch_add(1, std::memory_order_release);
      if (e->trace_on) {
        PlowTraceRec& tr = e->trace[pc[k]];
        tr.cu = ids[k]; tr.pc = pc[k] - cu[ids[k]]; tr.inst = se.inst; tr.op = insts[se.inst].op;
        tr.t_arrive = t_arrive; tr.t_ready = t_ready; tr.t_end = now_ns();
      }
      ++pc[k];
      progressed = true;
    }
    if (progressed) last_progress = now_ns();
    else if (live) {
      if ((now_ns() - last_progress) * 1e-9 > e->watchdog_s) { e->status.store(2); return; }  // unsatisfiable wait
      std::this_thread::yield();
    }
  }
}

void worker_main(Engine* e, int tid) {
  uint64_t seen = 0;
  while (true) {
    {
      std::unique_lock<std::mutex> lk(e->mu);
      e->cv_start.wait(lk, [&] { return e->quit || e->generation != seen; });
      if (e->quit) return;
      seen = e->generation;
    }
    run_worker_program(e, tid);
    {
      std::lock_guard<std::mutex> lk(e->mu);
      if (--e->pending == 0) e->cv_done.notify_all();
    }
  }
}

}  // namespace

extern "C" {

uint64_t plow_abi_sizeof(const char* name) {
  const std::string n(name);
  if (n == "PlowInst") return sizeof(PlowInst);
  if (n == "PlowStreamEnt") return sizeof(PlowStreamEnt);
  if (n == "PlowWait") return sizeof(PlowWait);
  if (n == "PlowTraceRec") return sizeof(PlowTraceRec);
  if (n == "PlowPktHeader") return sizeof(PlowPktHeader);
  if (n == "PlowTensorEnt") return sizeof(PlowTensorEnt);
  if (n == "PlowProgramEnt") return sizeof(PlowProgramEnt);
  if (n == "PlowSectionEnt") return sizeof(PlowSectionEnt);
  return 0;
}

int plow_abi_constant(const char* name) {
  const std::string n(name);
#define C(x) if (n == #x) return int(x);
  C(PLOW_OP_NOP) C(PLOW_OP_EMBED) C(PLOW_OP_RMSNORM) C(PLOW_OP_ADD_NORM) C(PLOW_OP_GEMM) C(PLOW_OP_ROPE_KV)
  C(PLOW_OP_ATTN) C(PLOW_OP_ROW_GATHER) C(PLOW_OP_ARGMAX) C(PLOW_OP_SAMPLE) C(PLOW_OP_RESIDUAL) C(PLOW_OP_GLU)
  C(PLOW_OP_QUANT_ACT) C(PLOW_OP_MLA_KV_WRITE) C(PLOW_OP_MLA_Q_ROPE) C(PLOW_OP_MLA_DECODE) C(PLOW_OP_MLA_PREFILL)
  C(PLOW_OP_MLA_ABSORB_Q) C(PLOW_OP_MLA_FOLD_V) C(PLOW_OP_DSA_INDEX) C(PLOW_OP_DSA_TOPK) C(PLOW_OP_ROUTER_TOPK)
  C(PLOW_OP_MOE_ALIGN) C(PLOW_OP_MOE_GATHER) C(PLOW_OP_MOE_GEMM) C(PLOW_OP_MOE_COMBINE) C(PLOW_OP_GDN_CONV)
  C(PLOW_OP_GDN_GATES) C(PLOW_OP_GDN_STEP) C(PLOW_OP_GDN_CHUNK) C(PLOW_OP_GATED_NORM) C(PLOW_OP_SIGMOID_GATE)
  C(PLOW_OP_XREDUCE) C(PLOW_OP_XREDUCE_ADD_NORM) C(PLOW_OP_XGATHER) C(PLOW_OP_XREDUCE_SCATTER)
  C(PLOW_OP_XA2A_DISPATCH) C(PLOW_OP_XA2A_COMBINE) C(PLOW_OP_XARGMAX_FIN) C(PLOW_OP_GEMM_XREDUCE)
  C(PLOW_OP_XGATHER_GEMM) C(PLOW_OP__COUNT)
  C(PLOW_PKT_VERSION) C(PLOW_CTR_STRIDE_U32) C(PLOW_KV_PAGE) C(PLOW_T_NONE)
  C(PLOW_GEMM_DUAL_SILU) C(PLOW_GEMM_FP8_BLOCK) C(PLOW_GEMM_OUT_F32) C(PLOW_GEMM_RESIDUAL) C(PLOW_GEMM_QUANT_OUT)
  C(PLOW_TC_WEIGHT) C(PLOW_TC_DERIVED) C(PLOW_TC_GEN) C(PLOW_TC_KV) C(PLOW_TC_STATE) C(PLOW_TC_ACT) C(PLOW_TC_INPUT)
  C(PLOW_TC_OUTPUT) C(PLOW_TC_PEER)
#undef C
  return -1;
}

void* plow_pkt_open(const char* path, char* err, int errlen) {
  FILE* f = std::fopen(path, "rb");
  if (!f) { std::snprintf(err, errlen, "cannot open %s", path); return nullptr; }
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  Pkt* p = nullptr;
  try {
    p = new Pkt;
    p->raw.resize(n < 0 ? 0 : n);
    const size_t got = std::fread(p->raw.data(), 1, p->raw.size(), f);
    std::fclose(f);
    f = nullptr;
    if (got != p->raw.size()) { std::snprintf(err, errlen, "short read"); delete p; return nullptr; }
    const std::string e = validate(*p);
    if (!e.empty()) { std::snprintf(err, errlen, "%s", e.c_str()); delete p; return nullptr; }
    return p;
  } catch (const std::exception& ex) {
    if (f) std::fclose(f);
    delete p;
    std::snprintf(err, errlen, "cannot load the packet: %s", ex.what());
    return nullptr;
  }
}
void plow_pkt_close(void* p) { delete static_cast<Pkt*>(p); }
int plow_pkt_n_tensor(void* p) { return static_cast<Pkt*>(p)->hdr->n_tensor; }
int plow_pkt_n_program(void* p) { return static_cast<Pkt*>(p)->hdr->n_program; }
const char* plow_pkt_tensor_name(void* p, int i) {
  Pkt* k = static_cast<Pkt*>(p);
  return k->strtab + k->tensors[i].name_ofs;
}

// null when the host cannot hold the packet's arena or start its threads (nothing is thrown across the C boundary)
void* plow_cpu_engine_create(void* pkt, int n_threads) {
  Engine* e = nullptr;
  try {
    e = new Engine;
    e->pkt = static_cast<Pkt*>(pkt);
    e->n_threads = n_threads < 1 ? 1 : n_threads;
    e->bound.assign(e->pkt->hdr->n_tensor, nullptr);
    e->arena.resize(e->pkt->hdr->act_arena_bytes + 256);
    for (int t = 0; t < e->n_threads; ++t) e->workers.emplace_back(worker_main, e, t);
    return e;
  } catch (const std::exception&) {
    if (e) {
      {
        std::lock_guard<std::mutex> lk(e->mu);
        e->quit = true;
      }
      e->cv_start.notify_all();
      for (auto& w : e->workers) w.join();
      delete e;
    }
    return nullptr;
  }
}
void plow_cpu_engine_destroy(void* h) {
  Engine* e = static_cast<Engine*>(h);
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->quit = true;
  }
  e->cv_start.notify_all();
  for (auto& w : e->workers) w.join();
  delete e;
}
int plow_cpu_bind(void* h, int handle, void* ptr) {
  Engine* e = static_cast<Engine*>(h);
  if (handle < 0 || size_t(handle) >= e->bound.size()) return -1;
  e->bound[handle] = ptr;
  return 0;
}
void plow_cpu_set_watchdog(void* h, double seconds) { static_cast<Engine*>(h)->watchdog_s = seconds; }
void plow_cpu_set_trace(void* h, int on) { static_cast<Engine*>(h)->trace_on = on != 0; }

// Runs one program to completion.  Returns 0, 1 = unbound tensor, 2 = watchdog (unsatisfiable
// wait), 100+op = opcode without a CPU body.
int plow_cpu_run(void* h, int program, const StepIO* io) {
  Engine* e = static_cast<Engine*>(h);
  if (program < 0 || uint32_t(program) >= e->pkt->hdr->n_program) return -1;
  e->prog = &e->pkt->programs[program];
  if (io->rows > int32_t(e->prog->rows)) return -2;
  e->io = *io;
  const PlowProgramEnt& g = *e->prog;
  const PlowInst* insts = reinterpret_cast<const PlowInst*>(e->pkt->raw.data() + g.inst_ofs);
  for (uint32_t i = 0; i < g.n_inst; ++i)
    for (int j = 0; j < 8; ++j) {
      const uint16_t t = insts[i].t[j];
      if (t != PLOW_T_NONE && e->pkt->tensors[t].tclass != PLOW_TC_ACT && !e->bound[t]) return 1;
    }
  std::vector<std::atomic<uint32_t>> ctr(size_t(g.n_ctr) * PLOW_CTR_STRIDE_U32);
  for (auto& c : ctr) c.store(0, std::memory_order_relaxed);
  e->counters.swap(ctr);
  e->status.store(0);
  if (e->trace_on) e->trace.assign(g.n_stream, PlowTraceRec{});
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->pending = e->n_threads;
    ++e->generation;
  }
  e->cv_start.notify_all();
  {
    std::unique_lock<std::mutex> lk(e->mu);
    e->cv_done.wait(lk, [&] { return e->pending == 0; });
  }
  return e->status.load();
}
int plow_cpu_trace(void* h, PlowTraceRec* out, int cap) {
  Engine* e = static_cast<Engine*>(h);
  const int n = std::min<int>(cap, int(e->trace.size()));
  std::memcpy(out, e->trace.data(), sizeof(PlowTraceRec) * n);
  return n;
}
// kernel tier of the GEMM op: 0 golden, 1 avx2, 2 avx512, 3 amx.  set returns the tier in force (an unsupported one is refused).
int plow_cpu_tier() { return cur_tier(); }
int plow_cpu_set_tier(int t) {
  if (t >= 0 && t <= TIER_AMX && tier_supported(t)) g_tier.store(t);
  return cur_tier();
}
void* plow_cpu_arena(void* h) { return static_cast<Engine*>(h)->arena.data(); }

}  // extern "C"
