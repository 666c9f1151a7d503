// Entry point of the GEMM family: argument checks, then dispatch to an instantiation.
#include "gemm_api.h"
#include "gemm_tc.cuh"

namespace plow {
int gemm_dispatch_bf16(const PlowGemmDesc& d, cudaStream_t s);
int gemm_dispatch_fp8(const PlowGemmDesc& d, cudaStream_t s);

#ifdef PLOW_DEVICE_TRACE
static long long* g_gemm_trace = nullptr;
#endif
GemmArgs to_args(const PlowGemmDesc& d) {
  GemmArgs a;
#ifdef PLOW_DEVICE_TRACE
  a.trace = g_gemm_trace;
#else
  a.trace = nullptr;
#endif
  a.x = d.x; a.w = d.w; a.y = d.y; a.sx = d.sx; a.sw = d.sw; a.residual = d.residual;
  a.yq = d.yq; a.syq = d.syq; a.grp_off = d.grp_off; a.tile_prefix = d.tile_prefix;
  a.status = d.status; a.M = d.M; a.N = d.N; a.K = d.K; a.ldy = d.ldy; a.ld_sx = d.ld_sx;
  a.ld_syq = d.ld_syq; a.E = d.E; a.out_f32 = d.out_f32; a.out_scale = d.out_scale;
  a.ws = d.ws; a.ws_ctr = d.ws_ctr;
  a.stream = (d.stream && d.swap && d.ws && d.ws_ctr && d.ar_world <= 1) ? 1 : 0;
  a.splits = (!a.stream && d.swap && d.E == 0 && d.ws && d.ws_ctr) ? d.splits : 1;
  for (int i = 0; i < 8; ++i) a.ar_peer[i] = static_cast<uint8_t*>(d.ar_peer[i]);
  a.ar_part_ofs = d.ar_part_ofs; a.ar_flag_ofs = d.ar_flag_ofs; a.ar_done_ofs = d.ar_done_ofs; a.ar_y_ofs = d.ar_y_ofs;
  a.ar_epoch = static_cast<uint32_t*>(d.ar_epoch); a.ar_world = d.ar_world; a.ar_me = d.ar_me;
  a.ar_oneshot = d.ar_oneshot; a.ar_half_bytes = d.ar_half_bytes;
  a.ar_mc = static_cast<uint8_t*>(d.ar_mc); a.ar_tdone_ofs = d.ar_tdone_ofs;
  a.wait_ctr = static_cast<const uint32_t*>(d.wait_ctr); a.wait_epoch = static_cast<const uint32_t*>(d.wait_epoch);
  a.wait_mult = static_cast<uint32_t>(d.wait_mult); a.wait_deadline_ms = static_cast<uint32_t>(d.wait_deadline_ms);
  return a;
}
}  // namespace plow

#ifdef PLOW_DEVICE_TRACE
// Builds with -DPLOW_DEVICE_TRACE only: device buffer of 64*8 int64 that CTA 0 fills with clock64() phase stamps.
extern "C" void plow_gemm_set_trace(void* p) { plow::g_gemm_trace = static_cast<long long*>(p); }
#endif

extern "C" int plow_gemm(const PlowGemmDesc* d, void* stream) {
  if (!d || !d->x || !d->w || !d->status || (!d->y && !d->yq)) return -1;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return -1;
  const int es = d->dtype == 1 ? 1 : 2;
  // TMA: 16-byte aligned bases and row pitches
  if ((reinterpret_cast<uintptr_t>(d->x) & 15) || (reinterpret_cast<uintptr_t>(d->w) & 15)) return -3;
  if (((d->ldx * es) & 15) || ((d->ldw * es) & 15)) return -3;
  if (d->dtype == 1 && (!d->sx || !d->sw)) return -4;
  if (d->E > 0 && !d->grp_off) return -5;
  if (d->E > 0 && !d->swap && !d->tile_prefix) return -5;
  if (d->E > 0 && (d->N % 128)) return -6;
  if (d->dual && (d->N % 128)) return -6;
  if (d->yq && !d->syq) return -7;
  if (d->yq && !d->swap && d->bn != 128 && !(d->bn == 256 && !d->dual)) return -7;
  if (d->ar_world > 1 && (!d->swap || d->dual || d->E || d->M > d->bn || d->splits > 1 || d->yq || d->out_f32 || !d->ar_epoch || (d->N % 8) || (d->ldy % 8))) return -8;
  if (d->ar_world > 1 && d->ar_oneshot == 2 && !d->ar_mc) return -8;
  if (d->ar_world > 1 && d->ar_oneshot == 1 &&
      static_cast<uint64_t>((d->N + 127) / 128) * d->ar_world * 128 * d->bn * 2 > d->ar_half_bytes) return -8;
  if (d->swap && d->E == 0 && d->splits > 1 && d->ws && d->ws_ctr && !d->stream) {
    // the CTAs of a split-K tile wait for one another: all tiles x splits of them must be resident at once
    const long long tiles = static_cast<long long>((d->N + 127) / 128) * ((d->M + d->bn - 1) / d->bn);
    if (tiles > 256 || tiles * d->splits > plow::sm_count()) return -9;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return d->dtype == 1 ? plow::gemm_dispatch_fp8(*d, s) : plow::gemm_dispatch_bf16(*d, s);
}
