// C ABI of the tcgen05 GEMM family (loaded from Python through ctypes).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct PlowGemmDesc {
  const void* x;          // [M, K] activations (bf16 or e4m3), row pitch ldx elements
  const void* w;          // [w_rows, K] weights, row pitch ldw elements
  void* y;                // [M, N] output (bf16, or f32 when out_f32); may be NULL with yq set
  const float* sx;        // e4m3: activation scales, transposed [ceil(K/128)][ld_sx]
  const float* sw;        // e4m3: weight scales [w_rows/128][ceil(K/128)]
  const void* residual;   // optional bf16 [M, N] (pitch ldy)
  void* yq;               // optional e4m3 output [M, N] (pitch ldy)
  float* syq;             // scales of yq, transposed [N/128][ld_syq]
  const int32_t* grp_off; // grouped: [E+1] row offsets (device)
  const int32_t* tile_prefix;  // grouped, swap=0: [E+1] prefix of 128-row tile counts (device)
  int32_t* status;        // device status word, 0 = ok
  int32_t M, N, K;
  int32_t ldx, ldw, ldy, ld_sx, ld_syq;
  int32_t E;              // experts (0 = dense)
  int64_t w_rows;         // rows of w (E * N * (dual ? 2 : 1), or N)
  int32_t dtype;          // 0 = bf16, 1 = e4m3 block-scaled
  int32_t dual;           // 1: silu(x w_gate^T) * (x w_up^T), w = [gate; up] per expert
  int32_t swap;           // 1: weights on the 128 TMEM lanes (small M)
  int32_t bn;             // UMMA N tile (tokens when swap, features otherwise)
  int32_t out_f32;
  float out_scale;
  float* ws;              // split-K workspace (fp32) and per-tile counters (zeroed once by the caller)
  int32_t* ws_ctr;
  int32_t splits;         // >1: split-K over CTAs (dense swap mode only)
  int32_t stream;         // 1: stream scheduling (swap mode): equal K-block ranges per CTA, partials through ws / ws_ctr
  // fused all-reduce over tensor-parallel ranks (swap mode, M <= bn, not dual): symmetric region of every
  // rank, byte offsets of the partial / flag / arrival / output areas inside it, launch-epoch word
  void* ar_peer[8];
  uint64_t ar_part_ofs, ar_flag_ofs, ar_done_ofs, ar_y_ofs;
  void* ar_epoch;
  int32_t ar_world, ar_me;
  const void* wait_ctr;   // optional arrival gate: start once *wait_ctr >= *wait_epoch * wait_mult
  const void* wait_epoch;
  int32_t wait_mult;
  int32_t wait_deadline_ms;
  int32_t ar_oneshot;     // fused all-reduce form: 0 = two-shot (owner reduces, stores to every rank), 1 = one-shot (push + local reduce)
  int32_t ar_pad;
  uint64_t ar_half_bytes; // one-shot: bytes of one parity half of the partial area; ar_epoch points at 4 device words
  void* ar_mc;            // ar_oneshot == 2: multicast (NVSwitch) mapping of the symmetric region
  uint64_t ar_tdone_ofs;  // ar_oneshot == 2: u32 [tiles] per-tile epoch words inside the region
} PlowGemmDesc;

// Launches on `stream` (a cudaStream_t).  Returns 0, or a host-side error code (<0 bad
// arguments, >=1000 tensor-map / launch failures).
int plow_gemm(const PlowGemmDesc* d, void* stream);

#ifdef __cplusplus
}
#endif
