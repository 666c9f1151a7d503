// Argument block of the expert-parallel kernels (csrc/comm/ep.cu); also read by the fused routing kernel
// (csrc/cuda/rowops.cu), whose last CTA publishes this rank's per-expert pair counts to every peer.
#pragma once
#include <stdint.h>

namespace plow {

struct EpLayout {         // byte offsets inside the symmetric region (identical on all ranks)
  uint64_t cnt_all;       // int32 [W][E]
  uint64_t cnt_flag;      // u32 [W] (stride 32 words)
  uint64_t data_ctr;      // u32
  uint64_t y_flag;        // u32 [W] (stride 32 words)
  uint64_t recv_x;        // u8  [Rmax][H]
  uint64_t recv_sx;       // f32 [H/128][Rmax]
  uint64_t y;             // bf16 [Rmax][H]
};

struct EpArgs {
  uint8_t* peer[8];
  EpLayout L;
  int W, me, E, e_local, Rmax, H;
  uint32_t* epoch;        // device word: layer-call counter (monotonic)
  int* status;
  unsigned long long deadline_ns;
  unsigned long long* trace;   // optional [1 + 2n] u64: count, then (tag, globaltimer) pairs (debug aid), NULL when off
};

}  // namespace plow
