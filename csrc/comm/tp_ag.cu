// Tensor-parallel all-gather that feeds a GEMM without a host or stream synchronisation in between.
//
// Sequence-parallel seam: after a row-parallel projection each rank holds a band of rows of the
// activation (rows [me*band, (me+1)*band)).  `ag_push` stores that band into the same rows of the
// gathered buffer of EVERY rank (16-byte stores over NVLink, so each band crosses every link once) and,
// when the last CTA of the grid has finished, adds one release arrival to every rank's counter.  The
// column-parallel GEMM that follows carries the wait inside the kernel (GemmArgs::wait_*: its TMA
// producer starts once the counter reaches epoch * world), so the gather of the slowest peer overlaps
// the GEMM's prologue and the weights' first tiles instead of a separate collective launch.
// Flags are monotonic device-side epochs (graph replayable); the wait is bounded in the GEMM.
// One gathered buffer is enough because reuse is handshaken on the device: after its GEMM every rank adds one release
// to every rank's release counter (`ag_release`), and a push of call n + 1 starts only once that counter shows that all
// ranks have finished reading call n (bounded wait, normally already satisfied).  Nothing depends on a host-side call
// count, so the sequence can be captured in a CUDA graph and replayed.
// Reference counterpart: runtime/amd/op_collective.h d_xall_gather_mega and the two-shot all-gather
// half in runtime/nvidia/op_collective.cuh:466-543.  Plain peer stores only.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace {
using namespace plow;

struct AgArgs {
  uint8_t* peer[8];
  uint64_t x_ofs;        // gathered buffer [rows][row_bytes] inside the symmetric region
  uint64_t ctr_ofs;      // u32 arrival counter
  uint32_t* epoch;       // device word, +1 per call
  uint32_t* done;        // device word: CTAs finished (reset by the last one)
  uint64_t rel_ofs;      // u32 release counter: +1 from every rank after it has consumed a call's gathered rows
  int* status;
  unsigned long long deadline_ns;
  int W, me;
  int band_rows, row_bytes;   // row_bytes % 16 == 0
};

__global__ void ag_push_kernel(const AgArgs a, const uint8_t* src, int ld_src_bytes) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  // every rank must be done reading the previous call's rows before they are overwritten
  __shared__ int fail;
  if (threadIdx.x == 0) {
    fail = 0;
    const uint32_t need = *a.epoch * static_cast<uint32_t>(a.W);
    const uint32_t* rel = reinterpret_cast<const uint32_t*>(a.peer[a.me] + a.rel_ofs);
    const unsigned long long t0 = globaltimer_ns();
    while (ld_acquire_sys(rel) < need) {
      if (globaltimer_ns() - t0 > a.deadline_ns) { fail = 1; atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagAg); break; }
      __nanosleep(128);
    }
  }
  __syncthreads();
  const int units = a.row_bytes / 16;
  const long long total = fail ? 0 : static_cast<long long>(a.band_rows) * units;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / units), u = static_cast<int>(i % units);
    const uint4 v = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * ld_src_bytes + u * 16);
    const size_t o = a.x_ofs + (static_cast<size_t>(a.me) * a.band_rows + r) * a.row_bytes + u * 16;
    for (int p = 0; p < a.W; ++p) *reinterpret_cast<uint4*>(a.peer[p] + o) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t n = atomicAdd(a.done, 1u);
    if (n == gridDim.x - 1) {
      *a.done = 0;
      *a.epoch += 1;
      __threadfence_system();
      for (int p = 0; p < a.W; ++p) red_add_release_sys(reinterpret_cast<uint32_t*>(a.peer[p] + a.ctr_ofs), 1u);
    }
  }
}

// After the consumer of a gathered buffer (the GEMM before this kernel in the stream) has finished: tell every rank.
__global__ void ag_release_kernel(const AgArgs a) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __threadfence_system();
  if (threadIdx.x < a.W) red_add_release_sys(reinterpret_cast<uint32_t*>(a.peer[threadIdx.x] + a.rel_ofs), 1u);
}

}  // namespace

extern "C" {

// peers: 8 pointers (host array) to the ranks' symmetric regions; src: this rank's band [band_rows][row_bytes].
int plow_ag_push(const void* const* peers, uint64_t x_ofs, uint64_t ctr_ofs, void* epoch, void* done, int world, int me,
                 const void* src, int ld_src_bytes, int band_rows, int row_bytes, uint64_t rel_ofs, int deadline_ms, int* status,
                 void* stream) {
  if (world < 1 || world > 8 || row_bytes % 16 || ld_src_bytes % 16 || band_rows <= 0 || !status) return -1;
  AgArgs a;
  for (int i = 0; i < 8; ++i) a.peer[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peers[i])) : nullptr;
  a.x_ofs = x_ofs; a.ctr_ofs = ctr_ofs; a.epoch = static_cast<uint32_t*>(epoch); a.done = static_cast<uint32_t*>(done);
  a.rel_ofs = rel_ofs; a.status = status; a.deadline_ns = static_cast<unsigned long long>(deadline_ms) * 1000000ull;
  a.W = world; a.me = me; a.band_rows = band_rows; a.row_bytes = row_bytes;
  const long long total = static_cast<long long>(band_rows) * (row_bytes / 16);
  int grid = static_cast<int>((total + 255) / 256);
  if (grid > 64) grid = 64;
  plow::launch_serial(ag_push_kernel, dim3(grid), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), a, static_cast<const uint8_t*>(src), ld_src_bytes);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// Launch after the kernel that consumed the gathered rows (same stream).
int plow_ag_release(const void* const* peers, uint64_t rel_ofs, int world, int me, void* stream) {
  if (world < 1 || world > 8) return -1;
  AgArgs a = {};
  for (int i = 0; i < 8; ++i) a.peer[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peers[i])) : nullptr;
  a.rel_ofs = rel_ofs; a.W = world; a.me = me;
  plow::launch_serial(ag_release_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
