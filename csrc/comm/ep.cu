// Expert-parallel token dispatch and combine over NVLink peer memory (one process per GPU).
//
// Every rank owns a symmetric region (same layout on all ranks, peers mapped into this address
// space).  Per MoE layer:
//   1. ep_counts   - histogram of this rank's (token, slot) pairs per expert, stored into every
//                    peer's count matrix, then one release flag per peer.
//   2. ep_push     - waits for all ranks' counts, derives the same global layout everywhere
//                    (rows of an expert ordered by source rank), and writes each local pair's
//                    quantised row + scales straight into the owning rank's expert-sorted
//                    buffer (st over NVLink); one release add per CTA on the owner's arrival
//                    counter.  The grouped expert GEMM of the owner waits on that counter from
//                    inside the kernel (GemmArgs::wait_*), so no host or stream sync separates
//                    dispatch from the expert GEMM.
//   3. ep_y_ready  - after the down projection, a release flag to every peer.
//   4. ep_combine  - each rank pulls its tokens' expert outputs from the owners' memory (ld over
//                    NVLink) and forms shared + sum_j gate_j * y_j in fixed slot order, f32.
// All flags are monotonic epochs kept in device memory, so the sequence can be replayed from a
// CUDA graph.  Every wait is bounded by a deadline; on expiry the kernel records
// PLOW_ERR_PEER_WAIT in the status word and returns, and the host fails the step.
//
// The reference's expert parallelism keeps whole experts per rank and combines with an
// all-reduce (crates/devgen/src/mla.rs:13016-13021, crates/packet/src/moe_ep.rs); its flag
// protocol (release store per peer, relaxed polling with a deadline, status line) is
// runtime/nvidia/op_collective.cuh:216-240.  Plain peer loads/stores only: no multimem and no
// TMA multicast anywhere in this file.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ep_args.h"
#include "ptx.cuh"

namespace {
using namespace plow;

__device__ __forceinline__ void trace_mark(const EpArgs& a, unsigned long long tag) {
  if (a.trace) {
    const unsigned long long i = atomicAdd(a.trace, 1ull);
    if (i < 4000) { a.trace[1 + 2 * i] = tag; a.trace[2 + 2 * i] = globaltimer_ns(); }
  }
}

__device__ __forceinline__ bool wait_ge(const uint32_t* p, uint32_t target, unsigned long long deadline_ns) {
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(p) < target) {
    if (globaltimer_ns() - t0 > deadline_ns) return false;
    __nanosleep(256);   // back off: the polled line is also the target of the peers' stores
  }
  return true;
}

// One warp copies a row of H bytes: up to eight 16-byte loads per lane are issued before the first store, so a row costs
// about one load round trip and one store burst instead of H / 512 dependent load -> store pairs (measured: the push of
// 576 rows took 30 us with the dependent form, most of it latency).
__device__ __forceinline__ void warp_copy_row(uint4* dst, const uint4* src, int n16, int lane) {
  for (int i0 = 0; i0 < n16; i0 += 256) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * 32 + lane;
      if (i < n16) v[u] = src[i];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * 32 + lane;
      if (i < n16) dst[i] = v[u];
    }
  }
}

__global__ void ep_counts_kernel(EpArgs a, const int2* table, int n_pairs, int* cursor) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ int hist[];
  if (threadIdx.x == 0) trace_mark(a, 1);
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) { hist[e] = 0; cursor[e] = 0; }   // cursor[E] is the push kernel's CTA counter
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&hist[table[p].x], 1);
  __syncthreads();
  const uint32_t ep = *a.epoch + 1;
  for (int d = 0; d < a.W; ++d) {
    int* dst = reinterpret_cast<int*>(a.peer[d] + a.L.cnt_all) + a.me * a.E;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) dst[e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.W)
    st_release_sys(reinterpret_cast<uint32_t*>(a.peer[threadIdx.x] + a.L.cnt_flag) + a.me * 32, ep);
  if (threadIdx.x == 0) { *a.epoch = ep; trace_mark(a, 2); }
}

// grid: any; 256 threads.  One warp per pair.
// shared_rows > 0: the shared expert is stacked behind this rank's routed experts as group e_local; its rows are this
// rank's own first `shared_rows` tokens, copied (locally) behind the routed rows, and grp_off / tile_prefix get one more entry.
__global__ void ep_push_kernel(EpArgs a, const int2* table, int n_pairs, int top_k, const uint8_t* xq, const float* sx,
                               int ld_sx, int* cursor, int* grp_off, int* tile_prefix, int* pair_dest, int shared_rows) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ int sm[];                 // cnt [W][E], base [E], tot [E]
  int* cnt = sm;
  int* base = sm + a.W * a.E;
  __shared__ int fail;
  if (threadIdx.x == 0) fail = 0;
  __syncthreads();
  const uint32_t ep = *a.epoch;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 3);
  if (threadIdx.x < a.W) {
    if (!wait_ge(reinterpret_cast<const uint32_t*>(a.peer[a.me] + a.L.cnt_flag) + threadIdx.x * 32, ep, a.deadline_ns)) fail = 1;
  }
  __syncthreads();
  if (fail) { if (threadIdx.x == 0) atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagEp); return; }
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 4);
  const int* call = reinterpret_cast<const int*>(a.peer[a.me] + a.L.cnt_all);
  int* tot = base + a.E;                      // [E] rows of expert e over all source ranks
  for (int i = threadIdx.x; i < a.W * a.E; i += blockDim.x) cnt[i] = __ldcg(call + i);
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 40);
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
    int c = 0;
    for (int s = 0; s < a.W; ++s) c += cnt[s * a.E + e];
    tot[e] = c;
  }
  __syncthreads();
  // base[e] = first row, on the owner of e, of the rows this rank sends for expert e
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
    const int e0 = (e / a.e_local) * a.e_local;
    int off = 0;
    for (int f = e0; f < e; ++f) off += tot[f];
    for (int s = 0; s < a.me; ++s) off += cnt[s * a.E + e];
    base[e] = off;
  }
  // layout of this rank's own experts: one thread per expert (exclusive prefix of rows and of 128-row tiles)
  __shared__ int routed_rows;     // rows this rank receives for its routed experts (same value in every CTA)
  for (int el = threadIdx.x; el <= a.e_local; el += blockDim.x) {
    int off = 0, tiles = 0;
    for (int f = 0; f < el; ++f) { const int c = tot[a.me * a.e_local + f]; off += c; tiles += (c + 127) >> 7; }
    if (el == a.e_local) routed_rows = off;
    if (blockIdx.x == 0) {
      grp_off[el] = off; tile_prefix[el] = tiles;
      if (el == a.e_local) {
        if (shared_rows > 0) { grp_off[el + 1] = off + shared_rows; tile_prefix[el + 1] = tiles + ((shared_rows + 127) >> 7); }
        if (off + shared_rows > a.Rmax) atomicCAS(a.status, 0, PLOW_ERR_BOUNDS | kTagEp);
      }
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int KB = a.H / 128;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 41);
  if (routed_rows + shared_rows <= a.Rmax) {
    for (int t = blockIdx.x * wpb + warp; t < shared_rows; t += gridDim.x * wpb) {
      const int row = routed_rows + t;
      const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<size_t>(t) * a.H);
      uint4* dst = reinterpret_cast<uint4*>(a.peer[a.me] + a.L.recv_x + static_cast<size_t>(row) * a.H);
      warp_copy_row(dst, src, a.H / 16, lane);
      float* dsx = reinterpret_cast<float*>(a.peer[a.me] + a.L.recv_sx);
      for (int kb = lane; kb < KB; kb += 32) dsx[static_cast<size_t>(kb) * a.Rmax + row] = sx[static_cast<size_t>(kb) * ld_sx + t];
    }
  }
  for (int p = blockIdx.x * wpb + warp; p < n_pairs; p += gridDim.x * wpb) {
    const int e = table[p].x;
    const int d = e / a.e_local;
    int idx = 0;
    if (lane == 0) idx = atomicAdd(&cursor[e], 1);
    idx = __shfl_sync(0xffffffffu, idx, 0);
    const int row = base[e] + idx;
    if (row >= a.Rmax) { if (lane == 0) atomicCAS(a.status, 0, PLOW_ERR_BOUNDS | kTagEp); continue; }
    const int tok = p / top_k;
    const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<size_t>(tok) * a.H);
    uint4* dst = reinterpret_cast<uint4*>(a.peer[d] + a.L.recv_x + static_cast<size_t>(row) * a.H);
    warp_copy_row(dst, src, a.H / 16, lane);
    float* dsx = reinterpret_cast<float*>(a.peer[d] + a.L.recv_sx);
    for (int kb = lane; kb < KB; kb += 32) dsx[static_cast<size_t>(kb) * a.Rmax + row] = sx[static_cast<size_t>(kb) * ld_sx + tok];
    if (lane == 0) pair_dest[p] = (d << 24) | row;
  }
  // One arrival per (source rank, owner): the CTA that finishes last signals for the whole kernel.
  // Every CTA makes its remote stores visible system-wide before it counts itself in, and the last
  // CTA's release add is ordered after all of those counts, so an owner that acquires the counter
  // sees every row this rank sent.  (One add per CTA made 256 remote atomics per layer fight with the
  // owner's pollers for one line: 1.3 ms per layer at 8 ranks.)
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 42);
  __threadfence_system();
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 43);
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const int old = atomicAdd(&cursor[a.E], 1);
    is_last = old == static_cast<int>(gridDim.x) - 1;
    if (is_last) cursor[a.E] = 0;
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    if (threadIdx.x < a.W) red_add_release_sys(reinterpret_cast<uint32_t*>(a.peer[threadIdx.x] + a.L.data_ctr), 1u);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 5);
}

__global__ void ep_y_ready_kernel(EpArgs a) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  if (threadIdx.x == 0) trace_mark(a, 6);
  __threadfence_system();
  const uint32_t ep = *a.epoch;
  if (threadIdx.x < a.W) st_release_sys(reinterpret_cast<uint32_t*>(a.peer[threadIdx.x] + a.L.y_flag) + a.me * 32, ep);
}

// shared_base != NULL: the shared expert ran as the last group of this rank's grouped GEMM; its output row of token t
// is row *shared_base + t of this rank's own y buffer (`shared` is ignored).
__global__ void ep_combine_kernel(EpArgs a, __nv_bfloat16* out, const __nv_bfloat16* shared, const int2* table,
                                  const int* pair_dest, int top_k, const int* shared_base, int signal_y) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ int fail;
  if (threadIdx.x == 0) fail = 0;
  __syncthreads();
  const uint32_t ep = *a.epoch;
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 7);
  if (signal_y && blockIdx.y == 0 && (blockIdx.x & 31) == 0) {
    // This rank's expert outputs were written by the kernel before this one in the stream: tell every rank they can
    // be pulled (a few CTAs repeat the same store, so the signal does not hinge on which CTA is scheduled first),
    // then wait for the others' signals like every other CTA.
    __threadfence_system();
    if (threadIdx.x < a.W) st_release_sys(reinterpret_cast<uint32_t*>(a.peer[threadIdx.x] + a.L.y_flag) + a.me * 32, ep);
  }
  if (threadIdx.x < a.W) {
    if (!wait_ge(reinterpret_cast<const uint32_t*>(a.peer[a.me] + a.L.y_flag) + threadIdx.x * 32, ep, a.deadline_ns)) fail = 1;
  }
  __syncthreads();
  if (fail) { if (threadIdx.x == 0) atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagEp); return; }
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 8);
  // Slot metadata first, then all of a thread's remote loads at once: the eight pulls of a 16-byte unit are
  // independent, so they cost one NVLink round trip instead of eight.  One unit per thread (grid.y covers H).
  constexpr int kMaxK = 16;
  __shared__ int s_dest[kMaxK];
  __shared__ float s_gate[kMaxK];
  const int t = blockIdx.x;
  if (threadIdx.x < top_k && threadIdx.x < kMaxK) {
    s_dest[threadIdx.x] = pair_dest[t * top_k + threadIdx.x];
    s_gate[threadIdx.x] = __int_as_float(table[t * top_k + threadIdx.x].y);
  }
  __syncthreads();
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i < a.H) {
    uint4 v[kMaxK];
#pragma unroll
    for (int s = 0; s < kMaxK; ++s) {
      if (s < top_k) {
        const int pd = s_dest[s];
        const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(a.peer[pd >> 24] + a.L.y);
        v[s] = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(pd & 0xffffff) * a.H + i);
      }
    }
    float acc[8];
    if (shared_base) shared = reinterpret_cast<const __nv_bfloat16*>(a.peer[a.me] + a.L.y) + static_cast<size_t>(*shared_base) * a.H;
    if (shared) {
      const uint4 sv = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * a.H + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&sv);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
#pragma unroll
    for (int s = 0; s < kMaxK; ++s) {          // fixed slot order
      if (s < top_k) {
        const float g = s_gate[s];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] += g * f.x; acc[2 * j + 1] += g * f.y; }
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * a.H + i) = o;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_mark(a, 9);
}

// A wait that nothing satisfies: used by the failure-detection test to exercise the deadline path
// without faulting or hanging anything.
__global__ void ep_wait_probe_kernel(const uint32_t* flag, uint32_t target, unsigned long long deadline_ns, int* status) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  if (threadIdx.x == 0 && !wait_ge(flag, target, deadline_ns)) atomicCAS(status, 0, PLOW_ERR_PEER_WAIT | kTagEp);
}

inline int ok() { cudaError_t e = cudaGetLastError(); return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e); }

}  // namespace

extern "C" {

// `args` is a host copy of EpArgs laid out as: 8 peer pointers, 7 u64 layout offsets, 6 ints (W, me, E, e_local, Rmax, H),
// epoch pointer, status pointer, u64 deadline (see plow_b200/parallel/ep.py for the ctypes mirror).
int plow_ep_counts(const void* args, const void* table, int n_pairs, int* cursor, void* st) {
  const EpArgs& a = *static_cast<const EpArgs*>(args);
  plow::launch_serial(ep_counts_kernel, dim3(1), dim3(1024), a.E * 4, reinterpret_cast<cudaStream_t>(st), a, static_cast<const int2*>(table), n_pairs, cursor);
  return ok();
}
int plow_ep_push(const void* args, const void* table, int n_pairs, int top_k, const void* xq, const float* sx, int ld_sx,
                 int* cursor, int* grp_off, int* tile_prefix, int* pair_dest, int n_cta, int shared_rows, void* st) {
  const EpArgs& a = *static_cast<const EpArgs*>(args);
  // one warp per row when the step is small (decode): the copy is latency-bound, so width beats reuse; n_cta caps it
  const int rows = n_pairs + shared_rows;
  int grid = (rows + 7) / 8;
  if (grid > n_cta) grid = n_cta;
  if (grid < 1) grid = 1;
  plow::launch_serial(ep_push_kernel, dim3(grid), dim3(256), (a.W + 2) * a.E * 4, reinterpret_cast<cudaStream_t>(st), 
      a, static_cast<const int2*>(table), n_pairs, top_k, static_cast<const uint8_t*>(xq), sx, ld_sx, cursor, grp_off,
      tile_prefix, pair_dest, shared_rows);
  return ok();
}
int plow_ep_y_ready(const void* args, void* st) {
  const EpArgs& a = *static_cast<const EpArgs*>(args);
  plow::launch_serial(ep_y_ready_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(st), a);
  return ok();
}
int plow_ep_combine(const void* args, void* out, const void* shared, const void* table, const int* pair_dest, int T, int top_k,
                    const int* shared_base, int signal_y, void* st) {
  const EpArgs& a = *static_cast<const EpArgs*>(args);
  if (top_k > 16 || a.H % 8) return -1;
  plow::launch_serial(ep_combine_kernel, dim3(T, (a.H / 8 + 255) / 256), dim3(256), 0, reinterpret_cast<cudaStream_t>(st), a, static_cast<__nv_bfloat16*>(out),
                                                                    static_cast<const __nv_bfloat16*>(shared),
                                                                    static_cast<const int2*>(table), pair_dest, top_k, shared_base, signal_y);
  return ok();
}
int plow_wait_probe(const void* flag, unsigned int target, unsigned long long deadline_ns, int* status, void* st) {
  plow::launch_serial(ep_wait_probe_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(st), static_cast<const uint32_t*>(flag), target, deadline_ns, status);
  return ok();
}

}  // extern "C"
