// Tensor-parallel all-reduce of activation rows with the residual add and RMSNorm that follow it, as one kernel over
// NVLink peer memory (no library collective, no second launch).
//
// Every rank holds a partial [M][H] (bf16) of a row-parallel projection.  CTA r of every rank owns row r:
//   1. it copies its partial row into this rank's slot of a symmetric buffer (two slots, alternating by call, so a
//      rank that is one call ahead never overwrites rows a slower peer still reads) and releases one flag per peer:
//      "row r of rank me, call e, is there";
//   2. it waits (bounded) for the same flag from every rank: a per-row dependency, not a grid-wide barrier, so a row
//      finishes as soon as its W partials exist;
//   3. it sums the W partial rows straight out of the peers' memory in rank order (f32, one rounding to bf16: every
//      rank forms the same bits), and, when a norm weight is given, continues exactly like the add + RMSNorm row
//      kernel: x_out = bf16(x_in + sum), h_out = bf16(rmsnorm(x_out) * gamma).
// Flags are monotonic call counters kept on the device (the last CTA of a launch publishes the new value), so the
// sequence replays from a CUDA graph.  On a wait that runs out the kernel records PLOW_ERR_PEER_WAIT and returns.
//
// Reference counterpart: the inline one-shot all-reduce of runtime/nvidia/op_collective.cuh:216-240 and its fused
// residual + norm consumer (crates/devgen/src/lib.rs:4015, XREDUCE_ADD_NORM).  Plain peer loads / stores only.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace {
using namespace plow;

struct ArArgs {
  uint8_t* peer[8];
  uint64_t part_ofs;     // two slots of [max_rows][H] bf16, `slot_bytes` apart
  uint64_t slot_bytes;
  uint64_t flag_ofs;     // u32 [W][max_rows]
  uint32_t* epoch;       // device words: [0] call counter, [1] CTAs through (ticket)
  int* status;
  unsigned long long deadline_ns;
  int W, me, max_rows, M, H;
};

__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t target, unsigned long long deadline_ns) {
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(p) < target) {
    if (globaltimer_ns() - t0 > deadline_ns) return false;
    __nanosleep(128);
  }
  return true;
}

__device__ __forceinline__ float block_sum512(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = l < nw ? sh[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__global__ void __launch_bounds__(512)
tp_ar_norm_kernel(const ArArgs a, const __nv_bfloat16* partial, int ld_partial, const __nv_bfloat16* x_in,
                  const __nv_bfloat16* gamma, __nv_bfloat16* x_out, __nv_bfloat16* h_out, float eps, int plus_one) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ float rowbuf[];      // H floats
  __shared__ float red[32];
  __shared__ int fail;
  const uint32_t ep = a.epoch[0] + 1;
  const uint64_t slot = a.part_ofs + (ep & 1) * a.slot_bytes;
  if (threadIdx.x == 0) fail = 0;
  // 1. this rank's partial rows into its own symmetric slot.  A CTA publishes ALL of its rows before it waits for any:
  //    the grid is no larger than what is resident at once, so every rank's rows get published whatever the peers do.
  for (int r = blockIdx.x; r < a.M; r += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(partial + static_cast<size_t>(r) * ld_partial);
    uint4* dst = reinterpret_cast<uint4*>(a.peer[a.me] + slot + static_cast<size_t>(r) * a.H * 2);
    for (int i = threadIdx.x; i < a.H / 8; i += blockDim.x) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  for (int r = blockIdx.x; r < a.M; r += gridDim.x)
    if (threadIdx.x < a.W)
      st_release_sys(reinterpret_cast<uint32_t*>(a.peer[threadIdx.x] + a.flag_ofs) + static_cast<size_t>(a.me) * a.max_rows + r, ep);
  for (int r = blockIdx.x; r < a.M && !fail; r += gridDim.x) {
  // 2. the same row of every rank
  if (threadIdx.x < a.W) {
    if (!wait_flag(reinterpret_cast<const uint32_t*>(a.peer[a.me] + a.flag_ofs) + static_cast<size_t>(threadIdx.x) * a.max_rows + r, ep,
                   a.deadline_ns))
      fail = 1;
  }
  __syncthreads();
  if (fail) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagTpAr);
    break;
  }
  {
    // 3. rank-ordered f32 sum out of peer memory; all W loads of a 16-byte unit are in flight together
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < a.H; i += blockDim.x * 8) {
      uint4 v[8];
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < a.W) v[p] = *reinterpret_cast<const uint4*>(a.peer[p] + slot + (static_cast<size_t>(r) * a.H + i) * 2);
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        if (p < a.W) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[p]);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 t = __bfloat1622float2(h[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);     // the all-reduce result
      if (x_in) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x_in + static_cast<size_t>(r) * a.H + i);
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 s = __bfloat1622float2(oh[j]), x = __bfloat1622float2(xh[j]);
          oh[j] = __floats2bfloat162_rn(x.x + s.x, x.y + s.y);      // rounded before the norm reads it, like the unfused pair
        }
      }
      *reinterpret_cast<uint4*>(x_out + static_cast<size_t>(r) * a.H + i) = o;
      if (gamma) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 b = __bfloat1622float2(oh[j]);
          rowbuf[i + 2 * j] = b.x; rowbuf[i + 2 * j + 1] = b.y;
          ss += b.x * b.x + b.y * b.y;
        }
      }
    }
    if (gamma) {
      const float tot = block_sum512(ss, red);
      const float rs = rsqrtf(tot / a.H + eps);
      for (int i = threadIdx.x * 8; i < a.H; i += blockDim.x * 8) {
        const uint4 gv = *reinterpret_cast<const uint4*>(gamma + i);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 g = __bfloat1622float2(gh[j]);
          if (plus_one) { g.x += 1.f; g.y += 1.f; }
          oh[j] = __floats2bfloat162_rn(rowbuf[i + 2 * j] * rs * g.x, rowbuf[i + 2 * j + 1] * rs * g.y);
        }
        *reinterpret_cast<uint4*>(h_out + static_cast<size_t>(r) * a.H + i) = o;
      }
    }
  }
  __syncthreads();       // rowbuf and red are reused by the next row
  }
  // the call counter moves on once every CTA of this launch is through
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&a.epoch[1], 1u) == gridDim.x - 1) { a.epoch[1] = 0; __threadfence(); a.epoch[0] = ep; }
  }
}

}  // namespace

extern "C" {

// partial bf16 [M][ld_partial]; x_in (residual) and gamma may be null: then x_out receives the plain all-reduce result
// and h_out is not written.  peers: 8 pointers (host array) to the ranks' symmetric regions.
int plow_tp_allreduce_norm(const void* const* peers, uint64_t part_ofs, uint64_t slot_bytes, uint64_t flag_ofs, void* epoch,
                           int world, int me, int max_rows, const void* partial, int ld_partial, const void* x_in, const void* gamma,
                           void* x_out, void* h_out, int M, int H, float eps, int plus_one, int deadline_ms, int* status,
                           void* stream) {
  if (world < 1 || world > 8 || M <= 0 || M > max_rows || H % 8 || ld_partial % 8 || !x_out || (gamma && !h_out)) return -1;
  if (static_cast<uint64_t>(M) * H * 2 > slot_bytes) return -2;
  ArArgs a;
  for (int i = 0; i < 8; ++i) a.peer[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peers[i])) : nullptr;
  a.part_ofs = part_ofs; a.slot_bytes = slot_bytes; a.flag_ofs = flag_ofs; a.epoch = static_cast<uint32_t*>(epoch);
  a.status = status; a.deadline_ns = static_cast<unsigned long long>(deadline_ms) * 1000000ull;
  a.W = world; a.me = me; a.max_rows = max_rows; a.M = M; a.H = H;
  const size_t smem = static_cast<size_t>(H) * 4;
  static plow::DeviceOnce attr;
  if (smem > 48 * 1024 && plow::ensure_smem(attr, tp_ar_norm_kernel, 200 * 1024) != cudaSuccess) return -3;
  if (smem > 200 * 1024) return -3;
  // every CTA must be resident at once (a CTA waits for peers only after it has published all of its own rows)
  int grid = 2 * plow::sm_count();
  if (smem > 100 * 1024) grid = plow::sm_count();
  if (grid > M) grid = M;
  plow::launch_serial(tp_ar_norm_kernel, dim3(grid), dim3(512), smem, reinterpret_cast<cudaStream_t>(stream), a,
                      static_cast<const __nv_bfloat16*>(partial), ld_partial, static_cast<const __nv_bfloat16*>(x_in),
                      static_cast<const __nv_bfloat16*>(gamma), static_cast<__nv_bfloat16*>(x_out), static_cast<__nv_bfloat16*>(h_out),
                      eps, plus_one);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
