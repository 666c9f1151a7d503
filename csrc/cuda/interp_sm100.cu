// Persistent on-device interpreter for sm_100a: one CTA per compute unit walks that unit's stream of the
// packet program exactly as the packet lays it out — for every stream entry: poll the wait counters
// (acquire, bounded by a %globaltimer deadline), run the entry's slice range of the instruction, fence,
// bump the instruction's counter (release).  The tables it reads (64-byte instructions, 24-byte stream
// entries, waits, successors, 128-byte-strided counters) are the packet's own bytes copied to the device;
// nothing is re-planned at run time.
//
// One launch executes a contiguous instruction range [inst_lo, inst_hi) — a *segment* in the packet's
// terms.  Row-class segments (embedding, norms, residuals, GLU, row gather, arg-max) run here; GEMM,
// attention and collective segments are separate role kernels bound to the packet by opcode, launched in
// stream order between interpreter launches, so a wait on an instruction outside the launch's range is
// already satisfied by stream order and is skipped.  CTAs of a launch wait on one another, so the kernel is
// launched cooperatively (all CTAs co-resident) and refuses a program planned for more units than fit.
//
// The reference's counterpart is runtime/nvidia/interp_sm120.cu (claim loop / static per-CU stream, gates,
// switch(in->op), :1453-3409) with role kernels bound to segments (crates/plow-asset/src/segment_roles.rs).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "plow_packet.h"
#include "ptx.cuh"

namespace plow {

struct InterpArgs {
  const PlowInst* insts;
  const PlowStreamEnt* stream;
  const uint32_t* cu_ofs;
  const PlowWait* waits;
  const uint32_t* succs;
  void* const* tensors;      // device pointer per tensor handle, resolved for this program
  const int2* aux;           // per instruction: (rows the op runs over, row width where the op needs one)
  const uint32_t* pc0;       // per unit: first stream index whose instruction is >= inst_lo (host-built per segment)
  uint32_t* ctr;             // n_ctr * PLOW_CTR_STRIDE_U32, zeroed before the launch for [inst_lo, inst_hi)
  PlowTraceRec* trace;       // optional, one record per stream entry
  int* status;
  uint32_t inst_lo, inst_hi, n_cu, deadline_ms;
};

constexpr int kInterpThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ float cta_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < kInterpThreads / 32; ++w) s += red[w];
  __syncthreads();
  return s;
}

template <class T> __device__ __forceinline__ T* tptr(const InterpArgs& a, const PlowInst& in, int j) {
  return in.t[j] == PLOW_T_NONE ? nullptr : static_cast<T*>(a.tensors[in.t[j]]);
}

// y = x * rsqrt(mean(x^2) + eps) * gamma for one row, all threads of the CTA
__device__ void norm_row(__nv_bfloat16* out, const __nv_bfloat16* x, const __nv_bfloat16* g, int W, float eps, int mode, float* red) {
  float ss = 0.f;
  const bool vec = (W & 1) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(g)) & 3) == 0;
  if (vec) {
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(x);
    for (int j = threadIdx.x; j < W / 2; j += kInterpThreads) { const float2 v = __bfloat1622float2(x2[j]); ss += v.x * v.x + v.y * v.y; }
    const float rs = rsqrtf(cta_sum(ss, red) / W + eps);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(g);
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(out);
    for (int j = threadIdx.x; j < W / 2; j += kInterpThreads) {
      const float2 v = __bfloat1622float2(x2[j]);
      float2 gm = g ? __bfloat1622float2(g2[j]) : make_float2(1.f, 1.f);
      if (g && mode) { gm.x += 1.f; gm.y += 1.f; }
      o2[j] = __floats2bfloat162_rn(v.x * rs * gm.x, v.y * rs * gm.y);
    }
    return;
  }
  for (int j = threadIdx.x; j < W; j += kInterpThreads) { const float v = __bfloat162float(x[j]); ss += v * v; }
  const float rs = rsqrtf(cta_sum(ss, red) / W + eps);
  for (int j = threadIdx.x; j < W; j += kInterpThreads) {
    const float gm = g ? (mode ? 1.0f + __bfloat162float(g[j]) : __bfloat162float(g[j])) : 1.0f;
    out[j] = __float2bfloat16(__bfloat162float(x[j]) * rs * gm);
  }
}

__device__ void run_slices(const InterpArgs& a, const PlowInst& in, uint32_t inst, int s0, int s1, float* red,
                           unsigned long long* red64) {
  const int ns = in.nslice;
  const long long R = a.aux[inst].x;
  const long long r0 = R * s0 / ns, r1 = R * s1 / ns;
  switch (in.op) {
    case PLOW_OP_NOP: break;
    case PLOW_OP_EMBED: {
      __nv_bfloat16* out = tptr<__nv_bfloat16>(a, in, 0);
      const __nv_bfloat16* tab = tptr<const __nv_bfloat16>(a, in, 1);
      const int* ids = tptr<const int>(a, in, 2);
      const int H = in.i[0];
      const float scale = in.w[0].f;
      for (long long r = r0; r < r1; ++r) {
        const __nv_bfloat16* src = tab + static_cast<size_t>(ids[r]) * H;
        for (int j = threadIdx.x; j < H; j += kInterpThreads)
          out[r * H + j] = scale == 1.0f ? src[j] : __float2bfloat16(__bfloat162float(src[j]) * scale);
      }
      break;
    }
    case PLOW_OP_RMSNORM: {
      __nv_bfloat16* out = tptr<__nv_bfloat16>(a, in, 0);
      const __nv_bfloat16* x = tptr<const __nv_bfloat16>(a, in, 1);
      const __nv_bfloat16* g = tptr<const __nv_bfloat16>(a, in, 2);
      const int W = in.i[0], mode = in.i[1], co = in.i[6], pitch = in.i[7] ? in.i[7] : W;
      for (long long r = r0; r < r1; ++r) norm_row(out + r * W, x + r * pitch + co, g, W, in.w[0].f, mode, red);
      break;
    }
    case PLOW_OP_ADD_NORM: {
      __nv_bfloat16* h = tptr<__nv_bfloat16>(a, in, 0);
      const __nv_bfloat16* x = tptr<const __nv_bfloat16>(a, in, 1);
      const __nv_bfloat16* d = tptr<const __nv_bfloat16>(a, in, 2);
      const __nv_bfloat16* g = tptr<const __nv_bfloat16>(a, in, 3);
      __nv_bfloat16* xo = tptr<__nv_bfloat16>(a, in, 4);
      const int W = in.i[0], mode = in.i[1];
      for (long long r = r0; r < r1; ++r) {
        // the sum is rounded to bf16 before the norm reads it, as the unfused pair would do
        for (int j = threadIdx.x; j < W; j += kInterpThreads)
          xo[r * W + j] = __float2bfloat16(__bfloat162float(x[r * W + j]) + __bfloat162float(d[r * W + j]));
        __syncthreads();
        norm_row(h + r * W, xo + r * W, g, W, in.w[0].f, mode, red);
      }
      break;
    }
    case PLOW_OP_RESIDUAL: {
      __nv_bfloat16* out = tptr<__nv_bfloat16>(a, in, 0);
      const __nv_bfloat16* x = tptr<const __nv_bfloat16>(a, in, 1);
      const __nv_bfloat16* y = tptr<const __nv_bfloat16>(a, in, 2);
      const long long W = in.i[0];
      for (long long k = r0 * W + threadIdx.x; k < r1 * W; k += kInterpThreads)
        out[k] = __float2bfloat16(__bfloat162float(x[k]) + __bfloat162float(y[k]));
      break;
    }
    case PLOW_OP_GLU: {
      __nv_bfloat16* out = tptr<__nv_bfloat16>(a, in, 0);
      const __nv_bfloat16* g = tptr<const __nv_bfloat16>(a, in, 1);
      const __nv_bfloat16* u = tptr<const __nv_bfloat16>(a, in, 2);
      const long long W = a.aux[inst].y;
      for (long long k = r0 * W + threadIdx.x; k < r1 * W; k += kInterpThreads) {
        const float gv = __bfloat162float(g[k]);
        out[k] = __float2bfloat16(gv / (1.0f + __expf(-gv)) * __bfloat162float(u[k]));
      }
      break;
    }
    case PLOW_OP_ROW_GATHER: {
      __nv_bfloat16* out = tptr<__nv_bfloat16>(a, in, 0);
      const __nv_bfloat16* x = tptr<const __nv_bfloat16>(a, in, 1);
      const int* rows = tptr<const int>(a, in, 2);
      const int W = in.i[0];
      for (long long s = r0; s < r1; ++s)
        for (int j = threadIdx.x; j < W; j += kInterpThreads) out[s * W + j] = x[static_cast<size_t>(rows[s]) * W + j];
      break;
    }
    case PLOW_OP_ARGMAX: {
      int* out = tptr<int>(a, in, 0);
      const float* lg = tptr<const float>(a, in, 1);
      const int V = in.i[0];
      for (long long s = r0; s < r1; ++s) {
        // packed (ordered value, ~index): the lowest index wins ties
        unsigned long long best = 0;
        for (int j = threadIdx.x; j < V; j += kInterpThreads) {
          const uint32_t b = __float_as_uint(lg[s * V + j]);
          const uint32_t o = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
          const unsigned long long k = (static_cast<unsigned long long>(o) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(j));
          best = k > best ? k : best;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o); best = t > best ? t : best; }
        if ((threadIdx.x & 31) == 0) red64[threadIdx.x >> 5] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
          for (int w = 1; w < kInterpThreads / 32; ++w) best = red64[w] > best ? red64[w] : best;
          out[s] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFu));
        }
        __syncthreads();
      }
      break;
    }
    default:
      if (threadIdx.x == 0) atomicCAS(a.status, 0, PLOW_ERR_BOUNDS | kTagInterp);   // an opcode without a body in this interpreter
      break;
  }
}

__global__ void __launch_bounds__(kInterpThreads)
interp_kernel(const InterpArgs a) {
  __shared__ float red[kInterpThreads / 32];
  __shared__ unsigned long long red64[kInterpThreads / 32];
  __shared__ int give_up;
  const uint32_t cu = blockIdx.x;
  if (cu >= a.n_cu) return;
  if (threadIdx.x == 0) give_up = 0;
  __syncthreads();
  const unsigned long long deadline = static_cast<unsigned long long>(a.deadline_ms ? a.deadline_ms : 2000) * 1000000ull;
  // a unit's stream is ordered by instruction: start at the segment's first entry, stop at its last
  const uint32_t pc_end = a.cu_ofs[cu + 1];
  for (uint32_t pc = a.pc0[cu]; pc < pc_end; ++pc) {
    const PlowStreamEnt se = a.stream[pc];
    if (se.inst >= a.inst_hi) break;
    if (se.inst < a.inst_lo) continue;
    unsigned long long t_arrive = 0, t_ready = 0;
    if (threadIdx.x == 0) {
      if (a.trace) t_arrive = globaltimer_ns();
      for (uint32_t w = 0; w < se.n_wait && !give_up; ++w) {
        const PlowWait pw = a.waits[se.wait_ofs + w];
        if (pw.ctr < a.inst_lo || pw.ctr >= a.inst_hi) continue;       // produced by an earlier launch of the stream
        const uint32_t* c = a.ctr + static_cast<size_t>(pw.ctr) * PLOW_CTR_STRIDE_U32;
        const unsigned long long t0 = globaltimer_ns();
        while (ld_acquire_gpu(c) < pw.target) {
          if (globaltimer_ns() - t0 > deadline || *reinterpret_cast<volatile int*>(a.status) != 0) {
            atomicCAS(a.status, 0, PLOW_ERR_GRID_WAIT | kTagInterp);
            give_up = 1;
            break;
          }
          __nanosleep(64);
        }
      }
      if (a.trace) t_ready = globaltimer_ns();
    }
    __syncthreads();
    if (give_up) break;
    const PlowInst in = a.insts[se.inst];
    run_slices(a, in, se.inst, se.slice0, se.slice0 + se.nslice, red, red64);
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      for (uint32_t s = 0; s < se.n_succ; ++s)
        red_add_release_gpu(a.ctr + static_cast<size_t>(a.succs[se.succ_ofs + s]) * PLOW_CTR_STRIDE_U32, 1u);
      if (a.trace) {
        PlowTraceRec tr;
        tr.cu = cu; tr.pc = pc; tr.inst = se.inst; tr.op = in.op;
        tr.t_arrive = t_arrive; tr.t_ready = t_ready; tr.t_end = globaltimer_ns();
        a.trace[pc] = tr;
      }
    }
  }
}

}  // namespace plow

extern "C" {

// Every pointer is device memory.  `ctr` entries of [inst_lo, inst_hi) are zeroed here (memset node) before
// the cooperative launch.  Returns -2 when the program's unit count does not fit on the device at once.
int plow_interp_run(const void* insts, const void* stream, const void* cu_ofs, const void* waits, const void* succs,
                    const void* tensors, const void* aux, const void* pc0, void* ctr, void* trace, int* status, uint32_t inst_lo,
                    uint32_t inst_hi, uint32_t n_cu, uint32_t deadline_ms, void* stream_) {
  using namespace plow;
  if (!insts || !stream || !cu_ofs || !tensors || !aux || !pc0 || !ctr || !status || inst_hi <= inst_lo || n_cu == 0) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  static int capacity = 0;
  if (!capacity) {
    int dev = 0, sms = 0, per = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, interp_kernel, kInterpThreads, 0) != cudaSuccess) return 3000;
    capacity = sms * per;
  }
  if (static_cast<int>(n_cu) > capacity) return -2;
  cudaMemsetAsync(static_cast<uint32_t*>(ctr) + static_cast<size_t>(inst_lo) * PLOW_CTR_STRIDE_U32, 0,
                  static_cast<size_t>(inst_hi - inst_lo) * PLOW_CTR_STRIDE_U32 * sizeof(uint32_t), st);
  InterpArgs a;
  a.insts = static_cast<const PlowInst*>(insts); a.stream = static_cast<const PlowStreamEnt*>(stream);
  a.cu_ofs = static_cast<const uint32_t*>(cu_ofs); a.waits = static_cast<const PlowWait*>(waits);
  a.succs = static_cast<const uint32_t*>(succs); a.tensors = static_cast<void* const*>(tensors);
  a.aux = static_cast<const int2*>(aux); a.pc0 = static_cast<const uint32_t*>(pc0); a.ctr = static_cast<uint32_t*>(ctr); a.trace = static_cast<PlowTraceRec*>(trace);
  a.status = status; a.inst_lo = inst_lo; a.inst_hi = inst_hi; a.n_cu = n_cu; a.deadline_ms = deadline_ms;
  void* params[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(interp_kernel), dim3(n_cu), dim3(kInterpThreads), params, 0, st);
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
