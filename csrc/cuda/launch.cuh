// Launch helpers shared by every kernel file of the library.
//
// * Programmatic dependent launch.  A decode step is a chain of short kernels, each of which
//   reads what the one before it wrote.  Launched the ordinary way, kernel i+1 cannot even be
//   scheduled before the last thread of kernel i has exited, so block scheduling, barrier and
//   TMEM set-up, tensor-map fetches and the first weight loads of i+1 all sit on the critical
//   path.  Every kernel here therefore begins with `pdl_launch_dependents()` (its successor may be
//   scheduled as soon as all of its own blocks are resident) and executes `pdl_wait()` before the
//   first access to anything a predecessor produced; whatever comes before the wait (set-up,
//   loads of *weights*, which no kernel writes) overlaps the predecessor's tail.  `pdl_wait()`
//   returns once every prerequisite grid has completed and its writes are visible, so ordering is
//   exactly that of a plain stream; in a launch without the attribute both are no-ops.
//   Rule for kernel authors: no global write and no read of an activation before `pdl_wait()`,
//   and every block executes it (a grid none of whose blocks waits could complete before its
//   predecessor).  PLOW_PDL=0 in the environment turns the attribute off.
// * Per-device "done once" flags for `cudaFuncSetAttribute` (function attributes and the SM
//   count are properties of a device, not of the process: a process that drives two GPUs must
//   set them on each).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

#include <utility>

namespace plow {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("PLOW_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// Diagnostic knob: PLOW_PDL_SKIP=absorb,fold launches every kernel whose (mangled) name contains one of the
// comma-separated substrings without the attribute, to bisect an ordering problem to a kernel.
inline bool pdl_skipped(const void* kern) {
  static const char* env = getenv("PLOW_PDL_SKIP");
  if (!env || !*env) return false;
  const char* name = nullptr;
  if (cudaFuncGetName(&name, kern) != cudaSuccess || !name) return false;
  const char* p = env;
  while (*p) {
    const char* q = p;
    while (*q && *q != ',') ++q;
    const size_t n = static_cast<size_t>(q - p);
    if (n > 0)
      for (const char* s = name; *s; ++s) {
        size_t i = 0;
        while (i < n && s[i] && s[i] == p[i]) ++i;
        if (i == n) return true;
      }
    p = *q ? q + 1 : q;
  }
  return false;
}

inline bool pdl_everywhere() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("PLOW_PDL_ALL");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}

// kern<<<grid, block, smem, stream>>>(args...), with the programmatic-serialization attribute when `early` is set.
// Which kernels ask for it is a measured choice: a decode step of the 61-layer MLA-MoE model ran 36.1 ms with the
// attribute on the GEMM only (its prologue and first weight stages overlap the row kernel before it), 36.6 ms with
// it nowhere and 37.6 ms with it on every kernel (row and attention kernels gain nothing from starting early and
// their resident, waiting blocks cost the running kernel).  PLOW_PDL_ALL=1 forces it everywhere.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_impl(bool early, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_enabled() && (early || pdl_everywhere()) && !pdl_skipped(reinterpret_cast<const void*>(kern))) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// Dependent launch allowed to start early (the kernel waits with pdl_wait() before touching its inputs).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_impl(true, kern, grid, block, smem, stream, std::forward<Args>(args)...);
}
// Ordinary stream-ordered launch (the kernel still releases its own dependents early).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_serial(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_impl(false, kern, grid, block, smem, stream, std::forward<Args>(args)...);
}

constexpr int kMaxDevices = 64;

inline int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

// One flag per device; `static DeviceOnce once;` beside a cudaFuncSetAttribute call.
struct DeviceOnce {
  bool done[kMaxDevices] = {};
  bool test() const { return done[current_device()]; }
  void mark() { done[current_device()] = true; }
};

// Raise a kernel's dynamic shared-memory limit once per device.  Returns cudaSuccess or the error.
template <typename K>
inline cudaError_t ensure_smem(DeviceOnce& once, K kern, int bytes) {
  if (once.test()) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) once.mark();
  return e;
}

}  // namespace plow
