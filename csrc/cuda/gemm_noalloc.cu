// Allocation-free variant of the split-K GEMM: same kernel template as the regular entry point,
// scratch in a file-scope device array instead of caller-provided buffers (see gemm_noalloc.h).
#include "gemm_noalloc.h"
#include "gemm_tc.cuh"

namespace {

constexpr size_t kWsBytes = 8u << 20;
constexpr size_t kCtrBytes = 64u << 10;
static_assert(kWsBytes + kCtrBytes == PLOW_NOALLOC_SCRATCH_BYTES, "header and array disagree");

// Partials first, then the arrival / departure counters (one per 128-byte line, 2 x 256 lines).
static __device__ __align__(256) unsigned char g_scratch[kWsBytes + kCtrBytes];

// Device address of g_scratch per device.  In host code `g_scratch` names a host-side stand-in, not
// device memory, so the address handed to the kernel must come from cudaGetSymbolAddress.
unsigned char* g_scratch_dev[64] = {nullptr};

int scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PLOW_NOALLOC_E_SYMBOL;
  if (!g_scratch_dev[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || !p) return PLOW_NOALLOC_E_SYMBOL;
    g_scratch_dev[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_dev[dev];
  return 0;
}

}  // namespace

extern "C" const char* plow_gemm_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case PLOW_NOALLOC_E_ARG: return "bad argument: null or misaligned pointer, M outside [1,128], or K not a multiple of 8";
    case PLOW_NOALLOC_E_TOO_LARGE: return "problem too large for the static scratch (8 MiB of partials, 128 tiles)";
    case PLOW_NOALLOC_E_SYMBOL: return "could not resolve the device address of the static scratch";
    default: return "launcher error";
  }
}

extern "C" int plow_gemm_splitk_noalloc(const void* x, const void* w, void* y, int32_t M, int32_t N, int32_t K,
                                        int32_t splits, int32_t* status, void* stream_) {
  using namespace plow;
  if (!x || !w || !y || !status || M < 1 || M > 128 || N < 1 || K < 8 || (K & 7)) return PLOW_NOALLOC_E_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15) return PLOW_NOALLOC_E_ARG;
  const int bn = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  const int tiles = (N + 127) / 128;
  const int kb = (K + 63) / 64;
  if (splits < 1) splits = 1;
  if (splits > kb) splits = kb;
  if (splits > bn) splits = bn;
  if (tiles > 128) return PLOW_NOALLOC_E_TOO_LARGE;   // checked first: tiles * splits below must not overflow
  const int sms = sm_count();
  if (tiles * splits > sms) splits = sms / tiles;      // every CTA of a tile must be resident at once
  if (splits < 1) return PLOW_NOALLOC_E_TOO_LARGE;
  if (static_cast<size_t>(tiles) * splits * 128 * bn * sizeof(float) > kWsBytes) return PLOW_NOALLOC_E_TOO_LARGE;
  unsigned char* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  // the array keeps whatever the previous call (possibly an aborted one) left: re-arm the counters
  if (cudaMemsetAsync(scratch + kWsBytes, 0, kCtrBytes, stream) != cudaSuccess) return 4999;
  GemmArgs a{};   // trace, arrival gate and fused all-reduce stay off
  a.x = x; a.w = w; a.y = y; a.status = status;
  a.M = M; a.N = N; a.K = K; a.ldy = N; a.E = 0; a.out_f32 = 0; a.out_scale = 1.0f;
  a.ws = reinterpret_cast<float*>(scratch);
  a.ws_ctr = reinterpret_cast<int*>(scratch + kWsBytes);
  a.splits = splits;
  a.stream = 0;
  if (bn == 32) return launch_gemm_tc<32, false, false, true>(a, K, K, N, stream);
  if (bn == 64) return launch_gemm_tc<64, false, false, true>(a, K, K, N, stream);
  return launch_gemm_tc<128, false, false, true>(a, K, K, N, stream);
}
