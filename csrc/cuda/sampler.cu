// Device sampler: temperature -> top-k -> softmax -> top-p -> min-p -> renormalise -> inverse-CDF draw,
// one CTA per sampled row, entirely in f32 over the row's logits (no sort: the top-k and top-p cut
// points are found by an 8-bit radix descent over the monotone integer image of the values, counting
// elements for top-k and probability mass for top-p).  Ties at a cut value are all kept.  Rows whose
// temperature is <= 0 take the arg-max (lowest index on ties).  The filter order is the host sampler's
// (plow_b200/text/sample.py); reference: runtime/nvidia/sample_sm120.cu, crates/plowrt/src/text/sample.rs.
// The uniform variate comes from the caller (u[row]) or, when u is NULL, from a counter hash of
// (seed[row], step) so a request with a seed replays identically.
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t ordered_key(float x) {   // monotone: larger float -> larger key
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < (kThreads / 32) ? red[lane] : (is_max ? -INFINITY : 0.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float t = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, t) : v + t;
    }
    if (lane == 0) red[32] = v;
  }
  __syncthreads();
  return red[32];
}

// Radix descent over 32-bit keys: returns the largest key T such that weight({key >= T}) >= target,
// where weight is the element count (MASS = false) or the summed value val(i) (MASS = true).
template <bool MASS, class KeyFn, class ValFn>
__device__ uint32_t radix_threshold(int V, float target, KeyFn key, ValFn val, float* hist, uint32_t* sh_u, float* sh_f) {
  uint32_t prefix = 0, mask = 0;
  float above = 0.f;   // weight of keys strictly above the current prefix bucket
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const uint32_t k = key(i);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], MASS ? val(i) : 1.0f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = above;
      int d = 255;
      for (; d > 0; --d) {
        if (acc + hist[d] >= target) break;
        acc += hist[d];
      }
      *sh_u = static_cast<uint32_t>(d);
      *sh_f = acc;
    }
    __syncthreads();
    prefix |= (*sh_u) << shift;
    mask |= 255u << shift;
    above = *sh_f;
    __syncthreads();
  }
  return prefix;
}

__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned long long ctr) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);   // [0, 1)
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(int* out, const float* logits, int ld, int V, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* u_in, const unsigned long long* seed,
              unsigned long long step) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ float red[33];
  __shared__ float hist[256];
  __shared__ uint32_t sh_u;
  __shared__ float sh_f;
  __shared__ float scan[kThreads / 32];
  __shared__ int sh_pick;
  const int row = blockIdx.x;
  const float* lg = logits + static_cast<size_t>(row) * ld;
  const float T = temperature ? temperature[row] : 1.0f;
  if (T <= 0.f) {
    // arg-max, lowest index on ties: packed (ordered value, ~index)
    unsigned long long best = 0;
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const unsigned long long k = (static_cast<unsigned long long>(ordered_key(lg[i])) << 32) | (0xFFFFFFFFu - i);
      best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
      best = t > best ? t : best;
    }
    __shared__ unsigned long long bw[kThreads / 32];
    if ((threadIdx.x & 31) == 0) bw[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kThreads / 32; ++w) best = bw[w] > best ? bw[w] : best;
      out[row] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFu));
    }
    return;
  }
  const float invT = 1.0f / fmaxf(T, 1e-6f);
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += kThreads) mx = fmaxf(mx, lg[i] * invT);
  mx = block_reduce(mx, red, true);
  // top-k: key of the k-th largest scaled logit
  uint32_t k_key = 0;
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < V)
    k_key = radix_threshold<false>(V, static_cast<float>(k), [&](int i) { return ordered_key(lg[i] * invT); },
                                   [&](int) { return 1.0f; }, hist, &sh_u, &sh_f);
  auto e_of = [&](int i) -> float {
    const float x = lg[i] * invT;
    return ordered_key(x) >= k_key ? __expf(x - mx) : 0.f;
  };
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += kThreads) z += e_of(i);
  z = block_reduce(z, red, false);
  const float invZ = 1.0f / z;
  // top-p: smallest set of the largest probabilities whose mass reaches top_p
  float p_cut = 0.f;
  const float tp = top_p ? top_p[row] : 1.0f;
  if (tp < 1.0f) {
    const uint32_t pk = radix_threshold<true>(V, tp, [&](int i) { return ordered_key(e_of(i) * invZ); },
                                              [&](int i) { return e_of(i) * invZ; }, hist, &sh_u, &sh_f);
    p_cut = __uint_as_float(pk & 0x7FFFFFFFu);   // probabilities are >= 0: the key is the float with the sign bit set
  }
  const float mp = min_p ? min_p[row] : 0.f;
  p_cut = fmaxf(p_cut, mp * invZ);               // the largest probability is exp(0) / Z
  auto p_of = [&](int i) -> float {
    const float p = e_of(i) * invZ;
    return (p >= p_cut && p > 0.f) ? p : 0.f;
  };
  // inverse CDF in index order: contiguous chunk per thread, block scan of the chunk sums
  const int chunk = (V + kThreads - 1) / kThreads;
  const int i0 = threadIdx.x * chunk, i1 = min(V, i0 + chunk);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) local += p_of(i);
  float incl = local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) scan[warp] = incl;
  if (threadIdx.x == 0) sh_pick = -1;
  __syncthreads();
  float base = 0.f, total = 0.f;
  for (int w = 0; w < kThreads / 32; ++w) {
    if (w < warp) base += scan[w];
    total += scan[w];
  }
  const float u = u_in ? u_in[row] : hash_uniform(seed ? seed[row] : 0ull, step);
  const float target = u * total;
  const float lo = base + incl - local, hi = base + incl;
  if (local > 0.f && target >= lo && target < hi) {
    float acc = lo;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float p = p_of(i);
      if (p > 0.f) { pick = i; acc += p; if (target < acc) break; }
    }
    atomicMax(&sh_pick, pick);
  }
  __syncthreads();
  if (sh_pick < 0) {
    // rounding left the target at or past the total: take the last kept index
    int last = -1;
    for (int i = i0; i < i1; ++i) if (p_of(i) > 0.f) last = i;
    atomicMax(&sh_pick, last);
    __syncthreads();
  }
  if (threadIdx.x == 0) out[row] = sh_pick;
}

}  // namespace

extern "C" {

// logits f32 [rows][ld]; temperature / top_p / min_p f32 [rows] and top_k int32 [rows] (each may be NULL =
// neutral); u f32 [rows] uniform variates in [0,1) or NULL to hash (seed[row], step); out int32 [rows].
int plow_sample(int* out, const float* logits, int ld, int rows, int V, const float* temperature, const int* top_k,
                const float* top_p, const float* min_p, const float* u, const void* seed, uint64_t step, void* stream) {
  if (rows <= 0 || V <= 0) return -1;
  plow::launch_serial(sample_kernel, dim3(rows), dim3(kThreads), 0, reinterpret_cast<cudaStream_t>(stream), 
      out, logits, ld, V, temperature, top_k, top_p, min_p, u, static_cast<const unsigned long long*>(seed), step);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
