// Row kernels of the materialised multi-head latent attention prefill.
//
// Decode reads the e4m3 latent cache directly with the absorbed query (576-wide dot products, 512-wide values).  For
// a long run of new rows of one request that costs 3.4x the arithmetic of plain multi-head attention over K / V rebuilt
// from the latent, so prefill rebuilds them once per layer:
//
//   gather : the request's cached latent rows, page by page, into one contiguous range.  The e4m3 bytes are copied as
//            they are together with their per-token scale laid out as the 1x128 activation scales of the block-scaled
//            GEMM (one scale per token covers all four 128-wide K blocks, so no re-quantisation happens), or
//            dequantised to bf16 when the up-projection weight is bf16.  The rotary key part is dequantised to bf16.
//   GEMM   : kvb[token][head][nope | v] = latent . W_kv_b^T (the library's GEMM)
//   rope   : the rotary part of the new query rows, in place
//   attend : the tcgen05 flash kernel of attn_gqa.cu with 192-wide keys and 128-wide values
//
// Reference counterpart: crates/devgen/src/mla.rs (prefill expands the latent through kv_b_proj before attention).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"

namespace {

constexpr int kPage = 64;

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __nv_fp8_e4m3 v;
  v.__x = b;
  return static_cast<float>(v);
}

// spans[s] = {slot, tokens, base, 0}: tokens [0, tokens) of `slot` land at rows [base, base + tokens) of the outputs
// (base is a multiple of 64).  One block per (64-token tile, span).  Rows of the last tile beyond `tokens` are zeroed so
// that nothing non-finite reaches the value product.  vpt[slot][tile] = base / 64 + tile is the tile index the
// attention kernel looks up.
__global__ void __launch_bounds__(256)
mla_latent_gather_kernel(uint8_t* lat8, float* lat_scale, int ld_scale, __nv_bfloat16* lat16, __nv_bfloat16* krope,
                         int* vpt, const uint8_t* kv8, const float* kv_scale, const int* page_table, int max_pages,
                         const int4* spans, int latent, int rope) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int4 sp = spans[blockIdx.y];
  const int tile = blockIdx.x;
  if (tile * kPage >= sp.y) return;
  const int W = latent + rope;
  const int page = page_table[static_cast<size_t>(sp.x) * max_pages + tile];
  const size_t src0 = static_cast<size_t>(page) * kPage;
  const size_t dst0 = static_cast<size_t>(sp.z) + static_cast<size_t>(tile) * kPage;
  if (threadIdx.x == 0) vpt[static_cast<size_t>(sp.x) * max_pages + tile] = sp.z / kPage + tile;
  const int live = min(kPage, sp.y - tile * kPage);
  const int chunks = W / 16;                       // 16-byte chunks per token row
  for (int c = threadIdx.x; c < kPage * chunks; c += blockDim.x) {
    const int tok = c / chunks, part = c % chunks;
    const bool ok = tok < live;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (ok) raw = *reinterpret_cast<const uint4*>(kv8 + (src0 + tok) * W + part * 16);
    const float sc = ok ? kv_scale[src0 + tok] : 0.f;
    const bool is_rope = part * 16 >= latent;
    if (!is_rope && lat8) {
      *reinterpret_cast<uint4*>(lat8 + (dst0 + tok) * W + part * 16) = raw;
      continue;
    }
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    __align__(16) __nv_bfloat16 o[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = __float2bfloat16(e4m3_to_float(b[i]) * sc);
    __nv_bfloat16* dst = is_rope ? krope + (dst0 + tok) * rope + (part * 16 - latent)
                                 : lat16 + (dst0 + tok) * latent + part * 16;
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(o)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(o)[1];
  }
  if (lat_scale)
    for (int t = threadIdx.x; t < kPage; t += blockDim.x) {
      const float sc = t < live ? kv_scale[src0 + t] : 0.f;
      for (int kb = 0; kb < latent / 128; ++kb) lat_scale[static_cast<size_t>(kb) * ld_scale + dst0 + t] = sc;
    }
}

// One warp per (row, head): rotate the trailing `rope` dims of the head's query in place (same pairing as the key
// side of the cache write: pair_mode 1 = interleaved pairs, 0 = halves).  Rows with pos < 0 are left alone.
__global__ void mla_q_rope_kernel(__nv_bfloat16* q, int pitch, const float* rope_tab, const int* pos, int T, int heads,
                                  int nope, int rope, int pair_mode) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(T) * heads) return;
  const int r = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  const int p = pos[r];
  if (p < 0) return;
  __nv_bfloat16* v = q + static_cast<size_t>(r) * pitch + static_cast<size_t>(h) * (nope + rope) + nope;
  const int half = rope / 2;
  const float* tab = rope_tab + static_cast<size_t>(p) * rope;
  for (int i = lane; i < half; i += 32) {
    const int ia = pair_mode ? 2 * i : i, ib = pair_mode ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(v[ia]), b = __bfloat162float(v[ib]);
    const float c = tab[i], s = tab[half + i];
    v[ia] = __float2bfloat16(a * c - b * s);
    v[ib] = __float2bfloat16(b * c + a * s);
  }
}

}  // namespace

extern "C" {

// lat8 e4m3 [n][latent+rope] with lat_scale f32 [latent/128][ld_scale] (fp8 up-projection), or lat16 bf16 [n][latent]
// (bf16 up-projection): exactly one of lat8 / lat16 is given.  krope bf16 [n][rope].  spans int32 [n_spans][4].
int plow_mla_latent_gather(void* lat8, float* lat_scale, int ld_scale, void* lat16, void* krope, int* vpt, const void* kv8,
                           const float* kv_scale, const int* page_table, int max_pages, const void* spans, int n_spans,
                           int max_tiles, int latent, int rope, void* stream) {
  if (n_spans <= 0 || max_tiles <= 0) return 0;
  if (latent % 128 || rope % 16 || (lat8 == nullptr) == (lat16 == nullptr)) return -1;
  if (lat8 && !lat_scale) return -1;
  plow::launch_serial(mla_latent_gather_kernel, dim3(max_tiles, n_spans), dim3(256), 0, static_cast<cudaStream_t>(stream),
                      static_cast<uint8_t*>(lat8), lat_scale, ld_scale, static_cast<__nv_bfloat16*>(lat16),
                      static_cast<__nv_bfloat16*>(krope), vpt, static_cast<const uint8_t*>(kv8), kv_scale, page_table, max_pages,
                      static_cast<const int4*>(spans), latent, rope);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

int plow_mla_q_rope(void* q, int pitch, const float* rope_tab, const int* pos, int T, int heads, int nope, int rope,
                    int pair_mode, void* stream) {
  if (T <= 0) return 0;
  const int wpb = 8;
  const long long items = static_cast<long long>(T) * heads;
  plow::launch_serial(mla_q_rope_kernel, dim3(static_cast<unsigned>((items + wpb - 1) / wpb)), dim3(wpb * 32), 0,
                      static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16*>(q), pitch, rope_tab, pos, T, heads, nope,
                      rope, pair_mode);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
