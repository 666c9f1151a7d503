// Row-wise sm_100a kernels: everything between the GEMMs and the attention kernels that is
// bound by HBM bandwidth, written so each activation row is read once and every consumer format
// (bf16 for the residual stream, e4m3 + 1x128 scales for the next block-scaled GEMM) is produced in
// the same pass.
//
//   embed, rmsnorm(+quant), add_norm(+quant), quant_act, MLA query prep / query quant /
//   latent-cache write, router top-k (sigmoid or softmax, group-limited), MoE align / gather /
//   combine, argmax.
//
// Reference counterparts: runtime/nvidia/op_norm.cuh (d_rmsnorm, d_add_norm, d_headnorm_rope),
// op_elementwise.cuh (embed, argmax packed-u64), quant_group.cuh (1x128 groups, s = max(amax,1e-10)/448),
// op_moe.cuh (moe_router_topk_pf / align_pf / combine_pf), crates/packet/src/moe.rs:97-160 (router oracle).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ep_args.h"
#include "launch.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = l < nw ? sh[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// ---- embed ------------------------------------------------------------------------------------
__global__ void embed_kernel(__nv_bfloat16* out, const __nv_bfloat16* tab, const int* ids, int H, float scale) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int r = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(tab + static_cast<size_t>(ids[r]) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    uint4 v = src[i];
    if (scale != 1.0f) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
      }
    }
    dst[i] = v;
  }
}

// ---- rmsnorm / add_norm with optional e4m3 1x128 output ---------------------------------------
// One CTA per row, 8 elements per thread per trip.  W % 8 == 0; quant output needs W % 128 == 0
// (16 threads own one 128-wide group, reduced with shuffles inside the half-warp).
template <bool ADD>
__global__ void __launch_bounds__(512)
norm_kernel(__nv_bfloat16* h_out, uint8_t* xq, float* sxq, int ld_sx, __nv_bfloat16* x_out,
            const __nv_bfloat16* x_in, const __nv_bfloat16* delta, const __nv_bfloat16* gamma, int W,
            int x_pitch, float eps, int plus_one) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ float rowbuf[];      // W floats
  __shared__ float red[32];
  const int r = blockIdx.x;
  const __nv_bfloat16* xr = x_in + static_cast<size_t>(r) * x_pitch;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(h[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
    if (ADD) {
      uint4 d = *reinterpret_cast<const uint4*>(delta + static_cast<size_t>(r) * W + i);
      const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&d);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __bfloat1622float2(dh[j]);
        // the sum is rounded to bf16 before the norm reads it, as the unfused pair would do
        oh[j] = __floats2bfloat162_rn(f[2 * j] + t.x, f[2 * j + 1] + t.y);
        float2 b = __bfloat1622float2(oh[j]);
        f[2 * j] = b.x; f[2 * j + 1] = b.y;
      }
      *reinterpret_cast<uint4*>(x_out + static_cast<size_t>(r) * W + i) = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { rowbuf[i + j] = f[j]; ss += f[j] * f[j]; }
  }
  const float tot = block_sum(ss, red);
  const float rs = rsqrtf(tot / W + eps);
  const int Wpad = (W + 255) & ~255;   // whole warps take every trip so the shuffles below are uniform
  for (int i = threadIdx.x * 8; i < Wpad; i += blockDim.x * 8) {
    const bool act = i < W;
    float y[8];
    float amax = 0.f;
    if (!act) {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = 0.f;
    } else if (gamma) {
      uint4 gv = *reinterpret_cast<const uint4*>(gamma + i);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 g = __bfloat1622float2(gh[j]);
        if (plus_one) { g.x += 1.f; g.y += 1.f; }
        y[2 * j] = rowbuf[i + 2 * j] * rs * g.x;
        y[2 * j + 1] = rowbuf[i + 2 * j + 1] * rs * g.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = rowbuf[i + j] * rs;
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      oh[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
      float2 b = __bfloat1622float2(oh[j]);     // quantise what the bf16 consumer would see
      y[2 * j] = b.x; y[2 * j + 1] = b.y;
      amax = fmaxf(amax, fmaxf(fabsf(b.x), fabsf(b.y)));
    }
    if (h_out && act) *reinterpret_cast<uint4*>(h_out + static_cast<size_t>(r) * W + i) = o;
    if (xq) {
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
      const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
      const float inv = 1.0f / sc;
      __nv_fp8x4_e4m3 q0(make_float4(y[0] * inv, y[1] * inv, y[2] * inv, y[3] * inv));
      __nv_fp8x4_e4m3 q1(make_float4(y[4] * inv, y[5] * inv, y[6] * inv, y[7] * inv));
      if (act) {
        *reinterpret_cast<uint2*>(xq + static_cast<size_t>(r) * W + i) =
            make_uint2(*reinterpret_cast<uint32_t*>(&q0), *reinterpret_cast<uint32_t*>(&q1));
        if ((threadIdx.x & 15) == 0) sxq[static_cast<size_t>(i >> 7) * ld_sx + r] = sc;
      }
    }
  }
}

__global__ void quant_act_kernel(uint8_t* xq, float* sxq, int ld_sx, const __nv_bfloat16* x, int K, int x_pitch) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int r = blockIdx.x;
  const int Kpad = (K + 255) & ~255;
  for (int i = threadIdx.x * 8; i < Kpad; i += blockDim.x * 8) {
    const bool act = i < K;
    uint4 v = act ? *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * x_pitch + i) : make_uint4(0, 0, 0, 0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float y[8], amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(h[j]); y[2 * j] = t.x; y[2 * j + 1] = t.y; amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y))); }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
    const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
    const float inv = 1.0f / sc;
    __nv_fp8x4_e4m3 q0(make_float4(y[0] * inv, y[1] * inv, y[2] * inv, y[3] * inv));
    __nv_fp8x4_e4m3 q1(make_float4(y[4] * inv, y[5] * inv, y[6] * inv, y[7] * inv));
    if (act) {
      *reinterpret_cast<uint2*>(xq + static_cast<size_t>(r) * K + i) = make_uint2(*reinterpret_cast<uint32_t*>(&q0), *reinterpret_cast<uint32_t*>(&q1));
      if ((threadIdx.x & 15) == 0) sxq[static_cast<size_t>(i >> 7) * ld_sx + r] = sc;
    }
  }
}

// ---- MLA --------------------------------------------------------------------------------------
// q [T][heads*(nope+rope)] -> q_nope_t [heads][T][nope] (the grouped absorb GEMM's A operand) and
// roped q_rope [heads][T][rope].  pair_mode 1 = interleaved (2i, 2i+1), 0 = half split.
__global__ void mla_q_prep_kernel(__nv_bfloat16* q_nope_t, __nv_bfloat16* q_rope, const __nv_bfloat16* q, int q_pitch,
                                  const float* rope_tab, const int* pos, int T, int heads, int nope, int rope, int pair_mode) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const __nv_bfloat16* src = q + static_cast<size_t>(t) * q_pitch + static_cast<size_t>(h) * (nope + rope);
  __nv_bfloat16* dn = q_nope_t + (static_cast<size_t>(h) * T + t) * nope;
  for (int i = threadIdx.x; i < nope; i += blockDim.x) dn[i] = src[i];
  const float* tab = rope_tab + static_cast<size_t>(pos[t]) * rope;
  const int half = rope / 2;
  __nv_bfloat16* dr = q_rope + (static_cast<size_t>(h) * T + t) * rope;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int ia = pair_mode ? 2 * i : i, ib = pair_mode ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(src[nope + ia]), b = __bfloat162float(src[nope + ib]);
    const float c = tab[i], s = tab[half + i];
    dr[ia] = __float2bfloat16(a * c - b * s);
    dr[ib] = __float2bfloat16(b * c + a * s);
  }
}

// q_abs [heads][T][latent] bf16 + q_rope [heads][T][rope] -> q8 [heads][T][latent+rope] e4m3, sq [heads][T]
__global__ void mla_q_quant_kernel(uint8_t* q8, float* sq, const __nv_bfloat16* q_abs, const __nv_bfloat16* q_rope,
                                   int T, int latent, int rope) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const size_t row = static_cast<size_t>(h) * T + t;
  const int W = latent + rope;
  __shared__ float red[32];
  float amax = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = __bfloat162float(i < latent ? q_abs[row * latent + i] : q_rope[row * rope + i - latent]);
    amax = fmaxf(amax, fabsf(v));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int w = 0; w < (blockDim.x + 31) / 32; ++w) amax = fmaxf(amax, red[w]);
  const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
  const float inv = 1.0f / sc;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = __bfloat162float(i < latent ? q_abs[row * latent + i] : q_rope[row * rope + i - latent]);
    q8[row * W + i] = __nv_fp8_e4m3(v * inv).__x;
  }
  if (threadIdx.x == 0) sq[row] = sc;
}

// kva [T][pitch] (latent | rope at col_ofs) -> RMSNorm(latent)*gamma, RoPE(rope) -> one e4m3 row of
// latent+rope bytes with one f32 scale, written to the token's cell of the paged cache.
__global__ void mla_kv_write_kernel(uint8_t* kv8, float* kv_scale, float* kv_smax, const __nv_bfloat16* kva, int pitch, int col_ofs,
                                    const __nv_bfloat16* gamma, const float* rope_tab, const int* pos, const int* slot_of,
                                    const int* page_table, int max_pages, int latent, int rope, float eps, int pair_mode) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ float rowf[];   // latent + rope
  __shared__ float red[32];
  const int t = blockIdx.x;
  const __nv_bfloat16* src = kva + static_cast<size_t>(t) * pitch + col_ofs;
  float ss = 0.f;
  for (int i = threadIdx.x; i < latent; i += blockDim.x) { const float v = __bfloat162float(src[i]); rowf[i] = v; ss += v * v; }
  const float tot = block_sum(ss, red);
  const float rs = rsqrtf(tot / latent + eps);
  const int p = pos[t];
  const float* tab = rope_tab + static_cast<size_t>(p) * rope;
  const int half = rope / 2;
  float amax = 0.f;
  for (int i = threadIdx.x; i < latent; i += blockDim.x) {
    const float v = __bfloat162float(__float2bfloat16(rowf[i] * rs * __bfloat162float(gamma[i])));
    rowf[i] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int ia = pair_mode ? 2 * i : i, ib = pair_mode ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(src[latent + ia]), b = __bfloat162float(src[latent + ib]);
    const float c = tab[i], s = tab[half + i];
    const float ra = __bfloat162float(__float2bfloat16(a * c - b * s)), rb = __bfloat162float(__float2bfloat16(b * c + a * s));
    rowf[latent + ia] = ra; rowf[latent + ib] = rb;
    amax = fmaxf(amax, fmaxf(fabsf(ra), fabsf(rb)));
  }
  amax = warp_max(amax);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int w = 0; w < (blockDim.x + 31) / 32; ++w) amax = fmaxf(amax, red[w]);
  const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
  const float inv = 1.0f / sc;
  const int page = page_table[static_cast<size_t>(slot_of[t]) * max_pages + p / 64];
  const size_t cell = static_cast<size_t>(page) * 64 + (p & 63);
  const int W = latent + rope;
  for (int i = threadIdx.x; i < W; i += blockDim.x) kv8[cell * W + i] = __nv_fp8_e4m3(rowf[i] * inv).__x;
  if (threadIdx.x == 0) {
    kv_scale[cell] = sc;
    // per-page upper bound of the scales (positive floats order like their bit patterns).  The
    // bound is never lowered when a page is recycled: the decode kernel only needs sk <= bound.
    if (kv_smax) atomicMax(reinterpret_cast<int*>(kv_smax) + static_cast<size_t>(page) * 4, __float_as_int(sc));
  }
}

// ---- router -----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ordered_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One warp per token.  table[t][j] = {expert id, gate bits}.  Selection key = score + bias, gate =
// unbiased score; groups are contiguous; group score = sum of the group's top-2 biased scores;
// ties go to the lowest group / expert id; gates renormalised over the k winners then scaled.
// One warp: the routing decision of token t from its E logits `lg` (global or shared memory); score / sel are E floats
// of scratch each.
__device__ void route_one_token(int2* table, const float* lg, const float* bias, int t, int E, int k, int n_group,
                                int topk_group, int sigmoid, int norm_topk, float route_scale, float* score, float* sel) {
  const int lane = threadIdx.x & 31;
  if (sigmoid) {
    for (int e = lane; e < E; e += 32) score[e] = 1.0f / (1.0f + __expf(-lg[e]));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = __expf(lg[e] - mx); score[e] = v; s += v; }
    s = warp_sum(s);
    for (int e = lane; e < E; e += 32) score[e] /= s;
  }
  for (int e = lane; e < E; e += 32) sel[e] = score[e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  if (n_group > 1) {
    const int gs = E / n_group;
    float gsc = -INFINITY;
    if (lane < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < gs; ++i) {
        const float v = sel[lane * gs + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gsc = a + b;
    }
    int rank = 0;
    for (int g = 0; g < n_group; ++g) {
      const float o = __shfl_sync(0xffffffffu, gsc, g);
      if (lane < n_group && (o > gsc || (o == gsc && g < lane))) ++rank;
    }
    const bool keep = lane < n_group && rank < topk_group;
    const uint32_t mask = __ballot_sync(0xffffffffu, keep);
    for (int e = lane; e < E; e += 32)
      if (!((mask >> (e / gs)) & 1u)) sel[e] = -INFINITY;
    __syncwarp();
  }
  float gsum = 0.f;
  float my_gate = 0.f;
  int my_eid = -1;
  for (int j = 0; j < k; ++j) {
    unsigned long long best = 0ull;
    for (int e = lane; e < E; e += 32) {
      const unsigned long long key = (static_cast<unsigned long long>(ordered_bits(sel[e])) << 32) | static_cast<uint32_t>(E - 1 - e);
      best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    const int e = E - 1 - static_cast<int>(best & 0xffffffffu);
    const float g = score[e];
    gsum += g;
    if (lane == j) { my_gate = g; my_eid = e; }
    __syncwarp();
    if (lane == 0) sel[e] = -INFINITY;
    __syncwarp();
  }
  if (lane < k) {
    float g = my_gate;
    if (norm_topk) g = g / fmaxf(gsum, 1e-20f);
    g *= route_scale;
    table[static_cast<size_t>(t) * k + lane] = make_int2(my_eid, __float_as_int(g));
  }
}

__global__ void router_topk_kernel(int2* table, const float* logits, const float* bias, int T, int E, int k,
                                   int n_group, int topk_group, int sigmoid, int norm_topk, float route_scale) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ float sm[];    // per warp: score[E], sel[E]
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* score = sm + warp * 2 * E;
  route_one_token(table, logits + static_cast<size_t>(t) * E, bias, t, E, k, n_group, topk_group, sigmoid, norm_topk,
                  route_scale, score, score + E);
}

// ---- MoE align / gather / combine -------------------------------------------------------------
// One CTA.  Counts the (token, slot) pairs routed to this rank's experts [e_base, e_base+e_local),
// writes grp_off[e_local+1], tile_prefix[e_local+1] (128-row tiles) and the pair<->row maps.
// shared_rows > 0 appends one more group (index e_local) that holds tokens [shared_tok_base, shared_tok_base +
// shared_rows) in order: the shared expert stacked behind the routed ones.  Its rows get pair_of_row = token * top_k,
// so the gather kernel (token = pair / top_k) copies them like any other row; grp_off / tile_prefix then have
// e_local + 2 entries and pair_of_row n_pairs + shared_rows.
// Body of the align step, run by one whole CTA; cnt = 2 * e_local ints of shared memory.
__device__ void moe_align_cta(const int2* table, int n_pairs, int e_base, int e_local, int* grp_off, int* tile_prefix,
                              int* row_of_pair, int* pair_of_row, int shared_rows, int shared_tok_base, int top_k, int* cnt) {
  int* cur = cnt + e_local;
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = table[p].x - e_base;
    if (e >= 0 && e < e_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, tiles = 0;
    for (int e = 0; e < e_local; ++e) {
      grp_off[e] = off; tile_prefix[e] = tiles; cur[e] = off;
      off += cnt[e]; tiles += (cnt[e] + 127) >> 7;
    }
    grp_off[e_local] = off; tile_prefix[e_local] = tiles;
    if (shared_rows > 0) { grp_off[e_local + 1] = off + shared_rows; tile_prefix[e_local + 1] = tiles + ((shared_rows + 127) >> 7); }
  }
  __syncthreads();
  const int routed = grp_off[e_local];
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = table[p].x - e_base;
    int row = -1;
    if (e >= 0 && e < e_local) { row = atomicAdd(&cur[e], 1); pair_of_row[row] = p; }
    row_of_pair[p] = row;
  }
  for (int t = threadIdx.x; t < shared_rows; t += blockDim.x) pair_of_row[routed + t] = (shared_tok_base + t) * top_k;
}

__global__ void moe_align_kernel(const int2* table, int n_pairs, int e_base, int e_local, int* grp_off, int* tile_prefix,
                                 int* row_of_pair, int* pair_of_row, int shared_rows, int shared_tok_base, int top_k) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ int cnt[];     // e_local counts, then e_local cursors
  moe_align_cta(table, n_pairs, e_base, e_local, grp_off, tile_prefix, row_of_pair, pair_of_row, shared_rows, shared_tok_base,
                top_k, cnt);
}

// Decode-size routing in one launch: router projection + top-k + align.  One CTA per token: the token's normalised
// hidden row is staged in shared memory as f32, each warp forms the dot products of its share of the E router rows
// (bf16 weights, f32 accumulation: the numerics of the GEMM it replaces), warp 0 makes the routing decision, and the
// CTA that finishes last (a ticket counter) lays the pairs out by expert.  Replaces a 1-tile GEMM (~20 us: a K = 7168
// reduction on one tile, split-K over a few CTAs), the top-k kernel and the align kernel.
// Shared memory: H floats | E logits | 2 E scratch | 2 e_local ints.
__global__ void __launch_bounds__(512)
moe_route_kernel(int2* table, float* logits_out, const __nv_bfloat16* x, int ldx, const __nv_bfloat16* w, const float* bias,
                 int T, int H, int E, int k, int n_group, int topk_group, int sigmoid, int norm_topk, float route_scale,
                 int do_align, int e_base, int e_local, int* grp_off, int* tile_prefix, int* row_of_pair, int* pair_of_row,
                 int shared_rows, int shared_tok_base, unsigned int* ticket, const plow::EpArgs epa, int use_ep, int* ep_cursor) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ float rsm[];
  float* xr = rsm;
  float* lg = xr + H;
  float* score = lg + E;
  int* cnt = reinterpret_cast<int*>(score + 2 * E);
  __shared__ int is_last;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const __nv_bfloat16* xp = x + static_cast<size_t>(t) * ldx;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(xp)[i];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h2[j]);
      xr[i * 8 + 2 * j] = f.x; xr[i * 8 + 2 * j + 1] = f.y;
    }
  }
  __syncthreads();
  // The loop is bound by L2 latency, not bandwidth: every lane keeps 16 independent 16-byte loads in flight.  A warp
  // works on four (router row, K part) slots at a time: R = 1, 2 or 4 rows, each cut into 4 / R parts along K.
  const int per_warp = (E + nw - 1) / nw;
  const int R = per_warp >= 4 ? 4 : per_warp >= 2 ? 2 : 1, P = 4 / R;
  const int C = H / 8;                                       // 16-byte chunks per row
  const int part_len = ((C + 32 * P - 1) / (32 * P)) * 32;   // chunks per part, a multiple of the warp width
  for (int e0 = warp; e0 < E; e0 += R * nw) {
    const uint4* wp[4];
    int lo[4];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wp[j] = reinterpret_cast<const uint4*>(w + static_cast<size_t>(min(e0 + (j % R) * nw, E - 1)) * H);
      lo[j] = (j / R) * part_len;
    }
    for (int i0 = lane; i0 < part_len; i0 += 128) {
      // phase 1: all 16 loads of this batch (4 slots x 4 strides) are issued before any is used
      uint4 v[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int ii = i0 + u * 32;
          v[u][j] = (ii < part_len && lo[j] + ii < C) ? __ldg(wp[j] + lo[j] + ii) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = min(lo[j] + i0 + u * 32, C - 1);
          const float4 a = *reinterpret_cast<const float4*>(xr + i * 8), b = *reinterpret_cast<const float4*>(xr + i * 8 + 4);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[u][j]);
          const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]), f2 = __bfloat1622float2(h2[2]),
                       f3 = __bfloat1622float2(h2[3]);
          float s = acc[j];
          s = fmaf(a.x, f0.x, s); s = fmaf(a.y, f0.y, s); s = fmaf(a.z, f1.x, s); s = fmaf(a.w, f1.y, s);
          s = fmaf(b.x, f2.x, s); s = fmaf(b.y, f2.y, s); s = fmaf(b.z, f3.x, s); s = fmaf(b.w, f3.y, s);
          acc[j] = s;
        }
    }
    // slots j, j + R, ... hold the K parts of row j
    if (R == 1) { acc[0] += acc[1] + acc[2] + acc[3]; }
    else if (R == 2) { acc[0] += acc[2]; acc[1] += acc[3]; }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j >= R) break;
      const float r = warp_sum(acc[j]);
      const int e = e0 + j * nw;
      if (lane == 0 && e < E) { lg[e] = r; if (logits_out) logits_out[static_cast<size_t>(t) * E + e] = r; }
    }
  }
  __syncthreads();
  if (warp == 0)
    route_one_token(table, lg, bias, t, E, k, n_group, topk_group, sigmoid, norm_topk, route_scale, score, score + E);
  if (!do_align && !use_ep) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    is_last = atomicAdd(ticket, 1u) == static_cast<unsigned int>(T) - 1u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x == 0) *ticket = 0u;       // re-armed for the next launch (stream order separates launches)
  if (use_ep) {
    // expert parallelism: this rank's per-expert pair counts go to every peer's count matrix, followed by one release
    // flag per peer (what the separate counts kernel of csrc/comm/ep.cu does); `cnt` holds E ints here
    for (int e = threadIdx.x; e < epa.E; e += blockDim.x) { cnt[e] = 0; ep_cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < T * k; p += blockDim.x) atomicAdd(&cnt[__ldcg(&table[p].x)], 1);
    __syncthreads();
    const uint32_t epn = *epa.epoch + 1;
    for (int d = 0; d < epa.W; ++d) {
      int* dst = reinterpret_cast<int*>(epa.peer[d] + epa.L.cnt_all) + epa.me * epa.E;
      for (int e = threadIdx.x; e < epa.E; e += blockDim.x) dst[e] = cnt[e];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < epa.W)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(epa.peer[threadIdx.x] + epa.L.cnt_flag) + epa.me * 32),
                   "r"(epn) : "memory");
    if (threadIdx.x == 0) *epa.epoch = epn;
    return;
  }
  moe_align_cta(table, T * k, e_base, e_local, grp_off, tile_prefix, row_of_pair, pair_of_row, shared_rows, shared_tok_base, k,
                cnt);
}

// Rows of the quantised activations gathered into expert order (scales are transposed [kb][row]).
__global__ void moe_gather_kernel(uint8_t* xs, float* sxs, int ld_sxs, const uint8_t* xq, const float* sx, int ld_sx,
                                  const int* pair_of_row, const int* n_rows, int top_k, int K) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int row = blockIdx.x;
  if (row >= *n_rows) return;
  const int tok = pair_of_row[row] / top_k;
  const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<size_t>(tok) * K);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * K);
  for (int i = threadIdx.x; i < K / 16; i += blockDim.x) dst[i] = src[i];
  for (int kb = threadIdx.x; kb < K / 128; kb += blockDim.x) sxs[static_cast<size_t>(kb) * ld_sxs + row] = sx[static_cast<size_t>(kb) * ld_sx + tok];
}

// out[t] = shared[t] (optional) + sum_j gate[t][j] * y[row_of_pair[t*k+j]]   (fixed slot order, f32)
// shared_base != NULL: the shared expert ran as a group of the grouped GEMM and its row of token t is
// shared[*shared_base + t] (the group's first row is only known on the device).
__global__ void moe_combine_kernel(__nv_bfloat16* out, const __nv_bfloat16* y, const __nv_bfloat16* shared,
                                   const int2* table, const int* row_of_pair, int top_k, int H, const int* shared_base) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  // slot metadata first, then all of a thread's loads at once (one 16-byte unit per thread, grid.y covers H)
  constexpr int kMaxK = 16;
  __shared__ int s_row[kMaxK];
  __shared__ float s_gate[kMaxK];
  const int t = blockIdx.x;
  if (threadIdx.x < top_k && threadIdx.x < kMaxK) {
    s_row[threadIdx.x] = row_of_pair[t * top_k + threadIdx.x];
    s_gate[threadIdx.x] = __int_as_float(table[t * top_k + threadIdx.x].y);
  }
  __syncthreads();
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= H) return;
  uint4 v[kMaxK];
#pragma unroll
  for (int s = 0; s < kMaxK; ++s) {
    v[s] = make_uint4(0u, 0u, 0u, 0u);
    if (s < top_k && s_row[s] >= 0) v[s] = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(s_row[s]) * H + i);
  }
  float acc[8];
  if (shared) {
    const size_t srow = static_cast<size_t>(t) + (shared_base ? *shared_base : 0);
    const uint4 sv = *reinterpret_cast<const uint4*>(shared + srow * H + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&sv);
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  }
#pragma unroll
  for (int s = 0; s < kMaxK; ++s) {            // fixed slot order
    if (s < top_k && s_row[s] >= 0) {
      const float g = s_gate[s];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); acc[2 * j] += g * f.x; acc[2 * j + 1] += g * f.y; }
    }
  }
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + i) = o;
}


// ---- argmax / gather --------------------------------------------------------------------------
__global__ void argmax_kernel(int* out, const float* logits, int V) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ unsigned long long red[32];
  const float* row = logits + static_cast<size_t>(blockIdx.x) * V;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const unsigned long long key = (static_cast<unsigned long long>(ordered_bits(row[i])) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(i));
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
    if (threadIdx.x == 0) out[blockIdx.x] = static_cast<int>(~static_cast<uint32_t>(best & 0xffffffffu));
  }
}

// Vocabulary-sharded arg-max: the row's best (ordered score << 32 | ~global index) key of this rank's shard; the ranks'
// keys are folded with a max (lowest global index wins ties), see argmax_fin_kernel.
__global__ void argmax_key_kernel(unsigned long long* keys, const float* logits, int V, int vocab_ofs) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ unsigned long long red[32];
  const float* row = logits + static_cast<size_t>(blockIdx.x) * V;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const unsigned long long key = (static_cast<unsigned long long>(ordered_bits(row[i])) << 32) |
                                   static_cast<uint32_t>(~static_cast<uint32_t>(i + vocab_ofs));
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
    if (threadIdx.x == 0) keys[blockIdx.x] = best;
  }
}

// keys [world][R] gathered from the ranks -> ids [R]
__global__ void argmax_fin_kernel(int* out, const unsigned long long* keys, int R, int world) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  unsigned long long best = 0ull;
  for (int w = 0; w < world; ++w) { const unsigned long long k = keys[static_cast<size_t>(w) * R + r]; best = k > best ? k : best; }
  out[r] = static_cast<int>(~static_cast<uint32_t>(best & 0xffffffffu));
}

__global__ void row_gather_kernel(__nv_bfloat16* out, const __nv_bfloat16* x, const int* rows, int W) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(rows[blockIdx.x]) * W);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(blockIdx.x) * W);
  for (int i = threadIdx.x; i < W / 8; i += blockDim.x) dst[i] = src[i];
}

// [heads][T][W] -> [T][heads*W] (attention output back to token-major for o_proj)
__global__ void head_to_token_kernel(__nv_bfloat16* out, const __nv_bfloat16* x, int T, int heads, int W) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(x + (static_cast<size_t>(h) * T + t) * W);
  uint4* dst = reinterpret_cast<uint4*>(out + (static_cast<size_t>(t) * heads + h) * W);
  for (int i = threadIdx.x; i < W / 8; i += blockDim.x) dst[i] = src[i];
}

// ---- residual add / SiLU-GLU on bf16 rows (8 elements per thread) ------------------------------
// mode 0: out = a + b;  mode 1: out = silu(a) * b.  Both are computed in f32 and rounded once.
__global__ void eltwise2_kernel(__nv_bfloat16* out, const __nv_bfloat16* a, const __nv_bfloat16* b, size_t n8, int mode) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint4 va = reinterpret_cast<const uint4*>(a)[i], vb = reinterpret_cast<const uint4*>(b)[i];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hb[j]);
      if (mode == 0) oh[j] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
      else oh[j] = __floats2bfloat162_rn(x.x / (1.0f + __expf(-x.x)) * y.x, x.y / (1.0f + __expf(-x.y)) * y.y);
    }
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

inline int ok() { cudaError_t e = cudaGetLastError(); return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e); }

}  // namespace

#define S(x) reinterpret_cast<cudaStream_t>(x)
typedef __nv_bfloat16 bf16;

extern "C" {

int plow_embed(void* out, const void* tab, const int* ids, int R, int H, float scale, void* st) {
  if (H % 8) return -1;
  plow::launch_serial(embed_kernel, dim3(R), dim3(256), 0, S(st), (bf16*)out, (const bf16*)tab, ids, H, scale);
  return ok();
}

int plow_rmsnorm(void* h_out, void* xq, float* sxq, int ld_sx, const void* x, const void* gamma, int R, int W,
                 int x_pitch, float eps, int plus_one, void* st) {
  if (W % 8 || (xq && W % 128) || W * 4 > 200 * 1024) return -1;
  static plow::DeviceOnce attr;
  if (plow::ensure_smem(attr, norm_kernel<false>, 200 * 1024) != cudaSuccess) return 3000;
  const int threads = W >= 4096 ? 512 : (W >= 1024 ? 128 : 64);
  plow::launch_serial(norm_kernel<false>, dim3(R), dim3(threads), W * 4, S(st), (bf16*)h_out, (uint8_t*)xq, sxq, ld_sx, nullptr, (const bf16*)x, nullptr,
                                                   (const bf16*)gamma, W, x_pitch ? x_pitch : W, eps, plus_one);
  return ok();
}

int plow_add_norm(void* h_out, void* xq, float* sxq, int ld_sx, void* x_out, const void* x_in, const void* delta,
                  const void* gamma, int R, int W, float eps, int plus_one, void* st) {
  if (W % 8 || (xq && W % 128) || W * 4 > 200 * 1024) return -1;
  static plow::DeviceOnce attr;
  if (plow::ensure_smem(attr, norm_kernel<true>, 200 * 1024) != cudaSuccess) return 3000;
  const int threads = W >= 4096 ? 512 : (W >= 1024 ? 128 : 64);
  plow::launch_serial(norm_kernel<true>, dim3(R), dim3(threads), W * 4, S(st), (bf16*)h_out, (uint8_t*)xq, sxq, ld_sx, (bf16*)x_out, (const bf16*)x_in,
                                                  (const bf16*)delta, (const bf16*)gamma, W, W, eps, plus_one);
  return ok();
}

int plow_quant_act(void* xq, float* sxq, int ld_sx, const void* x, int R, int K, int x_pitch, void* st) {
  if (K % 128) return -1;
  plow::launch_serial(quant_act_kernel, dim3(R), dim3(K >= 4096 ? 512 : 128), 0, S(st), (uint8_t*)xq, sxq, ld_sx, (const bf16*)x, K, x_pitch ? x_pitch : K);
  return ok();
}

int plow_mla_q_prep(void* q_nope_t, void* q_rope, const void* q, int q_pitch, const float* rope_tab, const int* pos, int T,
                    int heads, int nope, int rope, int pair_mode, void* st) {
  plow::launch_serial(mla_q_prep_kernel, dim3(T, heads), dim3(64), 0, S(st), (bf16*)q_nope_t, (bf16*)q_rope, (const bf16*)q, q_pitch, rope_tab, pos, T,
                                                      heads, nope, rope, pair_mode);
  return ok();
}

int plow_mla_q_quant(void* q8, float* sq, const void* q_abs, const void* q_rope, int T, int heads, int latent, int rope, void* st) {
  plow::launch_serial(mla_q_quant_kernel, dim3(T, heads), dim3(128), 0, S(st), (uint8_t*)q8, sq, (const bf16*)q_abs, (const bf16*)q_rope, T, latent, rope);
  return ok();
}

int plow_mla_kv_write(void* kv8, float* kv_scale, float* kv_smax, const void* kva, int pitch, int col_ofs, const void* gamma,
                      const float* rope_tab, const int* pos, const int* slot_of, const int* page_table, int max_pages, int T,
                      int latent, int rope, float eps, int pair_mode, void* st) {
  plow::launch_serial(mla_kv_write_kernel, dim3(T), dim3(128), (latent + rope) * 4, S(st), (uint8_t*)kv8, kv_scale, kv_smax, (const bf16*)kva, pitch, col_ofs,
                                                              (const bf16*)gamma, rope_tab, pos, slot_of, page_table, max_pages,
                                                              latent, rope, eps, pair_mode);
  return ok();
}

int plow_router_topk(void* table, const float* logits, const float* bias, int T, int E, int k, int n_group, int topk_group,
                     int sigmoid, int norm_topk, float route_scale, void* st) {
  if (k > 32 || n_group > 32 || E % (n_group > 0 ? n_group : 1)) return -1;
  const int wpb = 4;
  plow::launch_serial(router_topk_kernel, dim3((T + wpb - 1) / wpb), dim3(wpb * 32), wpb * 2 * E * 4, S(st), (int2*)table, logits, bias, T, E, k, n_group,
                                                                                topk_group, sigmoid, norm_topk, route_scale);
  return ok();
}

// x bf16 [T][ldx] (normalised hidden rows), w bf16 [E][H].  logits_out (f32 [T][E]) may be null.  With do_align the
// align outputs are written as by plow_moe_align; `ticket` is one zero-initialised word that the kernel re-arms.
int plow_moe_route(void* table, float* logits_out, const void* x, int ldx, const void* w, const float* bias, int T, int H, int E,
                   int k, int n_group, int topk_group, int sigmoid, int norm_topk, float route_scale, int do_align, int e_base,
                   int e_local, int* grp_off, int* tile_prefix, int* row_of_pair, int* pair_of_row, int shared_rows,
                   int shared_tok_base, void* ticket, const void* ep_args, int* ep_cursor, void* st) {
  if (k > 32 || n_group > 32 || E % (n_group > 0 ? n_group : 1) || H % 8 || (ldx % 8) || T <= 0) return -1;
  if (ep_args && (do_align || !ep_cursor)) return -1;
  const size_t smem = static_cast<size_t>(H + 3 * E) * 4 + static_cast<size_t>(do_align ? 2 * e_local : (ep_args ? E : 0)) * 4;
  if (smem > 200 * 1024) return -2;
  static plow::DeviceOnce attr;
  if (plow::ensure_smem(attr, moe_route_kernel, 200 * 1024) != cudaSuccess) return -3;
  plow::launch_serial(moe_route_kernel, dim3(T), dim3(512), smem, S(st), (int2*)table, logits_out, (const bf16*)x, ldx, (const bf16*)w,
                      bias, T, H, E, k, n_group, topk_group, sigmoid, norm_topk, route_scale, do_align, e_base, e_local, grp_off,
                      tile_prefix, row_of_pair, pair_of_row, shared_rows, shared_tok_base, (unsigned int*)ticket,
                      ep_args ? *static_cast<const plow::EpArgs*>(ep_args) : plow::EpArgs{}, ep_args ? 1 : 0, ep_cursor);
  return ok();
}

int plow_moe_align(const void* table, int n_pairs, int e_base, int e_local, int* grp_off, int* tile_prefix, int* row_of_pair,
                   int* pair_of_row, int shared_rows, int shared_tok_base, int top_k, void* st) {
  plow::launch_serial(moe_align_kernel, dim3(1), dim3(1024), 2 * e_local * 4, S(st), (const int2*)table, n_pairs, e_base, e_local, grp_off, tile_prefix,
                                                        row_of_pair, pair_of_row, shared_rows, shared_tok_base, top_k);
  return ok();
}

int plow_moe_gather(void* xs, float* sxs, int ld_sxs, const void* xq, const float* sx, int ld_sx, const int* pair_of_row,
                    const int* n_rows, int max_rows, int top_k, int K, void* st) {
  if (K % 128) return -1;
  plow::launch_serial(moe_gather_kernel, dim3(max_rows), dim3(128), 0, S(st), (uint8_t*)xs, sxs, ld_sxs, (const uint8_t*)xq, sx, ld_sx, pair_of_row, n_rows, top_k, K);
  return ok();
}

int plow_moe_combine(void* out, const void* y, const void* shared, const void* table, const int* row_of_pair, int T, int top_k,
                     int H, const int* shared_base, void* st) {
  if (H % 8 || top_k > 16) return -1;
  plow::launch_serial(moe_combine_kernel, dim3(T, (H / 8 + 255) / 256), dim3(256), 0, S(st), (bf16*)out, (const bf16*)y, (const bf16*)shared, (const int2*)table, row_of_pair, top_k, H, shared_base);
  return ok();
}

int plow_argmax(int* out, const float* logits, int R, int V, void* st) {
  plow::launch_serial(argmax_kernel, dim3(R), dim3(1024), 0, S(st), out, logits, V);
  return ok();
}

int plow_argmax_key(void* keys, const float* logits, int R, int V, int vocab_ofs, void* st) {
  plow::launch_serial(argmax_key_kernel, dim3(R), dim3(1024), 0, S(st), static_cast<unsigned long long*>(keys), logits, V, vocab_ofs);
  return ok();
}

int plow_argmax_fin(int* out, const void* keys, int R, int world, void* st) {
  plow::launch_serial(argmax_fin_kernel, dim3((R + 127) / 128), dim3(128), 0, S(st), out, static_cast<const unsigned long long*>(keys), R, world);
  return ok();
}

int plow_row_gather(void* out, const void* x, const int* rows, int n, int W, void* st) {
  if (W % 8) return -1;
  plow::launch_serial(row_gather_kernel, dim3(n), dim3(128), 0, S(st), (bf16*)out, (const bf16*)x, rows, W);
  return ok();
}

// out = a + b (mode 0) or silu(a) * b (mode 1) over n bf16 elements (n % 8 == 0, 16-byte aligned pointers)
int plow_eltwise2(void* out, const void* a, const void* b, long long n, int mode, void* st) {
  if (n % 8 || n <= 0) return -1;
  const size_t n8 = static_cast<size_t>(n) / 8;
  const unsigned grid = static_cast<unsigned>(n8 / 256 + 1 < 1184 ? n8 / 256 + 1 : 1184);
  plow::launch_serial(eltwise2_kernel, dim3(grid), dim3(256), 0, S(st), (bf16*)out, (const bf16*)a, (const bf16*)b, n8, mode);
  return ok();
}

int plow_head_to_token(void* out, const void* x, int T, int heads, int W, void* st) {
  if (W % 8) return -1;
  plow::launch_serial(head_to_token_kernel, dim3(T, heads), dim3(32), 0, S(st), (bf16*)out, (const bf16*)x, T, heads, W);
  return ok();
}

}  // extern "C"
