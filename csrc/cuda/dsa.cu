// Sparse-attention "lightning indexer": index-key cache write, index scores on tcgen05, exact top-k.
//
//   k_idx[t]   = RoPE(LayerNorm(wk x_t) * gamma + beta)                    -> e4m3 row + f32 scale, paged
//   score[r,t] = sum_h w[r,h] * ReLU(q_idx[r,h] . k_idx[t])                 for t <= pos[r]
//   sel[r]     = the top_k positions by (score desc, lowest index on ties);  rows with at most top_k
//                visible positions emit the identity, trailing slots are -1.
// Reference semantics: runtime/common/dev_isa.h:516-534 and :1083-1115 (7-pass radix select over a
// monotone packed key, live token-granular kv_len), runtime/nvidia/op_dsa.cuh.
//
// Scores: one CTA per (128-token tile, query row).  The tile's keys are the A operand (M = 128 tokens),
// the row's 64 index heads the B operand (N = 64), K = 128 e4m3: D[token][head] lands with one token
// per TMEM lane, so the weighted ReLU sum over heads is a private 64-column loop per thread and the
// score leaves the kernel with one coalesced store.  Small CTAs (24 KB smem, 64 TMEM columns) let
// eight of them overlap per SM, which hides the single TMA -> MMA -> epilogue chain of each.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace plow {

constexpr int kIdxDim = 128;
constexpr int kIdxHeads = 64;
constexpr int kIdxPage = 64;

// One warp per row: LayerNorm (+bias), RoPE on the first `rot` dims, e4m3 quantisation with one scale.
__global__ void dsa_k_write_kernel(uint8_t* cache, float* cache_scale, const __nv_bfloat16* k, int ld_k,
                                   const float* gamma, const float* beta, const float* rope_tab, const int* pos,
                                   const int* seq, const int* page_table, int max_pages, int rows, int rot,
                                   int pair_mode, float eps) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ float buf[8][kIdxDim];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + wib;
  if (r >= rows) return;
  const int p = pos[r];
  if (p < 0) return;
  float v[4], s = 0.f, ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = __bfloat162float(k[static_cast<size_t>(r) * ld_k + lane + 32 * j]); s += v[j]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float mean = s / kIdxDim;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] -= mean; ss += v[j] * v[j]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rs = rsqrtf(ss / kIdxDim + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    buf[wib][c] = v[j] * rs * gamma[c] + (beta ? beta[c] : 0.f);
  }
  __syncwarp();
  const int half = rot / 2;
  const float* tab = rope_tab + static_cast<size_t>(p) * rot;
  float o4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    float y = buf[wib][c];
    if (c < rot) {
      int i, partner; bool first;
      if (pair_mode) { i = c >> 1; first = !(c & 1); partner = c ^ 1; }
      else { first = c < half; i = first ? c : c - half; partner = first ? c + half : c - half; }
      const float x = buf[wib][c], z = buf[wib][partner], cs = tab[i], sn = tab[half + i];
      y = first ? x * cs - z * sn : x * cs + z * sn;
    }
    o4[j] = y;
  }
  float amax = fmaxf(fmaxf(fabsf(o4[0]), fabsf(o4[1])), fmaxf(fabsf(o4[2]), fabsf(o4[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = fmaxf(amax, 1e-10f) / 448.0f, inv = 1.0f / sc;
  const int page = page_table[static_cast<size_t>(seq[r]) * max_pages + p / kIdxPage];
  const size_t cell = static_cast<size_t>(page) * kIdxPage + p % kIdxPage;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_fp8_e4m3 q(o4[j] * inv);
    cache[cell * kIdxDim + lane + 32 * j] = *reinterpret_cast<const uint8_t*>(&q);
  }
  if (lane == 0) cache_scale[cell] = sc;
}

// One warp per (row, head): RoPE on the first `rot` dims, e4m3 with one scale; the scale and the head
// weight are folded into w_out[r][h] = w[r][h] * scale so the score kernel multiplies once.
__global__ void dsa_q_prep_kernel(uint8_t* q8, float* w_out, const __nv_bfloat16* q, int ld_q, const float* w, int ld_w,
                                  const float* rope_tab, const int* pos, int rows, int rot, int pair_mode) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ float buf[8][kIdxDim];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * 8 + wib;
  if (item >= rows * kIdxHeads) return;
  const int r = item / kIdxHeads, h = item % kIdxHeads;
  const int p = max(pos[r], 0);
#pragma unroll
  for (int j = 0; j < 4; ++j) buf[wib][lane + 32 * j] = __bfloat162float(q[static_cast<size_t>(r) * ld_q + h * kIdxDim + lane + 32 * j]);
  __syncwarp();
  const int half = rot / 2;
  const float* tab = rope_tab + static_cast<size_t>(p) * rot;
  float o4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    float y = buf[wib][c];
    if (c < rot) {
      int i, partner; bool first;
      if (pair_mode) { i = c >> 1; first = !(c & 1); partner = c ^ 1; }
      else { first = c < half; i = first ? c : c - half; partner = first ? c + half : c - half; }
      const float x = buf[wib][c], z = buf[wib][partner], cs = tab[i], sn = tab[half + i];
      y = first ? x * cs - z * sn : x * cs + z * sn;
    }
    o4[j] = y;
  }
  float amax = fmaxf(fmaxf(fabsf(o4[0]), fabsf(o4[1])), fmaxf(fabsf(o4[2]), fabsf(o4[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = fmaxf(amax, 1e-10f) / 448.0f, inv = 1.0f / sc;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_fp8_e4m3 e(o4[j] * inv);
    q8[(static_cast<size_t>(r) * kIdxHeads + h) * kIdxDim + lane + 32 * j] = *reinterpret_cast<const uint8_t*>(&e);
  }
  if (lane == 0) w_out[r * kIdxHeads + h] = w[static_cast<size_t>(r) * ld_w + h] * sc;
}

__global__ void __launch_bounds__(128)
dsa_score_kernel(float* scores, int ld_scores, const float* w, const float* kscale, const int* pos, const int* seq,
                 const int* page_table, int max_pages, int* status, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_q) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int r = blockIdx.y, t0 = blockIdx.x * 128;
  const int len = pos[r] + 1;
  if (t0 >= len) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* k_smem = smem;                 // 128 tokens x 128 B
  uint8_t* q_smem = smem + 16384;         // 64 heads x 128 B
  uint64_t* tma_bar = reinterpret_cast<uint64_t*>(smem + 24576);
  uint64_t* mma_bar = tma_bar + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(mma_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* w_smem = reinterpret_cast<float*>(smem + 24576 + 64);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(tma_bar, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (threadIdx.x < kIdxHeads) w_smem[threadIdx.x] = w[r * kIdxHeads + threadIdx.x];
  if (warp == 0) { tmem_alloc(tmem_holder, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_holder;
  const int* pt = page_table + static_cast<size_t>(seq[r]) * max_pages;
  const int pg0 = pt[t0 / kIdxPage];
  const int pg1 = (t0 + kIdxPage < len) ? pt[t0 / kIdxPage + 1] : pg0;
  if (warp == 0 && elect_one()) {
    mbar_expect_tx(tma_bar, 16384 + 8192);
    tma_load_2d(k_smem, &tm_k, 0, pg0 * kIdxPage, tma_bar);
    tma_load_2d(k_smem + 8192, &tm_k, 0, pg1 * kIdxPage, tma_bar);
    tma_load_2d(q_smem, &tm_q, 0, r * kIdxHeads, tma_bar);
    if (mbar_wait(tma_bar, 0, abort_flag)) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc(128, 64, 0, 0);
      const uint64_t kd = umma_desc_k128(smem_u32(k_smem)), qd = umma_desc_k128(smem_u32(q_smem));
#pragma unroll
      for (int k = 0; k < 4; ++k) tc_mma_f8(tm, kd + 2 * k, qd + 2 * k, idesc, k > 0);
    } else {
      *abort_flag = 1;
      atomicCAS(status, 0, PLOW_ERR_TMA_WAIT | kTagDsa);
    }
    tc_commit(mma_bar);
  }
  __syncwarp();
  const bool ok = mbar_wait(mma_bar, 0, abort_flag) && !*abort_flag;
  tc_fence_after();
  if (ok) {
    uint32_t d[64];
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    tmem_ld32(tm + lane_addr, d);
    tmem_ld32(tm + lane_addr + 32, d + 32);
    tmem_ld_wait();
    float acc = 0.f;
#pragma unroll
    for (int h = 0; h < 64; ++h) acc = fmaf(w_smem[h], fmaxf(__uint_as_float(d[h]), 0.f), acc);
    const int t = t0 + threadIdx.x;
    if (t < len) {
      const int page = threadIdx.x < kIdxPage ? pg0 : pg1;
      scores[static_cast<size_t>(r) * ld_scores + t] = acc * kscale[static_cast<size_t>(page) * kIdxPage + (t % kIdxPage)];
    }
  } else if (threadIdx.x == 0) {
    atomicCAS(status, 0, PLOW_ERR_TMEM_WAIT | kTagDsa);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tm, 64); }
}

__device__ __forceinline__ unsigned long long dsa_key(float s, int idx) {
  const uint32_t b = __float_as_uint(s);
  const uint32_t o = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(o) << 20) | static_cast<unsigned long long>(0xFFFFFu - static_cast<uint32_t>(idx));
}

// One CTA per row.  Keys are unique (the index is part of the key), so exactly top_k survive.
__global__ void __launch_bounds__(1024)
dsa_topk_kernel(int* sel, const float* scores, int ld_scores, const int* pos, int top_k) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sh_digit, sh_above;
  __shared__ int scan[32];
  const int r = blockIdx.x;
  const int len = pos[r] + 1;
  int* out = sel + static_cast<size_t>(r) * top_k;
  if (len <= top_k) {
    for (int j = threadIdx.x; j < top_k; j += blockDim.x) out[j] = j < len ? j : -1;
    return;
  }
  const float* sc = scores + static_cast<size_t>(r) * ld_scores;
  unsigned long long prefix = 0, mask = 0;
  uint32_t above = 0;
  for (int shift = 48; shift >= 0; shift -= 8) {     // 52-bit keys: 7 passes of 8 bits
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      const unsigned long long k = dsa_key(sc[i], i);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t acc = above;
      int d = 255;
      for (; d > 0; --d) {
        if (acc + hist[d] >= static_cast<uint32_t>(top_k)) break;
        acc += hist[d];
      }
      sh_digit = d; sh_above = acc;
    }
    __syncthreads();
    prefix |= static_cast<unsigned long long>(sh_digit) << shift;
    mask |= 255ull << shift;
    above = sh_above;
    __syncthreads();
  }
  // compaction in index order
  const int chunk = (len + blockDim.x - 1) / blockDim.x;
  const int i0 = threadIdx.x * chunk, i1 = min(len, i0 + chunk);
  int local = 0;
  for (int i = i0; i < i1; ++i) local += dsa_key(sc[i], i) >= prefix;
  int incl = local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) scan[warp] = incl;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < warp; ++w) base += scan[w];
  int at = base + incl - local;
  for (int i = i0; i < i1; ++i)
    if (dsa_key(sc[i], i) >= prefix && at < top_k) out[at++] = i;
}

// One warp per (query row, selected slot): copies the selected token's latent-cache row (row_bytes) and scale into
// the row's compact cache, whose pages the dense decode kernel then walks; the per-page scale bound is kept with an
// integer atomic max (scales are positive floats).  Unselected slots (-1) are left alone: the compact length hides them.
__global__ void dsa_gather_kernel(uint8_t* ckv, float* cscale, float* csmax, int* clen, const int* sel, int top_k,
                                  const uint8_t* cache, const float* scale, const int* pos, const int* seq,
                                  const int* page_table, int max_pages, int rows, int row_bytes) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + wib;
  if (item >= static_cast<long long>(rows) * top_k) return;
  const int r = static_cast<int>(item / top_k), j = static_cast<int>(item % top_k);
  if (j == 0 && lane == 0) clen[r] = max(0, min(pos[r] + 1, top_k));
  const int t = sel[item];
  if (t < 0) return;
  const int page = page_table[static_cast<size_t>(seq[r]) * max_pages + t / kIdxPage];
  const size_t src = static_cast<size_t>(page) * kIdxPage + t % kIdxPage;
  const size_t dst = static_cast<size_t>(r) * top_k + j;                 // compact pages are contiguous per row
  const uint4* s4 = reinterpret_cast<const uint4*>(cache + src * row_bytes);
  uint4* d4 = reinterpret_cast<uint4*>(ckv + dst * row_bytes);
  for (int u = lane; u < row_bytes / 16; u += 32) d4[u] = s4[u];
  if (lane == 0) {
    const float sc = scale[src];
    cscale[dst] = sc;
    atomicMax(reinterpret_cast<int*>(csmax + (dst / kIdxPage) * 4), __float_as_int(sc));
  }
}

}  // namespace plow

extern "C" {

// k bf16 [rows][ld_k] (128 index dims); cache e4m3 [n_pages][64][128]; cache_scale f32 [n_pages][64].
int plow_dsa_k_write(void* cache, float* cache_scale, const void* k, int ld_k, const float* gamma, const float* beta,
                     const float* rope_tab, const int* pos, const int* seq, const int* page_table, int max_pages,
                     int rows, int rot, int pair_mode, float eps, void* stream) {
  using namespace plow;
  if (rows <= 0 || rot > kIdxDim || rot % 2) return -1;
  plow::launch_serial(dsa_k_write_kernel, dim3((rows + 7) / 8), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      static_cast<uint8_t*>(cache), cache_scale, static_cast<const __nv_bfloat16*>(k), ld_k, gamma, beta, rope_tab, pos, seq,
      page_table, max_pages, rows, rot, pair_mode, eps);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// q bf16 [rows][ld_q] (64 heads x 128); w f32 [rows][ld_w] head weights; scratch q8 e4m3 [rows][64][128], wq f32 [rows][64];
// scores f32 [rows][ld_scores] (scratch, ld_scores >= max visible length); sel int32 [rows][top_k].
int plow_dsa_select(int* sel, float* scores, int ld_scores, void* q8, float* wq, const void* q, int ld_q, const float* w,
                    int ld_w, const void* cache, const float* cache_scale, int64_t n_pages, const float* rope_tab,
                    const int* pos, const int* seq, const int* page_table, int max_pages, int rows, int rot, int pair_mode,
                    int top_k, int max_len, int* status, void* stream_) {
  using namespace plow;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0 || top_k <= 0 || max_len <= 0 || max_len > ld_scores || max_len > (1 << 20)) return -1;
  plow::launch_serial(dsa_q_prep_kernel, dim3((rows * kIdxHeads + 7) / 8), dim3(256), 0, stream, static_cast<uint8_t*>(q8), wq, static_cast<const __nv_bfloat16*>(q),
                                                                    ld_q, w, ld_w, rope_tab, pos, rows, rot, pair_mode);
  CUtensorMap tk, tq;
  int rc = make_tmap_2d(&tk, cache, 1, static_cast<uint64_t>(n_pages) * kIdxPage, kIdxDim, kIdxDim, kIdxPage, 128);
  if (rc) return 1100 + rc;
  rc = make_tmap_2d(&tq, q8, 1, static_cast<uint64_t>(rows) * kIdxHeads, kIdxDim, kIdxDim, kIdxHeads, 128);
  if (rc) return 1200 + rc;
  constexpr int kSmem = 1024 + 24576 + 64 + 256 + 64;
  static DeviceOnce attr;
  if (ensure_smem(attr, dsa_score_kernel, kSmem) != cudaSuccess) return 3000;
  plow::launch_serial(dsa_score_kernel, dim3((max_len + 127) / 128, rows), dim3(128), kSmem, stream, scores, ld_scores, wq, cache_scale, pos, seq, page_table,
                                                                            max_pages, status, tk, tq);
  plow::launch_serial(dsa_topk_kernel, dim3(rows), dim3(1024), 0, stream, sel, scores, ld_scores, pos, top_k);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// Gather the selected cache rows of every query row into its compact cache: ckv [rows*top_k/64 pages][64][row_bytes],
// cscale f32 [pages][64], csmax f32 [pages][4] (zeroed here), clen int32 [rows] = min(pos+1, top_k).  top_k % 64 == 0.
int plow_dsa_gather(void* ckv, float* cscale, float* csmax, int* clen, const int* sel, int top_k, const void* cache,
                    const float* scale, const int* pos, const int* seq, const int* page_table, int max_pages, int rows,
                    int row_bytes, void* stream_) {
  using namespace plow;
  if (rows <= 0 || top_k <= 0 || top_k % kIdxPage || row_bytes % 16) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const size_t pages = static_cast<size_t>(rows) * (top_k / kIdxPage);
  cudaMemsetAsync(csmax, 0, pages * 4 * sizeof(float), stream);
  const long long items = static_cast<long long>(rows) * top_k;
  plow::launch_serial(dsa_gather_kernel, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), 0, stream, 
      static_cast<uint8_t*>(ckv), cscale, csmax, clen, sel, top_k, static_cast<const uint8_t*>(cache), scale, pos, seq,
      page_table, max_pages, rows, row_bytes);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
