// Per-head MLA projections around the absorbed decode kernel, each a single tcgen05 tile per CTA.
//
//   mla_absorb:  q[T][heads*(128+64)] (bf16)  ->  q8[heads][T][576] (e4m3) + sq[heads][T]
//                q_abs[h] = q_nope[h] . W_uk[h]   (M = 128 tokens, N = 512 latent, K = 128; the 512
//                fp32 columns fill TMEM exactly), RoPE on the 64 rope dims, one e4m3 scale per
//                (token, head) over all 576 values.  Replaces three launches (split/transpose +
//                rope, grouped GEMM, quantise) and two HBM round trips of the bf16 intermediates.
//   mla_fold:    opart[T][splits][heads][512] + lse -> ao[T][heads*128] (bf16) and its e4m3 twin
//                merges the split-KV partials (weights 2^(lse_s - max)) while writing the A operand
//                into swizzled shared memory, multiplies by W_uv[h] (N = 128, K = 512 in two
//                phases), writes token-major output and quantises it for the o_proj GEMM (the
//                1x128 quant group is exactly one head's 128 values, i.e. thread-local).
//
// Reference counterparts: the q_abs / MLA_MERGE_FOLD steps of the decode op sequence
// (crates/devgen/src/mla.rs:6252-6323, runtime/nvidia/op_mla.cuh d_mla_merge_fold).
#include "ptx.cuh"
#include "tmap.cuh"

namespace plow {

constexpr int kProjThreads = 160;
constexpr int kFoldSplits = 16;   // KV splits per request the fold kernel merges at most   // warp 0: TMA + MMA issue, warps 1-4: one TMEM lane quarter each

struct AbsorbArgs {
  const __nv_bfloat16* q;    // [T][q_pitch]
  const float* rope_tab;     // [max_pos][64] (cos 32 | sin 32)
  const int* pos;            // [T]
  uint8_t* q8;               // [heads][T][576]
  float* sq;                 // [heads][T]
  int* status;
  int T, heads, q_pitch, pair_mode;
};

__global__ void __launch_bounds__(kProjThreads, 1)
mla_absorb_kernel(const AbsorbArgs a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sa = smem;                    // 2 chunks x [128 x 128 B]
  uint8_t* sb = smem + 32768;            // [nh][kc] x [256 x 128 B]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + 32768 + 131072);
  uint64_t* done = full + 1;
  uint32_t* holder = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, t0 = blockIdx.y * 128;
  pdl_launch_dependents();
  if (threadIdx.x == 0) { mbar_init(full, 1); mbar_init(done, 1); *abort_flag = 0; fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *holder;
  if (warp == 0) {
    if (elect_one()) {
      // the head's W_uk (a weight) is requested before the dependency wait, the queries after it
      mbar_expect_tx(full, 32768 + 131072);
      for (int nh = 0; nh < 2; ++nh)
        for (int kc = 0; kc < 2; ++kc) tma_load_2d(sb + (nh * 2 + kc) * 32768, &tm_w, kc * 64, h * 512 + nh * 256, full);
      pdl_wait();
      for (int kc = 0; kc < 2; ++kc) tma_load_2d(sa + kc * 16384, &tm_q, h * 192 + kc * 64, t0, full);
      if (mbar_wait(full, 0, abort_flag)) {
        tc_fence_after();
        const uint32_t idesc = umma_idesc(128, 256, 1, 1);
        for (int nh = 0; nh < 2; ++nh)
          for (int kc = 0; kc < 2; ++kc) {
            const uint64_t ad = umma_desc_k128(smem_u32(sa + kc * 16384));
            const uint64_t bd = umma_desc_k128(smem_u32(sb + (nh * 2 + kc) * 32768));
            for (int k = 0; k < 4; ++k) tc_mma_f16(tm + nh * 256, ad + 2 * k, bd + 2 * k, idesc, (kc | k) != 0);
          }
        tc_commit(done);
      } else {
        *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagMlaProj);
      }
    }
  } else {
    const int lq = warp & 3;
    const int li = lq * 32 + lane;
    const int t = t0 + li;
    const uint32_t lane_addr = static_cast<uint32_t>(lq * 32) << 16;
    // RoPE of this token's 64 rope dims while the MMA runs
    pdl_wait();
    float rp[64];
    const bool live = t < a.T;
    {
      const __nv_bfloat16* src = a.q + static_cast<size_t>(live ? t : 0) * a.q_pitch + h * 192 + 128;
      const float* tab = a.rope_tab + static_cast<size_t>(live ? a.pos[t] : 0) * 64;
      float x[64];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = reinterpret_cast<const uint4*>(src)[j];
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(hh[u]); x[8 * j + 2 * u] = f.x; x[8 * j + 2 * u + 1] = f.y; }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float c = tab[i], s = tab[32 + i];
        if (a.pair_mode) {
          rp[2 * i] = __bfloat162float(__float2bfloat16(x[2 * i] * c - x[2 * i + 1] * s));
          rp[2 * i + 1] = __bfloat162float(__float2bfloat16(x[2 * i + 1] * c + x[2 * i] * s));
        } else {
          rp[i] = __bfloat162float(__float2bfloat16(x[i] * c - x[i + 32] * s));
          rp[i + 32] = __bfloat162float(__float2bfloat16(x[i + 32] * c + x[i] * s));
        }
      }
    }
    if (mbar_wait(done, 0, abort_flag)) {
      tc_fence_after();
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 64; ++j) amax = fmaxf(amax, fabsf(rp[j]));
#pragma unroll 1
      for (int c = 0; c < 512; c += 32) {
        uint32_t v[32];
        tmem_ld32(tm + lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(__uint_as_float(v[j])));
      }
      const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
      const float inv = 1.0f / sc;
      uint8_t* dst = a.q8 + (static_cast<size_t>(h) * a.T + (live ? t : 0)) * 576;
#pragma unroll 1
      for (int c = 0; c < 512; c += 32) {
        uint32_t v[32];
        tmem_ld32(tm + lane_addr + c, v);
        tmem_ld_wait();
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_fp8x4_e4m3 q4(make_float4(__uint_as_float(v[4 * j]) * inv, __uint_as_float(v[4 * j + 1]) * inv,
                                         __uint_as_float(v[4 * j + 2]) * inv, __uint_as_float(v[4 * j + 3]) * inv));
          pk[j] = *reinterpret_cast<uint32_t*>(&q4);
        }
        if (live) {
          reinterpret_cast<uint4*>(dst + c)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          reinterpret_cast<uint4*>(dst + c)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
      uint32_t pr[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        __nv_fp8x4_e4m3 q4(make_float4(rp[4 * j] * inv, rp[4 * j + 1] * inv, rp[4 * j + 2] * inv, rp[4 * j + 3] * inv));
        pr[j] = *reinterpret_cast<uint32_t*>(&q4);
      }
      if (live) {
#pragma unroll
        for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst + 512)[j] = make_uint4(pr[4 * j], pr[4 * j + 1], pr[4 * j + 2], pr[4 * j + 3]);
        a.sq[static_cast<size_t>(h) * a.T + t] = sc;
      }
    } else {
      *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaProj);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

// ---------------------------------------------------------------------------------------------
struct FoldArgs {
  const __nv_bfloat16* opart;  // [T][max_splits][heads][512]
  const float* lse;            // [T][max_splits][heads]
  const int* kvlen;            // [T]
  __nv_bfloat16* ao;           // [T][heads*128]
  uint8_t* aq;                 // optional e4m3 twin [T][heads*128]
  float* saq;                  // its scales, transposed [heads][ld_saq]
  int* status;
  int T, heads, max_splits, tiles_per_split, ld_saq;
};

__global__ void __launch_bounds__(kProjThreads, 1)
mla_fold_kernel(const FoldArgs a, const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sa = smem;              // 4 chunks x [128 tokens x 128 B], written by the merge threads
  uint8_t* sb = smem + 65536;      // 4 chunks x [128 v-dims x 128 B]
  uint64_t* b_full = reinterpret_cast<uint64_t*>(smem + 131072);
  uint64_t* a_ready = b_full + 1;
  uint64_t* done = a_ready + 1;    // [2]
  uint32_t* holder = reinterpret_cast<uint32_t*>(done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, t0 = blockIdx.y * 128;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    mbar_init(b_full, 1); mbar_init(a_ready, 4); mbar_init(&done[0], 1); mbar_init(&done[1], 1);
    *abort_flag = 0; fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(holder, 128); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *holder;
  if (warp == 0) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc(128, 128, 1, 1);
      for (int p = 0; p < 2; ++p) {
        if (p == 1 && !mbar_wait(&done[0], 0, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaProj); break; }
        mbar_expect_tx(b_full, 65536);
        for (int c = 0; c < 4; ++c) tma_load_2d(sb + c * 16384, &tm_w, p * 256 + c * 64, h * 128, b_full);
        if (!mbar_wait(b_full, p, abort_flag) || !mbar_wait(a_ready, p, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagMlaProj); break;
        }
        tc_fence_after();
        for (int c = 0; c < 4; ++c) {
          const uint64_t ad = umma_desc_k128(smem_u32(sa + c * 16384)), bd = umma_desc_k128(smem_u32(sb + c * 16384));
          for (int k = 0; k < 4; ++k) tc_mma_f16(tm, ad + 2 * k, bd + 2 * k, idesc, (p | c | k) != 0);
        }
        tc_commit(&done[p]);
      }
    }
  } else {
    const int lq = warp & 3;
    const int li = lq * 32 + lane;
    const int t = t0 + li;
    const bool live = t < a.T;
    const uint32_t lane_addr = static_cast<uint32_t>(lq * 32) << 16;
    pdl_wait();      // partials and log-sum-exps come from the attention kernel (warp 0 only touches W_uv, a weight)
    // merge weights of this (token, head), shared with the other merge warps through shared memory
    float* wsm = reinterpret_cast<float*>(smem + 131072 + 256);       // [128 rows][kFoldSplits]
    int* nsm = reinterpret_cast<int*>(wsm + 128 * kFoldSplits);       // [128 rows]
    {
      float wgt[kFoldSplits];
#pragma unroll
      for (int s = 0; s < kFoldSplits; ++s) wgt[s] = 0.f;
      int ns = 0;
      if (live) {
        const int tiles = (a.kvlen[t] + 63) / 64;
        int per_unused;
        ns = kv_splits(tiles, a.tiles_per_split, a.max_splits, &per_unused);
        if (ns > kFoldSplits) ns = kFoldSplits;
        float ls[kFoldSplits];
#pragma unroll
        for (int s = 0; s < kFoldSplits; ++s) ls[s] = s < ns ? a.lse[(static_cast<size_t>(t) * a.max_splits + s) * a.heads + h] : -INFINITY;
        float mx = -INFINITY;
#pragma unroll
        for (int s = 0; s < kFoldSplits; ++s) mx = fmaxf(mx, ls[s]);
        float sum = 0.f;
#pragma unroll
        for (int s = 0; s < kFoldSplits; ++s) { wgt[s] = s < ns ? exp2f(ls[s] - mx) : 0.f; sum += wgt[s]; }
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
#pragma unroll
        for (int s = 0; s < kFoldSplits; ++s) wgt[s] *= inv;
      }
#pragma unroll
      for (int s = 0; s < kFoldSplits; ++s) wsm[li * kFoldSplits + s] = wgt[s];
      nsm[li] = ns;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int n_live = min(128, a.T - t0);
    bool ok = true;
    for (int p = 0; p < 2 && ok; ++p) {
      if (p == 1 && !mbar_wait(&done[0], 0, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaProj); ok = false; break; }
      // A operand: warp w fills rows w, w+4, w+8, ... (so the live rows are spread over all four warps), eight
      // rows at a time.  For one row the 32 lanes fetch the row's 256 latent columns of this phase as one
      // coalesced 512-byte read per split (lane = 16-byte unit); the eight rows' loads of a split are issued
      // together, so a batch costs one memory round trip per split.  The merged unit goes to its swizzled
      // place: unit u of chunk c at (u ^ (row & 7)) * 16.
      for (int kb = 0; kb < 32; kb += 8) {
        if (lq + 4 * kb >= n_live) break;          // rows ascend: nothing live further on (warp-uniform)
        float acc[8][8];
        int nsr[8];
        int ns_b = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = lq + 4 * (kb + i);
          nsr[i] = row < n_live ? nsm[row] : 0;
          ns_b = max(ns_b, nsr[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
        }
        for (int sp = 0; sp < ns_b; ++sp) {
          uint4 v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = lq + 4 * (kb + i);
            v[i] = make_uint4(0u, 0u, 0u, 0u);
            if (sp < nsr[i])
              v[i] = *reinterpret_cast<const uint4*>(a.opart + ((static_cast<size_t>(t0 + row) * a.max_splits + sp) * a.heads + h) * 512 + p * 256 + lane * 8);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = lq + 4 * (kb + i);
            const float wv = wsm[(row & 127) * kFoldSplits + sp];
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(hh[j]); acc[i][2 * j] += wv * f.x; acc[i][2 * j + 1] += wv * f.y; }
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = lq + 4 * (kb + i);
          uint4 o;
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[i][2 * j], acc[i][2 * j + 1]);
          const int c = lane >> 3, uu = lane & 7;
          *reinterpret_cast<uint4*>(sa + c * 16384 + row * 128 + ((uu ^ (row & 7)) << 4)) = o;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready);
    }
    if (ok && mbar_wait(&done[1], 0, abort_flag)) {
      tc_fence_after();
      float r[128];
      float amax = 0.f;
#pragma unroll
      for (int c = 0; c < 128; c += 32) {
        uint32_t v[32];
        tmem_ld32(tm + lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { r[c + j] = __bfloat162float(__float2bfloat16(__uint_as_float(v[j]))); amax = fmaxf(amax, fabsf(r[c + j])); }
      }
      if (live) {
        __nv_bfloat16* dst = a.ao + static_cast<size_t>(t) * a.heads * 128 + h * 128;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          uint4 o;
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int u = 0; u < 4; ++u) oh[u] = __floats2bfloat162_rn(r[8 * j + 2 * u], r[8 * j + 2 * u + 1]);
          reinterpret_cast<uint4*>(dst)[j] = o;
        }
        if (a.aq) {
          const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
          const float inv = 1.0f / sc;
          uint8_t* dq = a.aq + static_cast<size_t>(t) * a.heads * 128 + h * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t pk[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              __nv_fp8x4_e4m3 q4(make_float4(r[16 * j + 4 * u] * inv, r[16 * j + 4 * u + 1] * inv, r[16 * j + 4 * u + 2] * inv, r[16 * j + 4 * u + 3] * inv));
              pk[u] = *reinterpret_cast<uint32_t*>(&q4);
            }
            reinterpret_cast<uint4*>(dq)[j] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
          a.saq[static_cast<size_t>(h) * a.ld_saq + t] = sc;
        }
      }
    } else if (ok) {
      *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaProj);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tm, 128); }
}

}  // namespace plow

extern "C" {

// q bf16 [T][q_pitch] (heads x (128 nope + 64 rope)); wuk_t bf16 [heads*512][128]; out q8 [heads][T][576], sq [heads][T]
int plow_mla_absorb(const void* q, int q_pitch, const void* wuk_t, const float* rope_tab, const int* pos, void* q8, float* sq,
                    int T, int heads, int pair_mode, int* status, void* stream_) {
  using namespace plow;
  CUtensorMap tq, tw;
  int r = make_tmap_2d(&tq, q, 2, T, static_cast<uint64_t>(heads) * 192, static_cast<uint64_t>(q_pitch) * 2, 128);
  if (r) return 1000 + r;
  r = make_tmap_2d(&tw, wuk_t, 2, static_cast<uint64_t>(heads) * 512, 128, 256, 256);
  if (r) return 1100 + r;
  const int smem = 1024 + 32768 + 131072 + 256;
  static DeviceOnce attr;
  if (ensure_smem(attr, mla_absorb_kernel, smem) != cudaSuccess) return 3000;
  AbsorbArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q); a.rope_tab = rope_tab; a.pos = pos; a.q8 = static_cast<uint8_t*>(q8); a.sq = sq;
  a.status = status; a.T = T; a.heads = heads; a.q_pitch = q_pitch; a.pair_mode = pair_mode;
  cudaError_t e = launch_serial(mla_absorb_kernel, dim3(heads, (T + 127) / 128), dim3(kProjThreads), smem,
                             reinterpret_cast<cudaStream_t>(stream_), a, tq, tw);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// opart/lse from plow_mla_decode's workspace; wuv bf16 [heads*128][512]; ao bf16 [T][heads*128]; aq/saq optional e4m3 twin
int plow_mla_fold(const void* opart, const float* lse, const int* kvlen, const void* wuv, void* ao, void* aq, float* saq, int ld_saq,
                  int T, int heads, int max_splits, int tiles_per_split, int* status, void* stream_) {
  using namespace plow;
  if (max_splits > kFoldSplits) return -1;
  CUtensorMap tw;
  int r = make_tmap_2d(&tw, wuv, 2, static_cast<uint64_t>(heads) * 128, 512, 1024, 128);
  if (r) return 1000 + r;
  const int smem = 1024 + 131072 + 256 + 128 * kFoldSplits * 4 + 128 * 4;
  static DeviceOnce attr;
  if (ensure_smem(attr, mla_fold_kernel, smem) != cudaSuccess) return 3000;
  FoldArgs a;
  a.opart = static_cast<const __nv_bfloat16*>(opart); a.lse = lse; a.kvlen = kvlen; a.ao = static_cast<__nv_bfloat16*>(ao);
  a.aq = static_cast<uint8_t*>(aq); a.saq = saq; a.status = status; a.T = T; a.heads = heads; a.max_splits = max_splits;
  a.tiles_per_split = tiles_per_split; a.ld_saq = ld_saq;
  cudaError_t e = launch_serial(mla_fold_kernel, dim3(heads, (T + 127) / 128), dim3(kProjThreads), smem,
                             reinterpret_cast<cudaStream_t>(stream_), a, tw);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
