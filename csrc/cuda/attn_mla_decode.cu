// Absorbed multi-head-latent-attention decode over a paged e4m3 latent cache, on tcgen05.
//
// Per token the cache holds one 576-byte row (512 latent + 64 rope dims, e4m3) and one f32
// scale.  For a request with query q[h] (already multiplied by W_uk, so it lives in latent
// space; quantised to e4m3 with one scale per (token, head)):
//     score[h][t] = softmax_scale * sq[h] * sk[t] * (q8[h] . kv8[t])
//     oacc[h]     = sum_t p[h][t] * sk[t] * kv8[t][0:512]          (latent-wide, W_uv is folded later)
// The 128 heads of a request are the 128 TMEM lanes of one CTA, so QK^T is a single UMMA
// M=128 x N=64 (one KV page) x K=576 and a row of the score matrix is private to one thread
// (lane = head): the online softmax needs no cross-thread reduction.  The accumulator for all
// 512 latent columns does not fit in TMEM next to S, so two CTAs ("halves") work on the same
// (request, split) and each accumulates 256 latent columns; both compute S.
//
// The same shared-memory KV tile feeds both products: as the K-major B operand of QK^T and as
// the MN-major B operand of P.V (tokens are the reduction dimension there).  P is written by
// the softmax threads to shared memory as e4m3 with the 64-byte swizzle the UMMA descriptor
// expects.  The per-token scale sk[t] is folded into P; to keep P in e4m3 range it is divided
// by a running maximum SK of the scales seen so far, which is handled exactly like the running
// row maximum of online softmax (the accumulator is rescaled in TMEM when either changes).
//
// Work is a device-built list of (request, half, split, first page, page count) items walked
// by a persistent grid; splits are merged by `plow_mla_merge`.  The reference's kernel for this
// op is a scalar-FMA split-KV kernel (runtime/nvidia/op_mla.cuh:23-58, d_flash_mla_decode and
// d_mla_merge_fold); it argues HBM-bound on a 64-head model — with 128 heads and an fp8 cache
// the op is tensor-core-bound, hence this design.
#include "ptx.cuh"
#include "tmap.cuh"

namespace plow {

constexpr int kMlaHeads = 128;
constexpr int kMlaLatent = 512;
constexpr int kMlaRope = 64;
constexpr int kMlaRow = 576;
constexpr int kMlaPage = 64;
constexpr int kMlaStages = 3;
constexpr int kQBytes = 4 * 128 * 128 + 128 * 64;            // 73728
constexpr int kKvTileBytes = 4 * 64 * 128 + 64 * 64;         // 36864
constexpr int kKvStageBytes = 37 * 1024;                     // tile + 256 B of scales, 1 KiB aligned
constexpr int kPBytes = 128 * 64;
constexpr int kMlaSmem = 1024 + kQBytes + kMlaStages * kKvStageBytes + 2 * kPBytes + 1024 + 4096;
constexpr int kMlaThreads = 320;   // TMA warp, MMA warp, 8 softmax warps (two threads per head)

struct MlaItem { int req, half, split, tile0, ntiles, pad0, pad1, pad2; };

struct MlaArgs {
  const float* sq;          // [heads][T] query scales
  const float* kv_scale;    // [n_pages][64]
  const int* page_table;    // [n_slots][max_pages]
  const int* slot_of;       // [T] slot of each query row
  const int* kvlen;         // [T] tokens visible to each query row (including itself)
  const MlaItem* items;
  const int* n_items;
  __nv_bfloat16* opart;     // [T][max_splits][heads][512]
  float* lse;               // [T][max_splits][heads]   (log2 domain)
  int* status;
  int T, max_pages, max_splits;
  float scale_log2e;        // softmax scale * log2(e)
};

// ---------------------------------------------------------------------------------------------
__global__ void mla_build_items(const int* kvlen, int T, int tiles_per_split, int max_splits,
                                MlaItem* items, int* n_items) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int n = 0;
  // longest splits first would balance better; requests are walked in order and splits are
  // uniform, so the persistent grid's round-robin already spreads long requests
  for (int r = 0; r < T; ++r) {
    const int tiles = (kvlen[r] + kMlaPage - 1) / kMlaPage;
    int split = 0;
    for (int t0 = 0; t0 < tiles && split < max_splits; t0 += tiles_per_split, ++split) {
      const int nt = (split == max_splits - 1) ? tiles - t0 : min(tiles_per_split, tiles - t0);
      for (int half = 0; half < 2; ++half) items[n++] = MlaItem{r, half, split, t0, nt, 0, 0, 0};
    }
  }
  *n_items = n;
}

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_kernel(const MlaArgs a, const __grid_constant__ CUtensorMap tm_q,
                  const __grid_constant__ CUtensorMap tm_qr, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_kvr) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + kQBytes;
  uint8_t* p_smem = kv_smem + kMlaStages * kKvStageBytes;
  uint8_t* ctrl = p_smem + 2 * kPBytes;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* q_empty = q_full + 1;
  uint64_t* kv_full = q_empty + 1;           // [3]
  uint64_t* kv_empty = kv_full + kMlaStages; // [3]
  uint64_t* s_full = kv_empty + kMlaStages;  // [2]
  uint64_t* s_empty = s_full + 2;            // [2]
  uint64_t* p_full = s_empty + 2;            // [2]
  uint64_t* pv_done = p_full + 2;            // [2] indexed by tile parity (see the softmax warps)
  uint64_t* o_free = pv_done + 2;            // [1]
  uint64_t* drain_bar = o_free + 1;          // [1]
  uint64_t* xchg_bar = drain_bar + 1;        // [2] softmax half-row exchange
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(xchg_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* never_flag = abort_flag + 1;
  float2* xchg = reinterpret_cast<float2*>(ctrl + 1024);   // [2 parity][2 half][128 rows] (max, sk max)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < kMlaStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 8); mbar_init(&p_full[b], 8); mbar_init(&xchg_bar[b], 8); }
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    mbar_init(o_free, 8);
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    *never_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_qr); tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_kvr);
  }
  if (warp == 1) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_s = tmem_base;          // S buffers: columns [0,64) and [64,128)
  const uint32_t tm_o = tmem_base + 128;    // O: 256 columns
  const int n_items = *a.n_items;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t item_it = 0, kv_it = 0;
      bool ok = true;
      for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x, ++item_it) {
        const MlaItem w = a.items[it];
        if (!mbar_wait(q_empty, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT); break; }
        mbar_expect_tx(q_full, kQBytes);
        for (int c = 0; c < 4; ++c) tma_load_3d(q_smem + c * 16384, &tm_q, c * 128, w.req, 0, q_full);
        tma_load_3d(q_smem + 65536, &tm_qr, 512, w.req, 0, q_full);
        const int* pt = a.page_table + static_cast<size_t>(a.slot_of[w.req]) * a.max_pages;
        int page_next = pt[w.tile0];
        for (int i = 0; i < w.ntiles; ++i, ++kv_it) {
          const int s = kv_it % kMlaStages;
          // the page id of the next tile is fetched before waiting for this tile's stage, so the
          // table lookup never sits between a freed stage and its refill
          const int page = page_next;
          if (i + 1 < w.ntiles) page_next = pt[w.tile0 + i + 1];
          if (!mbar_wait(&kv_empty[s], ((kv_it / kMlaStages) & 1) ^ 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT); ok = false; break;
          }
          uint8_t* st = kv_smem + s * kKvStageBytes;
          mbar_expect_tx(&kv_full[s], kKvTileBytes + 256);
          for (int c = 0; c < 4; ++c) tma_load_2d(st + c * 8192, &tm_kv, c * 128, page * kMlaPage, &kv_full[s]);
          tma_load_2d(st + 32768, &tm_kvr, 512, page * kMlaPage, &kv_full[s]);
          bulk_load_1d(st + kKvTileBytes, a.kv_scale + static_cast<size_t>(page) * kMlaPage, 256, &kv_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_qk = umma_idesc(128, 64, 0, 0);
      const uint32_t idesc_pv = umma_idesc(128, 256, 0, 0, 0, 1);
      uint32_t item_it = 0, kv_it = 0, tile_it = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t kvi, uint32_t ti) -> bool {
        const int s = kvi % kMlaStages;
        if (!mbar_wait(&kv_full[s], (kvi / kMlaStages) & 1, abort_flag)) { atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT); return false; }
        if (!mbar_wait(&s_empty[ti & 1], ((ti >> 1) & 1) ^ 1, abort_flag)) { atomicCAS(a.status, 0, PLOW_ERR_TMEM_FREE_WAIT); return false; }
        tc_fence_after();
        const uint32_t d = tm_s + (ti & 1) * 64;
        const uint32_t qa = smem_u32(q_smem), ka = smem_u32(kv_smem + s * kKvStageBytes);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint64_t qd = umma_desc_k128(qa + c * 16384), kd = umma_desc_k128(ka + c * 8192);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f8(d, qd + 2 * k, kd + 2 * k, idesc_qk, (c | k) != 0);
        }
        const uint64_t qd = umma_desc_k64(qa + 65536), kd = umma_desc_k64(ka + 32768);
        tc_mma_f8(d, qd, kd, idesc_qk, 1);
        tc_mma_f8(d, qd + 2, kd + 2, idesc_qk, 1);
        tc_commit(&s_full[ti & 1]);
        return true;
      };
      for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x, ++item_it) {
        const MlaItem w = a.items[it];
        if (!mbar_wait(q_full, item_it & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT); break; }
        if (!issue_qk(kv_it, tile_it)) { *abort_flag = 1; break; }
        for (int i = 0; i < w.ntiles; ++i) {
          if (i + 1 < w.ntiles) {
            if (!issue_qk(kv_it + i + 1, tile_it + i + 1)) { *abort_flag = 1; ok = false; break; }
          } else {
            tc_commit(q_empty);   // every QK^T of this item is issued: Q may be overwritten once they retire
          }
          const uint32_t ti = tile_it + i;
          if (i == 0 && !mbar_wait(o_free, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_FREE_WAIT); ok = false; break; }
          if (!mbar_wait(&p_full[ti & 1], (ti >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT); ok = false; break; }
          tc_fence_after();
          const int s = (kv_it + i) % kMlaStages;
          const uint32_t pa = smem_u32(p_smem + (ti & 1) * kPBytes);
          const uint32_t va = smem_u32(kv_smem + s * kKvStageBytes) + w.half * 2 * 8192;
          tc_mma_f8(tm_o, umma_desc_k64(pa), umma_desc_mn128(va, 8192, 1024), idesc_pv, i > 0);
          tc_mma_f8(tm_o, umma_desc_k64(pa) + 2, umma_desc_mn128(va + 4096, 8192, 1024), idesc_pv, 1);
          tc_commit(&kv_empty[s]);
          tc_commit(&pv_done[ti & 1]);
        }
        kv_it += w.ntiles;
        tile_it += w.ntiles;
      }
      if (!ok || *abort_flag) { tc_commit(drain_bar); mbar_wait(drain_bar, 0, never_flag); }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue warps
    // Eight warps: warps w and w+4 share a TMEM lane quarter; thread (row, ch) owns columns
    // [32 ch, 32 ch + 32) of the row's 64 scores and 128 of the CTA's 256 accumulator columns.
    const int lq = warp & 3;
    const int ch = (warp - 2) >> 2;  // column half
    const int li = lq * 32 + lane;   // head
    const uint32_t lane_addr = static_cast<uint32_t>(lq * 32) << 16;
    uint32_t item_it = 0, kv_it = 0, tile_it = 0, xit = 0;
    bool ok = true;
    // exchange one float2 with the partner thread of the row (bounded)
    auto exchange = [&](float a0, float a1, float& b0, float& b1) -> bool {
      float2* buf = xchg + (xit & 1) * 256;
      buf[ch * 128 + li] = make_float2(a0, a1);
      __syncwarp();
      if (lane == 0) mbar_arrive(&xchg_bar[xit & 1]);
      if (!mbar_wait(&xchg_bar[xit & 1], (xit >> 1) & 1, abort_flag)) return false;
      const float2 o = buf[(ch ^ 1) * 128 + li];
      b0 = o.x; b1 = o.y;
      ++xit;
      return true;
    };
    for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x, ++item_it) {
      const MlaItem w = a.items[it];
      const int kv_len = a.kvlen[w.req];
      const float qs = a.sq[static_cast<size_t>(li) * a.T + w.req] * a.scale_log2e;
      float m = 0.f, l = 0.f, SK = 1.f;
      for (int i = 0; i < w.ntiles; ++i) {
        const uint32_t ti = tile_it + i;
        if (!mbar_wait(&s_full[ti & 1], (ti >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT); ok = false; break; }
        tc_fence_after();
        uint32_t sv[32];
        tmem_ld32(tm_s + lane_addr + (ti & 1) * 64 + ch * 32, sv);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[ti & 1]);
        const int s = (kv_it + i) % kMlaStages;
        // the per-token scales arrived with the tile: observe the stage barrier directly so the
        // bulk copy's writes are ordered before the reads below
        if (!mbar_wait(&kv_full[s], ((kv_it + i) / kMlaStages) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT); ok = false; break; }
        const float4* sk4 = reinterpret_cast<const float4*>(kv_smem + s * kKvStageBytes + kKvTileBytes) + ch * 8;
        const int valid = min(kMlaPage, kv_len - (w.tile0 + i) * kMlaPage) - ch * 32;   // valid columns of this half
        float x[32], skv[32];
        float mx = -INFINITY, skmax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 k4 = sk4[j];
          skv[4 * j] = k4.x; skv[4 * j + 1] = k4.y; skv[4 * j + 2] = k4.z; skv[4 * j + 3] = k4.w;
        }
        if (valid >= 32) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            x[j] = __uint_as_float(sv[j]) * (qs * skv[j]);
            mx = fmaxf(mx, x[j]);
            skmax = fmaxf(skmax, skv[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool in = j < valid;
            x[j] = in ? __uint_as_float(sv[j]) * (qs * skv[j]) : -INFINITY;
            mx = fmaxf(mx, x[j]);
            skmax = in ? fmaxf(skmax, skv[j]) : skmax;
          }
        }
        float omx, osk;
        if (!exchange(mx, skmax, omx, osk)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT); ok = false; break; }
        mx = fmaxf(mx, omx);
        skmax = fmaxf(skmax, osk);
        // Lazy rescaling: the running maximum m is only raised when a tile exceeds it by more
        // than kTau (log2 units), so p = 2^(x - m) stays below 2^kTau, well inside e4m3 range,
        // and the accumulator in TMEM is almost never touched.  The running scale bound SK is
        // raised with 2x head-room for the same reason.  Any (m, SK) is valid as long as O and
        // l are kept consistent with it; both threads of a row see the same (mx, skmax) and
        // therefore take the same decision.
        constexpr float kTau = 7.0f;
        if (i == 0) {
          m = mx;
          SK = skmax * 2.0f;
        } else {
          const bool up_m = mx > m + kTau;
          const bool up_sk = skmax > SK;
          if (__any_sync(0xffffffffu, up_m || up_sk)) {
            const float m_new = up_m ? mx : m;
            const float SK_new = up_sk ? skmax * 2.0f : SK;
            const float alpha_l = exp2f(m - m_new);
            const float alpha_o = alpha_l * (SK / SK_new);
            l *= alpha_l;
            m = m_new;
            SK = SK_new;
            // accumulator must be quiescent: P.V of the previous tile has retired.  QK^T of this
            // tile was issued after P.V of tile ti-2, so at most tile ti-1 is pending on its
            // parity's barrier and the phase below cannot alias.
            if (!mbar_wait(&pv_done[(ti - 1) & 1], ((ti - 1) >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT); ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
              uint32_t o[32];
              tmem_ld32(tm_o + lane_addr + ch * 128 + c, o);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha_o);
              tmem_st16(tm_o + lane_addr + ch * 128 + c, o);
              tmem_st16(tm_o + lane_addr + ch * 128 + c + 16, o + 16);
            }
            tmem_st_wait();
            tc_fence_before();
          }
        }
        const float inv_sk = 1.0f / SK;
        float sum = 0.f;
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float p[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float e;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x[j + u] - m));
            sum += e;
            p[u] = e * (skv[j + u] * inv_sk);
          }
          __nv_fp8x4_e4m3 q4(make_float4(p[0], p[1], p[2], p[3]));
          pk[j >> 2] = *reinterpret_cast<uint32_t*>(&q4);
        }
        l += sum;
        // P row (64 bytes) with the 64-byte swizzle: 16-byte unit c lands at c ^ ((row >> 1) & 3);
        // this thread owns units 2 ch and 2 ch + 1
        uint8_t* prow = p_smem + (ti & 1) * kPBytes + li * 64;
        const int sw = (li >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 2; ++c)
          *reinterpret_cast<uint4*>(prow + (((2 * ch + c) ^ sw) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[ti & 1]);
      }
      if (!ok) break;
      // ---- finalize this item: O * SK / l, log-sum-exp in the log2 domain
      float ol, unused;
      if (!exchange(l, 0.f, ol, unused)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT); break; }
      l += ol;
      const uint32_t ti_last = tile_it + w.ntiles - 1;
      if (!mbar_wait(&pv_done[ti_last & 1], (ti_last >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT); break; }
      tc_fence_after();
      const float fin = l > 0.f ? SK / l : 0.f;
      const size_t obase = ((static_cast<size_t>(w.req) * a.max_splits + w.split) * kMlaHeads + li) * kMlaLatent + w.half * 256 + ch * 128;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t o[32];
        tmem_ld32(tm_o + lane_addr + ch * 128 + c, o);
        tmem_ld_wait();
        uint32_t h2[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * fin, __uint_as_float(o[2 * j + 1]) * fin);
          h2[j] = *reinterpret_cast<uint32_t*>(&v);
        }
        uint4* dst = reinterpret_cast<uint4*>(a.opart + obase + c);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(h2[4 * q], h2[4 * q + 1], h2[4 * q + 2], h2[4 * q + 3]);
      }
      if (w.half == 0 && ch == 0) a.lse[(static_cast<size_t>(w.req) * a.max_splits + w.split) * kMlaHeads + li] = m + log2f(fmaxf(l, 1e-30f));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
      kv_it += w.ntiles;
      tile_it += w.ntiles;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {}
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// Merge the splits of each (request, head): out[h][t][:] = sum_s 2^(lse_s - LSE) * opart_s.
__global__ void mla_merge_kernel(const __nv_bfloat16* opart, const float* lse, const int* kvlen, int T,
                                 int max_splits, int tiles_per_split, __nv_bfloat16* out /*[heads][T][512]*/) {
  const int t = blockIdx.x, h = blockIdx.y;
  const int tiles = (kvlen[t] + kMlaPage - 1) / kMlaPage;
  int ns = (tiles + tiles_per_split - 1) / tiles_per_split;
  ns = ns < 1 ? 1 : (ns > max_splits ? max_splits : ns);
  float mx = -INFINITY;
  for (int s = 0; s < ns; ++s) mx = fmaxf(mx, lse[(static_cast<size_t>(t) * max_splits + s) * kMlaHeads + h]);
  float wsum = 0.f;
  for (int s = 0; s < ns; ++s) wsum += exp2f(lse[(static_cast<size_t>(t) * max_splits + s) * kMlaHeads + h] - mx);
  for (int c = threadIdx.x * 2; c < kMlaLatent; c += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int s = 0; s < ns; ++s) {
      const size_t base = (static_cast<size_t>(t) * max_splits + s) * kMlaHeads + h;
      const float wgt = exp2f(lse[base] - mx) / wsum;
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(opart + base * kMlaLatent + c);
      a0 += wgt * __bfloat162float(v.x);
      a1 += wgt * __bfloat162float(v.y);
    }
    *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<size_t>(h) * T + t) * kMlaLatent + c) = __floats2bfloat162_rn(a0, a1);
  }
}

}  // namespace plow

extern "C" {

// Scratch the caller provides: items (8 ints per item, capacity 2*T*max_splits), n_items (1 int),
// opart bf16 [T][max_splits][128][512], lse f32 [T][max_splits][128].
// q8 e4m3 [128 heads][T][576]; sq f32 [128][T]; kv e4m3 [n_pages][64][576]; kv_scale f32 [n_pages][64];
// out bf16 [128][T][512].
int plow_mla_decode(const void* q8, const float* sq, const void* kv, const float* kv_scale, int64_t n_pages,
                    const int* page_table, int max_pages, const int* slot_of, const int* kvlen, int T,
                    int tiles_per_split, int max_splits, void* items, int* n_items, void* opart, float* lse,
                    void* out, float softmax_scale, int* status, void* stream_) {
  using namespace plow;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || max_splits <= 0 || tiles_per_split <= 0) return -1;
  CUtensorMap tq, tqr, tkv, tkvr;
  int r = make_tmap_3d(&tq, q8, 1, kMlaRow, T, kMlaHeads, kMlaRow, static_cast<uint64_t>(T) * kMlaRow, 1, 128, 128);
  if (r) return 1000 + r;
  r = make_tmap_3d(&tqr, q8, 1, kMlaRow, T, kMlaHeads, kMlaRow, static_cast<uint64_t>(T) * kMlaRow, 1, 128, 64);
  if (r) return 1100 + r;
  r = make_tmap_2d(&tkv, kv, 1, static_cast<uint64_t>(n_pages) * kMlaPage, kMlaRow, kMlaRow, kMlaPage, 128);
  if (r) return 1200 + r;
  r = make_tmap_2d(&tkvr, kv, 1, static_cast<uint64_t>(n_pages) * kMlaPage, kMlaRow, kMlaRow, kMlaPage, 64);
  if (r) return 1300 + r;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem) != cudaSuccess) return 3000;
    attr = true;
  }
  mla_build_items<<<1, 32, 0, stream>>>(kvlen, T, tiles_per_split, max_splits, static_cast<MlaItem*>(items), n_items);
  MlaArgs a;
  a.sq = sq; a.kv_scale = kv_scale; a.page_table = page_table; a.slot_of = slot_of; a.kvlen = kvlen;
  a.items = static_cast<const MlaItem*>(items); a.n_items = n_items;
  a.opart = static_cast<__nv_bfloat16*>(opart); a.lse = lse; a.status = status;
  a.T = T; a.max_pages = max_pages; a.max_splits = max_splits;
  a.scale_log2e = softmax_scale * 1.4426950408889634f;
  int grid = sm_count();
  const int cap = 2 * T * max_splits;
  if (cap < grid) grid = cap;
  mla_decode_kernel<<<grid, kMlaThreads, kMlaSmem, stream>>>(a, tq, tqr, tkv, tkvr);
  mla_merge_kernel<<<dim3(T, kMlaHeads), 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(opart), lse, kvlen, T,
                                                          max_splits, tiles_per_split, static_cast<__nv_bfloat16*>(out));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
