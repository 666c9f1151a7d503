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
// the MN-major B operand of P.V (tokens are the reduction dimension there).  The A operands
// live in TMEM: the latent part of Q (128 columns, stored once per item by the softmax threads)
// and P, which the softmax threads write as e4m3 over the first 16 columns of the S buffer it
// was computed from.  Only Q's 64 rope bytes per head stay in shared memory, which leaves room
// for five KV stages: a stage is pinned from its TMA issue until the P.V that reads it retires,
// i.e. for the whole QK^T -> softmax -> P.V latency chain, so depth is what hides that chain.  The per-token scale sk[t] is folded into P; to keep P in e4m3 range it is divided
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
constexpr int kMlaStages = 5;
constexpr int kQBytes = 128 * 64;                            // rope part of Q only (64-byte swizzle)
constexpr int kKvTileBytes = 4 * 64 * 128 + 64 * 64;         // 36864
constexpr int kKvStageBytes = 37 * 1024;                     // tile + 256 B of scales, 1 KiB aligned
constexpr int kMlaSmem = 1024 + kQBytes + kMlaStages * kKvStageBytes + 1024 + 4096;
constexpr int kMlaThreads = 320;   // TMA warp, MMA warp, 8 softmax warps (two threads per head)

struct MlaItem { int req, half, split, tile0, ntiles, pad0, pad1, pad2; };

struct MlaArgs {
  const uint8_t* q8;        // [heads][T][576] e4m3 queries
  const float* sq;          // [heads][T] query scales
  const float* kv_scale;    // [n_pages][64]
  const float* kv_smax;     // [n_pages][4]: [0] = upper bound of the page's 64 scales
  const int* page_table;    // [n_slots][max_pages]
  const int* slot_of;       // [T] slot of each query row
  const int* kvlen;         // [T] tokens visible to each query row (including itself)
  const MlaItem* items;
  const int* n_items;
  int* claim;               // work counter of this launch: CTAs take items from it one at a time (zeroed by the build kernel)
  __nv_bfloat16* opart;     // [T][max_splits][heads][512]
  float* lse;               // [T][max_splits][heads]   (log2 domain)
  int* status;
  long long* trace;         // phase timestamps of CTA 0; only read by builds with -DPLOW_DEVICE_TRACE
  int T, max_pages, max_splits;
  float scale_log2e;        // softmax scale * log2(e)
};

// ---------------------------------------------------------------------------------------------
constexpr int kMlaClaimSlots = 256;   // one work counter per launch between two builds of the list (layers of a step)

__global__ void mla_build_items(const int* kvlen, int T, int tiles_per_split, int max_splits,
                                MlaItem* items, int* n_items, int* claims) {
  // one thread per request: split count and tiles per split, then its offset in the list.  Up to 256 requests the
  // list is ordered by decreasing tiles per item (longest first), which together with the dynamic hand-out in the
  // attention kernel keeps the last CTAs from finishing long after the rest; larger batches keep request order.
  extern __shared__ int cnt[];     // [T] splits, then [T] tiles per split
  int* pers = cnt + T;
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < kMlaClaimSlots; i += blockDim.x) claims[i] = 0;
  for (int r = threadIdx.x; r < T; r += blockDim.x) {
    int per = 0;
    const int tiles = (kvlen[r] + kMlaPage - 1) / kMlaPage;
    cnt[r] = tiles > 0 ? kv_splits(tiles, tiles_per_split, max_splits, &per) : 0;     // nothing cached: no work item
    pers[r] = tiles > 0 ? per : 0;
  }
  __syncthreads();
  const bool by_size = T <= 256;
  for (int r = threadIdx.x; r < T; r += blockDim.x) {
    const int my = pers[r];
    int off = 0;
    for (int q = 0; q < T; ++q) {
      const bool before = by_size ? (pers[q] > my || (pers[q] == my && q < r)) : q < r;
      off += before ? cnt[q] : 0;
    }
    const int tiles = (kvlen[r] + kMlaPage - 1) / kMlaPage;
    const int ns = cnt[r], per = my > 0 ? my : 1;
    for (int split = 0; split < ns; ++split) {
      const int t0 = split * per;
      const int nt = min(per, tiles - t0);
      items[2 * (off + split)] = MlaItem{r, 0, split, t0, nt, 0, 0, 0};
      items[2 * (off + split) + 1] = MlaItem{r, 1, split, t0, nt, 0, 0, 0};
    }
  }
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int q = 0; q < T; ++q) tot += cnt[q];
    *n_items = 2 * tot;
  }
}

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_kernel(const MlaArgs a, const __grid_constant__ CUtensorMap tm_qr,
                  const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_kvr) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + kQBytes;
  uint8_t* ctrl = kv_smem + kMlaStages * kKvStageBytes;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* q_empty = q_full + 1;
  uint64_t* kv_full = q_empty + 1;           // [kMlaStages]
  uint64_t* kv_empty = kv_full + kMlaStages; // [kMlaStages]
  uint64_t* s_full = kv_empty + kMlaStages;  // [2]
  uint64_t* qt_full = s_full + 2;            // [1] latent Q stored to TMEM by the softmax warps
  uint64_t* p_full = qt_full + 1;            // [2]
  uint64_t* pv_done = p_full + 2;            // [2] indexed by tile parity (see the softmax warps)
  uint64_t* o_free = pv_done + 2;            // [1]
  uint64_t* drain_bar = o_free + 1;          // [1]
  uint64_t* xchg_bar = drain_bar + 1;        // [2] softmax half-row exchange
  uint64_t* it_full = xchg_bar + 2;          // [4] the producer has published the item index of item n in slot n & 3
  volatile int* item_slot = reinterpret_cast<volatile int*>(it_full + 4);   // [4]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(const_cast<int*>(item_slot) + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* never_flag = abort_flag + 1;
  float2* xchg = reinterpret_cast<float2*>(ctrl + 1024);   // [2 parity][2 half][128 rows] (max, sk max)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < kMlaStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 8); mbar_init(&xchg_bar[b], 8); }
    mbar_init(qt_full, 8);
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    mbar_init(o_free, 8);
    mbar_init(drain_bar, 1);
    for (int b = 0; b < 4; ++b) mbar_init(&it_full[b], 1);
    *abort_flag = 0;
    *never_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_qr); tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_kvr);
  }
  if (warp == 1) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_s = tmem_base;          // S buffers: columns [0,64) and [64,128); P aliases the first 16 of each
  const uint32_t tm_o = tmem_base + 128;    // O: 256 columns
  const uint32_t tm_q = tmem_base + 384;    // latent Q as e4m3 A operand: 128 columns (4 bytes of K per column)
  pdl_wait();     // work list, queries and this step's cache rows come from the kernels before this one
  const int n_items = *a.n_items;
  // Items are handed out dynamically: requests differ eightfold in length, and a static deal left some CTAs with
  // half again the average work.  The producer thread takes the next index from the launch's counter and publishes
  // it (or -1 at the end) through shared memory; the other roles pick it up from there.
  auto consumer_item = [&](uint32_t n) -> int {
    if (!mbar_wait(&it_full[n & 3], (n >> 2) & 1, abort_flag)) return -2;
    return item_slot[n & 3];
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t item_it = 0, kv_it = 0;
      bool ok = true;
      for (;; ++item_it) {
        int it = ok ? atomicAdd(a.claim, 1) : n_items;
        if (it >= n_items) it = -1;
        item_slot[item_it & 3] = it;
        mbar_arrive(&it_full[item_it & 3]);     // release: the slot write is visible to whoever sees the phase complete
        if (it < 0) break;
        const MlaItem w = a.items[it];
        if (!mbar_wait(q_empty, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagMlaDecode); ok = false; continue; }
        mbar_expect_tx(q_full, kQBytes);
        tma_load_3d(q_smem, &tm_qr, 512, w.req, 0, q_full);
        const int* pt = a.page_table + static_cast<size_t>(a.slot_of[w.req]) * a.max_pages;
        int page_next = pt[w.tile0];
        for (int i = 0; i < w.ntiles; ++i, ++kv_it) {
          const int s = kv_it % kMlaStages;
          // the page id of the next tile is fetched before waiting for this tile's stage, so the
          // table lookup never sits between a freed stage and its refill
          const int page = page_next;
          if (i + 1 < w.ntiles) page_next = pt[w.tile0 + i + 1];
          if (!mbar_wait(&kv_empty[s], ((kv_it / kMlaStages) & 1) ^ 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagMlaDecode); ok = false; break;
          }
          uint8_t* st = kv_smem + s * kKvStageBytes;
          mbar_expect_tx(&kv_full[s], kKvTileBytes + 256 + 16);
          for (int c = 0; c < 4; ++c) tma_load_2d(st + c * 8192, &tm_kv, c * 128, page * kMlaPage, &kv_full[s]);
          tma_load_2d(st + 32768, &tm_kvr, 512, page * kMlaPage, &kv_full[s]);
          bulk_load_1d(st + kKvTileBytes, a.kv_scale + static_cast<size_t>(page) * kMlaPage, 256, &kv_full[s]);
          bulk_load_1d(st + kKvTileBytes + 256, a.kv_smax + static_cast<size_t>(page) * 4, 16, &kv_full[s]);
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
        if (!mbar_wait(&kv_full[s], (kvi / kMlaStages) & 1, abort_flag)) { atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagMlaDecode); return false; }
        tc_fence_after();
        // S buffer ti&1 (and the P written over it) was last read by P.V of tile ti-2, which was
        // issued before this point and executes in order ahead of these MMAs.
        const uint32_t d = tm_s + (ti & 1) * 64;
        const uint32_t ka = smem_u32(kv_smem + s * kKvStageBytes);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint64_t kd = umma_desc_k128(ka + c * 8192);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f8_ts(d, tm_q + (c * 4 + k) * 8, kd + 2 * k, idesc_qk, (c | k) != 0);
        }
        const uint64_t qd = umma_desc_k64(smem_u32(q_smem)), kd = umma_desc_k64(ka + 32768);
        tc_mma_f8(d, qd, kd, idesc_qk, 1);
        tc_mma_f8(d, qd + 2, kd + 2, idesc_qk, 1);
        tc_commit(&s_full[ti & 1]);
        return true;
      };
      for (; ok; ++item_it) {
        const int it = consumer_item(item_it);
        if (it < 0) { if (it == -2) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagMlaDecode); } break; }
        const MlaItem w = a.items[it];
        if (!mbar_wait(q_full, item_it & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagMlaDecode); break; }
        if (!mbar_wait(qt_full, item_it & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); break; }
        tc_fence_after();
        if (!issue_qk(kv_it, tile_it)) { *abort_flag = 1; break; }
        for (int i = 0; i < w.ntiles; ++i) {
          if (i + 1 < w.ntiles) {
            if (!issue_qk(kv_it + i + 1, tile_it + i + 1)) { *abort_flag = 1; ok = false; break; }
          } else {
            tc_commit(q_empty);   // every QK^T of this item is issued: Q may be overwritten once they retire
          }
          const uint32_t ti = tile_it + i;
          if (i == 0 && !mbar_wait(o_free, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_FREE_WAIT | kTagMlaDecode); ok = false; break; }
          if (!mbar_wait(&p_full[ti & 1], (ti >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); ok = false; break; }
          tc_fence_after();
          const int s = (kv_it + i) % kMlaStages;
          const uint32_t pt = tm_s + (ti & 1) * 64;   // P: 16 columns = 64 tokens of e4m3
          const uint32_t va = smem_u32(kv_smem + s * kKvStageBytes) + w.half * 2 * 8192;
          tc_mma_f8_ts(tm_o, pt, umma_desc_mn128(va, 8192, 1024), idesc_pv, i > 0);
          tc_mma_f8_ts(tm_o, pt + 8, umma_desc_mn128(va + 4096, 8192, 1024), idesc_pv, 1);
          tc_commit(&kv_empty[s]);
          tc_commit(&pv_done[ti & 1]);
          PLOW_TRACE(if (a.trace && blockIdx.x == 0 && ti < 64) a.trace[ti * 8 + 7] = clock64();)
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
    for (; ok; ++item_it) {
      const int it = consumer_item(item_it);
      if (it < 0) { if (it == -2) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagMlaDecode); } break; }
      const MlaItem w = a.items[it];
      const int kv_len = a.kvlen[w.req];
      const float qs = a.sq[static_cast<size_t>(li) * a.T + w.req] * a.scale_log2e;
      float m = 0.f, l = 0.f, SK = 1.f, M = 0.f;
      {
        // latent Q of this (head, request) into TMEM: this thread owns bytes [256 ch, 256 ch + 256)
        // of the row, i.e. TMEM columns [64 ch, 64 ch + 64).  The previous item's QK^T must have
        // retired before its Q is overwritten.
        if (!mbar_wait(q_empty, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_FREE_WAIT | kTagMlaDecode); ok = false; break; }
        tc_fence_after();
        const uint4* qrow = reinterpret_cast<const uint4*>(a.q8 + (static_cast<size_t>(li) * a.T + w.req) * kMlaRow + ch * 256);
        uint32_t qv[64];
#pragma unroll
        for (int j = 0; j < 16; ++j) { const uint4 v = qrow[j]; qv[4 * j] = v.x; qv[4 * j + 1] = v.y; qv[4 * j + 2] = v.z; qv[4 * j + 3] = v.w; }
#pragma unroll
        for (int j = 0; j < 4; ++j) tmem_st16(tm_q + lane_addr + ch * 64 + j * 16, qv + j * 16);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(qt_full);
      }
      for (int i = 0; i < w.ntiles; ++i) {
        const uint32_t ti = tile_it + i;
        PLOW_TRACE(const bool tr = a.trace && blockIdx.x == 0 && warp == 2 && lane == 0 && ti < 64;)
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 0] = clock64();)
        // (a) per-token scales (they arrived with the KV tile, usually long before S is ready)
        const int s = (kv_it + i) % kMlaStages;
        if (!mbar_wait(&kv_full[s], ((kv_it + i) / kMlaStages) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagMlaDecode); ok = false; break; }
        const float* sk_base = reinterpret_cast<const float*>(kv_smem + s * kKvStageBytes + kKvTileBytes);
        const float4* sk4 = reinterpret_cast<const float4*>(sk_base) + ch * 8;
        const float skmax = fmaxf(sk_base[64], 1e-30f);   // upper bound of this page's scales, kept by the cache writer
        const int valid = min(kMlaPage, kv_len - (w.tile0 + i) * kMlaPage) - ch * 32;   // valid columns of this half
        float skv[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 k4 = sk4[j];
          skv[4 * j] = k4.x; skv[4 * j + 1] = k4.y; skv[4 * j + 2] = k4.z; skv[4 * j + 3] = k4.w;
        }
        // (b) scores
        if (!mbar_wait(&s_full[ti & 1], (ti >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); ok = false; break; }
        tc_fence_after();
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 1] = clock64();)
        uint32_t sv[32];
        tmem_ld32(tm_s + lane_addr + (ti & 1) * 64 + ch * 32, sv);
        tmem_ld_wait();
        float x[32];
        float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (valid >= 32) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            x[j] = __uint_as_float(sv[j]) * (qs * skv[j]);
            mxa[j & 3] = fmaxf(mxa[j & 3], x[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            x[j] = j < valid ? __uint_as_float(sv[j]) * (qs * skv[j]) : -INFINITY;
            mxa[j & 3] = fmaxf(mxa[j & 3], x[j]);
          }
        }
        float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
        float omx, unused0;
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 2] = clock64();)
        if (!exchange(mx, 0.f, omx, unused0)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); ok = false; break; }
        mx = fmaxf(mx, omx);
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 3] = clock64();)
        // Lazy rescaling with one running offset M = m + log2(SK): probabilities are formed as
        // p' = 2^(x - M) * sk <= 2^kTau * sk / SK <= 2^kTau, inside e4m3 range, and l' = sum 2^(x - M)
        // is kept with the same offset, so O / l' needs no further correction at the end.  m is
        // only raised when a tile exceeds it by more than kTau (log2 units) and SK (an upper bound
        // of the scales seen, with 2x head-room) only when a page exceeds it, so the accumulator in
        // TMEM is almost never touched.  Both threads of a row see the same (mx, skmax) and take
        // the same decision.
        constexpr float kTau = 7.0f;
        if (i == 0) {
          m = mx;
          SK = skmax * 2.0f;
          M = m + log2f(SK);
        } else {
          const bool up_m = mx > m + kTau;
          const bool up_sk = skmax > SK;
          if (__any_sync(0xffffffffu, up_m || up_sk)) {
            const float m_new = up_m ? mx : m;
            const float SK_new = up_sk ? skmax * 2.0f : SK;
            const float M_new = m_new + log2f(SK_new);
            const float alpha = exp2f(M - M_new);
            l *= alpha;
            m = m_new;
            SK = SK_new;
            M = M_new;
            // accumulator must be quiescent: P.V of the previous tile has retired.  QK^T of this
            // tile was issued after P.V of tile ti-2, so at most tile ti-1 is pending on its
            // parity's barrier and the phase below cannot alias.
            if (!mbar_wait(&pv_done[(ti - 1) & 1], ((ti - 1) >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
              uint32_t o[32];
              tmem_ld32(tm_o + lane_addr + ch * 128 + c, o);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
              tmem_st16(tm_o + lane_addr + ch * 128 + c, o);
              tmem_st16(tm_o + lane_addr + ch * 128 + c + 16, o + 16);
            }
            tmem_st_wait();
            tc_fence_before();
          }
        }
        // (c) exponentials.  The MUFU unit sustains 16 ex2 per clock per SM (512 clocks for a
        // 128 x 64 tile); one column in four is evaluated on the FMA pipe instead (round-down
        // magic add for floor, cubic for 2^frac, exponent spliced in with integer ops; 1e-4
        // relative error, far below e4m3's), so both pipes run side by side.
        float suma = 0.f, sumb = 0.f;
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float p[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float t = x[j + u] - M;
            float e;
            if (u == 3) {
              const float tc = fmaxf(t, -126.0f);
              const float r = __fadd_rd(tc, 12582912.0f);            // 1.5 * 2^23 + floor(t)
              const float f = tc - (r - 12582912.0f);                // frac in [0, 1)
              const float pf = fmaf(fmaf(fmaf(0.07908570f, f, 0.22451635f), f, 0.69639057f), f, 0.99989671f);
              e = __int_as_float(__float_as_int(pf) + (__float_as_int(r) << 23));
              sumb += e;
            } else {
              asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
              suma += e;
            }
            p[u] = e * skv[j + u];
          }
          __nv_fp8x4_e4m3 q4(make_float4(p[0], p[1], p[2], p[3]));
          pk[j >> 2] = *reinterpret_cast<uint32_t*>(&q4);
        }
        l += suma + sumb;
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 4] = clock64();)
        // P (e4m3, 4 tokens per 32-bit column) over the first 16 columns of the S buffer it came
        // from; this thread owns tokens [32 ch, 32 ch + 32) = columns [8 ch, 8 ch + 8).  The
        // partner thread finished reading its S columns before the exchange above completed.
        tmem_st8(tm_s + lane_addr + (ti & 1) * 64 + ch * 8, pk);
        tmem_st_wait();
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 5] = clock64();)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[ti & 1]);
        PLOW_TRACE(if (tr) a.trace[ti * 8 + 6] = clock64();)
      }
      if (!ok) break;
      // ---- finalize this item: O * SK / l, log-sum-exp in the log2 domain
      float ol, unused;
      if (!exchange(l, 0.f, ol, unused)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); break; }
      l += ol;
      const uint32_t ti_last = tile_it + w.ntiles - 1;
      if (!mbar_wait(&pv_done[ti_last & 1], (ti_last >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagMlaDecode); break; }
      tc_fence_after();
      const float fin = l > 0.f ? 1.0f / l : 0.f;
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
      if (w.half == 0 && ch == 0) a.lse[(static_cast<size_t>(w.req) * a.max_splits + w.split) * kMlaHeads + li] = M + log2f(fmaxf(l, 1e-30f));
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
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int tiles = (kvlen[t] + kMlaPage - 1) / kMlaPage;
  int per_unused;
  const int ns = kv_splits(tiles, tiles_per_split, max_splits, &per_unused);
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

#ifdef PLOW_DEVICE_TRACE
static long long* g_mla_trace = nullptr;
#endif

extern "C" {

#ifdef PLOW_DEVICE_TRACE
// Builds with -DPLOW_DEVICE_TRACE only: device buffer of 64*8 int64 that CTA 0 fills with clock64() phase stamps.
void plow_mla_set_trace(void* p) { g_mla_trace = static_cast<long long*>(p); }
#endif

// The work list depends only on the rows' KV lengths, which are the same for every layer of a step: the engine
// builds it once per step with this entry and passes build_items = 0 to plow_mla_decode for every layer.
// `claims`: int[256] work counters, zeroed here; every decode launch until the next build takes its own (claim_slot).
int plow_mla_build_items(const int* kvlen, int T, int tiles_per_split, int max_splits, void* items, int* n_items, int* claims, void* stream_) {
  using namespace plow;
  if (T <= 0 || max_splits <= 0 || tiles_per_split <= 0) return -1;
  cudaError_t e = launch_serial(mla_build_items, dim3(1), dim3(256), 2 * T * sizeof(int), reinterpret_cast<cudaStream_t>(stream_),
                             kvlen, T, tiles_per_split, max_splits, static_cast<MlaItem*>(items), n_items, claims);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// Scratch the caller provides: items (8 ints per item, capacity 2*T*max_splits), n_items (1 int),
// opart bf16 [T][max_splits][128][512], lse f32 [T][max_splits][128].
// q8 e4m3 [128 heads][T][576]; sq f32 [128][T]; kv e4m3 [n_pages][64][576]; kv_scale f32 [n_pages][64];
// kv_smax f32 [n_pages][4] (element 0: an upper bound of the page's scales, maintained by the cache writer);
// out bf16 [128][T][512].
int plow_mla_decode(const void* q8, const float* sq, const void* kv, const float* kv_scale, const float* kv_smax, int64_t n_pages,
                    const int* page_table, int max_pages, const int* slot_of, const int* kvlen, int T,
                    int tiles_per_split, int max_splits, void* items, int* n_items, void* opart, float* lse,
                    void* out, float softmax_scale, int build_items, int* claims, int claim_slot, int* status, void* stream_) {
  using namespace plow;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || max_splits <= 0 || tiles_per_split <= 0 || !claims) return -1;
  CUtensorMap tqr, tkv, tkvr;
  int r = make_tmap_3d(&tqr, q8, 1, kMlaRow, T, kMlaHeads, kMlaRow, static_cast<uint64_t>(T) * kMlaRow, 1, 128, 64);
  if (r) return 1100 + r;
  r = make_tmap_2d(&tkv, kv, 1, static_cast<uint64_t>(n_pages) * kMlaPage, kMlaRow, kMlaRow, kMlaPage, 128);
  if (r) return 1200 + r;
  r = make_tmap_2d(&tkvr, kv, 1, static_cast<uint64_t>(n_pages) * kMlaPage, kMlaRow, kMlaRow, kMlaPage, 64);
  if (r) return 1300 + r;
  static DeviceOnce attr;
  if (ensure_smem(attr, mla_decode_kernel, kMlaSmem) != cudaSuccess) return 3000;
  if (build_items)
    launch_serial(mla_build_items, dim3(1), dim3(256), 2 * T * sizeof(int), stream, kvlen, T, tiles_per_split, max_splits,
                  static_cast<MlaItem*>(items), n_items, claims);
  MlaArgs a;
  a.q8 = static_cast<const uint8_t*>(q8); a.sq = sq; a.kv_scale = kv_scale; a.kv_smax = kv_smax; a.page_table = page_table; a.slot_of = slot_of; a.kvlen = kvlen;
  a.items = static_cast<const MlaItem*>(items); a.n_items = n_items;
  a.claim = claims + (build_items ? 0 : ((claim_slot % kMlaClaimSlots) + kMlaClaimSlots) % kMlaClaimSlots);
  a.opart = static_cast<__nv_bfloat16*>(opart); a.lse = lse; a.status = status;
#ifdef PLOW_DEVICE_TRACE
  a.trace = g_mla_trace;
#else
  a.trace = nullptr;
#endif
  a.T = T; a.max_pages = max_pages; a.max_splits = max_splits;
  a.scale_log2e = softmax_scale * 1.4426950408889634f;
  int grid = sm_count();
  const int cap = 2 * T * max_splits;
  if (cap < grid) grid = cap;
  cudaError_t e = launch_serial(mla_decode_kernel, dim3(grid), dim3(kMlaThreads), kMlaSmem, stream, a, tqr, tkv, tkvr);
  if (e == cudaSuccess && out)   // NULL: the caller merges the splits itself (plow_mla_fold does it while folding W_uv)
    e = launch_serial(mla_merge_kernel, dim3(T, kMlaHeads), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(opart),
                   static_cast<const float*>(lse), kvlen, T, max_splits, tiles_per_split, static_cast<__nv_bfloat16*>(out));
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
