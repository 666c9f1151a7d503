// Grouped-query flash attention over a paged bf16 KV cache, on tcgen05 — one kernel for prefill and
// decode — plus the fused head-norm + RoPE + cache-write row op that feeds it.
//
// The step's query rows arrive as q[row][head][HD]; each row carries (slot, position) and attends
// to the cached positions t <= position of its slot (optionally t > position - window), which makes
// prefill causal and decode a one-row special case of the same rule.  The 128 TMEM lanes of a CTA
// hold (token, group head) pairs of ONE kv head: 128/group consecutive tokens of a sequence times
// the `group` query heads that share the kv head.  Per 64-token cache page:
//     S[128 x 64]  = Q[128 x HD] . K[64 x HD]^T           (UMMA, both operands in shared memory)
//     P            = 2^(S*scale*log2e - m)                (lane = row: no cross-thread reduction)
//     O[128 x HD] += P[128 x 64] . V[64 x HD]             (UMMA, P read from TMEM as the A operand,
//                                                          V as an MN-major B operand)
// K and V tiles come straight from the paged cache by TMA (3-D maps: HD x kv_heads x tokens), Q by
// one 3-D TMA per 64-column slab whose box is (64, group, 128/group), so shared memory receives the
// rows already ordered token-major / head-minor.  The accumulator is rescaled lazily (only when the
// running maximum grows by more than 2^7), as in the latent-attention decode kernel.
//
// Work items (row chunk, kv head, kv split) are built on the device from (slot, position), so the
// op can sit inside a captured decode graph; splits write normalised f32 partials + log-sum-exp and
// `gqa_merge_kernel` folds them (gm = max m_s; O = sum O_s 2^(lse_s - gm) / sum 2^(lse_s - gm)).
// Reference semantics: runtime/common/dev_isa.h:185-222 (split-KV partials + FLASH_MERGE, decode
// with kv_len / window) and :74-84 (HEADNORM_ROPE writing the cache row directly); the reference's
// own sm_120 kernels are mma.sync flash kernels (runtime/nvidia/op_attention*.cuh).
//
// e4m3 cache (KV8 instantiation): K and V cells are e4m3 bytes with one f32 scale per (token, kv head).  The TMA warp
// brings the raw byte tiles into a staging ring; converter warps rewrite each tile as bf16 operands in the layout the
// MMAs read (the 128-byte swizzle a bf16 TMA load would produce) and hand the stage to the MMA warp.  The rewrite is
// The rewrite is three integer instructions per element pair: the e4m3 byte s.eeee.mmm placed as the bf16
// s.0000eeee.mmm0000 is exactly value * 2^-120 (normal and subnormal codes alike), so no float conversion is needed;
// the per-token scales and the 2^120 go where a multiplication already is or costs one instruction: S columns are
// multiplied by k_scale[j] * scale * log2e * 2^120 instead of the constant, P columns by v_scale[j] * 2^60 before
// they are rounded to bf16, and the output by 2^60.  Half the cache bytes, same tiles
// (reference: runtime/common/dev_isa.h:388-398, HEADNORM_ROPE_FP8 / FLASH_*_FP8).
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace plow {

constexpr int kGqaPage = 64;
constexpr int kGqaThreads = 192;   // TMA warp, MMA warp, 4 softmax warps
constexpr int kGqaThreads8 = 320;  // + 4 converter warps (e4m3 cache)
constexpr int kGqaRaw = 3;         // raw e4m3 tiles in flight; 4 operand stages behind them

struct GqaItem { int r0, nt, kvh, split, tile0, ntiles, slot, ns; };

struct GqaArgs {
  const int* page_table;   // [n_slots][max_pages]
  const int* pos;          // [rows]
  const GqaItem* items;
  const int* n_items;
  float* opart;            // [rows][nq][max_splits][HD] normalised partial outputs
  float* lse;              // [rows][nq][max_splits] log2-domain log-sum-exp
  __nv_bfloat16* out;      // [rows][nq*HD]
  int* status;
  int rows, nq, nkv, group, max_pages, max_splits, window;
  float scale_log2e;
  // materialised multi-head latent attention: the last `kr_slabs` key slabs come from a separate tensor shared by
  // all heads (the rotary part), and the value tile sits `v_x0` columns into the key tensor's head block
  int kr_slabs, v_x0;
  int head_major;          // items are [chunk][head] (one split): visit them head by head
  const float* kv_scale;   // e4m3 cache: [n_pages][64][2 * nkv] f32, k scales then v scales of a token
};

// HDQ = width of a query / key row, HDV = width of a value row.  They differ for multi-head latent attention in its
// materialised form (192 = 128 no-position + 64 rotary dims against 128 value dims).
template <int HDQ, int HDV, bool KV8 = false> struct GqaCfg {
  static constexpr int kSlabsQ = HDQ / 64;               // 64-column (128-byte) slabs per query / key row
  static constexpr int kSlabsV = HDV / 64;
  static constexpr int kQBytes = kSlabsQ * 128 * 128;
  static constexpr int kKBytes = kSlabsQ * 64 * 128;     // one K tile
  static constexpr int kVBytes = kSlabsV * 64 * 128;     // one V tile
  static constexpr int kStageBytes = kKBytes + kVBytes;
  static constexpr int kRawK = 64 * HDQ;                 // one raw e4m3 K tile: HDQ / 128 slabs of 64 rows x 128 bytes
  static constexpr int kRawStage = 64 * (HDQ + HDV);
  static constexpr int kRawBytes = KV8 ? kGqaRaw * kRawStage : 0;
  static constexpr int kStagesFit = (200 * 1024 - kQBytes) / kStageBytes;
  static constexpr int kStages = KV8 ? 4 : (kStagesFit > 5 ? 5 : kStagesFit);
  // per operand stage: 64 S-column and 64 P-column factors; then a ring of 128 page numbers for the converter warps
  static constexpr int kColBytes = KV8 ? kStages * 128 * 4 + 128 * 4 : 0;
  static constexpr int kSmem = 1024 + kQBytes + kStages * kStageBytes + kRawBytes + kColBytes + 1024;
  static constexpr int kThreads = KV8 ? kGqaThreads8 : kGqaThreads;
  static constexpr int kTmemCols = HDV <= 128 ? 256 : 512; // S: 2 x 64, O: HDV
  static_assert(kStages >= 2, "K/V stages do not fit");
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
};

// ---------------------------------------------------------------------------------------------
// A chunk starts at every multiple of tq rows and wherever the (slot, position) run breaks, so a
// row can tell locally whether it starts one; that thread emits the chunk's items.
__global__ void gqa_build_items(const int* seq, const int* pos, int rows, int tq, int nkv, int window,
                                int tiles_per_split, int max_splits, GqaItem* items, int* n_items,
                                int* row_ns, int cap, int* status) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    if (pos[r] < 0) { row_ns[r] = 0; continue; }
    const bool start = (r % tq == 0) || pos[r - 1] < 0 || seq[r] != seq[r - 1] || pos[r] != pos[r - 1] + 1;
    if (!start) continue;
    int nt = 1;
    while ((r + nt) % tq != 0 && r + nt < rows && seq[r + nt] == seq[r] && pos[r + nt] == pos[r + nt - 1] + 1) ++nt;
    const int hi = pos[r + nt - 1];
    const int lo = window > 0 ? max(0, pos[r] - window + 1) : 0;
    const int tile_lo = lo / kGqaPage;
    const int tiles = hi / kGqaPage + 1 - tile_lo;
    int ns = min(max_splits, (tiles + tiles_per_split - 1) / tiles_per_split);
    const int per = (tiles + ns - 1) / ns;
    ns = (tiles + per - 1) / per;
    for (int j = 0; j < nt; ++j) row_ns[r + j] = ns;
    const int base = atomicAdd(n_items, nkv * ns);
    if (base + nkv * ns > cap) { atomicCAS(status, 0, PLOW_ERR_BOUNDS | kTagGqa); continue; }
    for (int h = 0; h < nkv; ++h)
      for (int s = 0; s < ns; ++s)
        items[base + h * ns + s] = GqaItem{r, nt, h, s, tile_lo + s * per, min(per, tiles - s * per), seq[r], ns};
  }
}

template <int HDQ, int HDV, bool KV8 = false>
__global__ void __launch_bounds__((GqaCfg<HDQ, HDV, KV8>::kThreads), 1)
gqa_attn_kernel(const GqaArgs a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kr) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  using Cfg = GqaCfg<HDQ, HDV, KV8>;
  constexpr int HD = HDV;      // width of the accumulator rows
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + Cfg::kQBytes;
  uint8_t* raw_smem = kv_smem + Cfg::kStages * Cfg::kStageBytes;     // e4m3 cache: raw byte tiles (1024-aligned: all sizes are)
  float* col_fac = reinterpret_cast<float*>(raw_smem + Cfg::kRawBytes);   // [kStages][128]
  uint8_t* ctrl = raw_smem + Cfg::kRawBytes + Cfg::kColBytes;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* q_empty = q_full + 1;
  uint64_t* kv_full = q_empty + 1;                 // [kStages]
  uint64_t* kv_empty = kv_full + Cfg::kStages;     // [kStages]
  uint64_t* s_full = kv_empty + Cfg::kStages;      // [2]
  uint64_t* p_full = s_full + 2;                   // [2]
  uint64_t* pv_done = p_full + 2;                  // [2] by tile parity
  uint64_t* o_free = pv_done + 2;                  // [1]
  uint64_t* drain_bar = o_free + 1;                // [1]
  uint64_t* raw_full = drain_bar + 1;              // [kGqaRaw] (e4m3 cache only)
  uint64_t* raw_empty = raw_full + kGqaRaw;        // [kGqaRaw]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(raw_empty + kGqaRaw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* never_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1); }
    mbar_init(o_free, 4);
    mbar_init(drain_bar, 1);
    for (int r = 0; r < kGqaRaw; ++r) { mbar_init(&raw_full[r], 1); mbar_init(&raw_empty[r], 1); }
    *abort_flag = 0;
    *never_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_kr);
  }
  if (warp == 1) { tmem_alloc(tmem_holder, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_s = tmem_base;         // S buffers [0,64) and [64,128); P (bf16 pairs) over the first 32 of each
  const uint32_t tm_o = tmem_base + 128;   // O: HD columns
  const int n_items = *a.n_items;
  // head-major visiting order (every chunk holds one item per head, no splits): the CTAs running at one time then
  // work on a handful of heads and share those heads' K / V through L2, instead of touching every head's K / V at once
  const int n_chunks = a.head_major ? n_items / a.nkv : 0;
  auto item_at = [&](int it) -> GqaItem {
    return a.items[a.head_major ? (it % n_chunks) * a.nkv + it / n_chunks : it];
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t item_it = 0, kv_it = 0;
      bool ok = true;
      for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x, ++item_it) {
        const GqaItem w = item_at(it);
        if (!mbar_wait(q_empty, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagGqa); break; }
        mbar_expect_tx(q_full, Cfg::kQBytes);
        for (int c = 0; c < Cfg::kSlabsQ; ++c) tma_load_3d(q_smem + c * 16384, &tm_q, c * 64, w.kvh * a.group, w.r0, q_full);
        const int* pt = a.page_table + static_cast<size_t>(w.slot) * a.max_pages;
        int page_next = pt[w.tile0];
        for (int i = 0; i < w.ntiles; ++i, ++kv_it) {
          const int s = kv_it % Cfg::kStages;
          const int page = page_next;
          if (i + 1 < w.ntiles) page_next = pt[w.tile0 + i + 1];
          if constexpr (KV8) {
            // raw byte tiles into the staging ring; the converter warps own the operand stages
            const int rs = kv_it % kGqaRaw;
            if (!mbar_wait(&raw_empty[rs], ((kv_it / kGqaRaw) & 1) ^ 1, abort_flag)) {
              *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagGqa); ok = false; break;
            }
            uint8_t* rw = raw_smem + rs * Cfg::kRawStage;
            mbar_expect_tx(&raw_full[rs], Cfg::kRawStage);
            for (int c = 0; c < HDQ / 128; ++c) tma_load_3d(rw + c * 8192, &tm_k, c * 128, w.kvh, page * kGqaPage, &raw_full[rs]);
            for (int c = 0; c < HDV / 128; ++c) tma_load_3d(rw + Cfg::kRawK + c * 8192, &tm_v, c * 128, w.kvh, page * kGqaPage, &raw_full[rs]);
            continue;
          }
          if (!mbar_wait(&kv_empty[s], ((kv_it / Cfg::kStages) & 1) ^ 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagGqa); ok = false; break;
          }
          uint8_t* st = kv_smem + s * Cfg::kStageBytes;
          mbar_expect_tx(&kv_full[s], Cfg::kStageBytes);
          for (int c = 0; c < Cfg::kSlabsQ; ++c) {
            if (c < Cfg::kSlabsQ - a.kr_slabs) tma_load_3d(st + c * 8192, &tm_k, c * 64, w.kvh, page * kGqaPage, &kv_full[s]);
            else tma_load_3d(st + c * 8192, &tm_kr, (c - (Cfg::kSlabsQ - a.kr_slabs)) * 64, 0, page * kGqaPage, &kv_full[s]);
          }
          for (int c = 0; c < Cfg::kSlabsV; ++c)
            tma_load_3d(st + Cfg::kKBytes + c * 8192, &tm_v, a.v_x0 + c * 64, w.kvh, page * kGqaPage, &kv_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_qk = umma_idesc(128, 64, 1, 1);
      const uint32_t idesc_pv = umma_idesc(128, HD, 1, 1, 0, 1);
      uint32_t item_it = 0, kv_it = 0, tile_it = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t kvi, uint32_t ti) -> bool {
        const int s = kvi % Cfg::kStages;
        if (!mbar_wait(&kv_full[s], (kvi / Cfg::kStages) & 1, abort_flag)) { atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagGqa); return false; }
        tc_fence_after();
        // S buffer ti&1 (and the P written over it) was last read by P.V of tile ti-2, issued
        // before this point; the tensor pipe executes in order.
        const uint32_t d = tm_s + (ti & 1) * 64;
        const uint32_t qa = smem_u32(q_smem), ka = smem_u32(kv_smem + s * Cfg::kStageBytes);
#pragma unroll
        for (int c = 0; c < Cfg::kSlabsQ; ++c) {
          const uint64_t qd = umma_desc_k128(qa + c * 16384), kd = umma_desc_k128(ka + c * 8192);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f16(d, qd + 2 * k, kd + 2 * k, idesc_qk, (c | k) != 0);
        }
        tc_commit(&s_full[ti & 1]);
        return true;
      };
      for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x, ++item_it) {
        const GqaItem w = item_at(it);
        if (!mbar_wait(q_full, item_it & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagGqa); break; }
        tc_fence_after();
        if (!issue_qk(kv_it, tile_it)) { *abort_flag = 1; break; }
        for (int i = 0; i < w.ntiles; ++i) {
          if (i + 1 < w.ntiles) {
            if (!issue_qk(kv_it + i + 1, tile_it + i + 1)) { *abort_flag = 1; ok = false; break; }
          } else {
            tc_commit(q_empty);   // all QK^T of this item are issued: Q may be overwritten once they retire
          }
          const uint32_t ti = tile_it + i;
          if (i == 0 && !mbar_wait(o_free, (item_it & 1) ^ 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_FREE_WAIT | kTagGqa); ok = false; break; }
          if (!mbar_wait(&p_full[ti & 1], (ti >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGqa); ok = false; break; }
          tc_fence_after();
          const int s = (kv_it + i) % Cfg::kStages;
          const uint32_t pt = tm_s + (ti & 1) * 64;   // P: 32 columns = 64 tokens of bf16
          const uint32_t va = smem_u32(kv_smem + s * Cfg::kStageBytes + Cfg::kKBytes);
#pragma unroll
          for (int j = 0; j < 4; ++j)   // 16 tokens per MMA: two 8-token groups of 1024 bytes
            tc_mma_f16_ts(tm_o, pt + j * 8, umma_desc_mn128(va + j * 2048, 8192, 1024), idesc_pv, (i | j) != 0);
          tc_commit(&kv_empty[s]);
          tc_commit(&pv_done[ti & 1]);
        }
        kv_it += w.ntiles;
        tile_it += w.ntiles;
      }
      if (!ok || *abort_flag) { tc_commit(drain_bar); mbar_wait(drain_bar, 0, never_flag); }
    }
  } else if (KV8 && warp >= 6) {
    // ------------------------------------------------------------------ converter warps (e4m3 cache -> bf16 operand stages)
    // Thread u of the 128 handles work units (row = u % 64, out slab): 64 e4m3 bytes of one token -> 64 bf16 (one
    // 128-byte operand row).  Raw tiles and operand slabs are both 64 rows x 128 bytes with the 128-byte swizzle: the
    // 16-byte chunk j of row r sits at chunk j ^ (r & 7).
    const int u = threadIdx.x - 192;
    static_assert(!KV8 || (Cfg::kSlabsQ == 2 && Cfg::kSlabsV == 2), "converter mapping: 256 units of 64 bytes per tile, two per thread");
    uint32_t kv_it = 0;
    bool ok = true;
    for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x) {
      const GqaItem w = item_at(it);
      const int* pt = a.page_table + static_cast<size_t>(w.slot) * a.max_pages + w.tile0;
      // page numbers of the item's tiles in a shared ring (128 entries, refilled 64 at a time, 64 tiles ahead): the
      // scale fetch of tile i + 2 then starts from a shared-memory read instead of a dependent global load
      int* pages = reinterpret_cast<int*>(col_fac + Cfg::kStages * 128);
      pages[u] = u < w.ntiles ? pt[u] : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // thread u owns column factor u of every tile: k scale of token u (u < 64) or v scale of token u - 64, fetched two
      // tiles ahead; three slots in rotation (the loop is unrolled by three: a register a load still fills is never copied)
      auto scale_of = [&](int page) -> float {
        return a.kv_scale[(static_cast<size_t>(page) * kGqaPage + (u & 63)) * 2 * a.nkv + (u >= 64 ? a.nkv : 0) + w.kvh];
      };
      const float fac = u < 64 ? a.scale_log2e * 0x1p120f : 0x1p60f;
      float sl[3] = {0.f, 0.f, 0.f};
      sl[0] = scale_of(pages[0]);
      if (w.ntiles > 1) sl[1] = scale_of(pages[1]);
      auto tile_step = [&](int i, float s_cur, float& s_nxt) -> bool {
        const int s = kv_it % Cfg::kStages, rs = kv_it % kGqaRaw;
        if (i + 2 < w.ntiles) s_nxt = scale_of(pages[(i + 2) & 127]);
        // refill: tiles [i + 64, i + 128) replace the half of the ring whose tiles are all behind (first read 62 tiles
        // and as many barriers from now)
        if (i > 0 && (i & 63) == 0 && u < 64) pages[(i + 64 + u) & 127] = i + 64 + u < w.ntiles ? pt[i + 64 + u] : 0;
        bool mine = mbar_wait(&raw_full[rs], (kv_it / kGqaRaw) & 1, abort_flag) &&
                    mbar_wait(&kv_empty[s], ((kv_it / Cfg::kStages) & 1) ^ 1, abort_flag);
        // column factors of the stage: [0,64) S factors, [64,128) the v scales the conversion below reads
        if (mine) col_fac[s * 128 + u] = fminf(s_cur * fac, 3.0e38f);
        // one decision for all 128 threads (a barrier with an OR over "my wait ran out or somebody gave up")
        uint32_t stop;
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(stop) : "r"(static_cast<uint32_t>(!mine || *abort_flag)) : "memory");
        if (stop) {
          if (u == 0) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagGqa); }
          return false;
        }
        const uint8_t* rw = raw_smem + rs * Cfg::kRawStage;
        uint8_t* st = kv_smem + s * Cfg::kStageBytes;
        {
          // thread u: the K unit and the V unit of (row u % 64, 64-dim half u / 64); both unrolled, so that the loads and
          // the integer rewrites of 128 bytes overlap
          const int slab = u >> 6, row = u & 63;
          uint4 rv[8];
#pragma unroll
          for (int kv = 0; kv < 2; ++kv)
#pragma unroll
            for (int c = 0; c < 4; ++c)
              rv[kv * 4 + c] = *reinterpret_cast<const uint4*>(rw + (kv ? Cfg::kRawK : 0) + row * 128 + ((slab * 4 + c) ^ (row & 7)) * 16);
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            uint8_t* dst = st + (kv ? Cfg::kKBytes : 0) + slab * 8192 + row * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {                           // 16 e4m3 bytes -> two 16-byte bf16 chunks
              const uint32_t wv[4] = {rv[kv * 4 + c].x, rv[kv * 4 + c].y, rv[kv * 4 + c].z, rv[kv * 4 + c].w};
              uint32_t o[8];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                // bytes (b0, b1) and (b2, b3) to the high bytes of two 16-bit lanes, then sign | (exp.mant >> 4)
                const uint32_t lo = __byte_perm(wv[q], 0, 0x1404), hi = __byte_perm(wv[q], 0, 0x3424);
                o[2 * q] = (lo & 0x80008000u) | ((lo >> 4) & 0x07f007f0u);
                o[2 * q + 1] = (hi & 0x80008000u) | ((hi >> 4) & 0x07f007f0u);
              }
              *reinterpret_cast<uint4*>(dst + ((2 * c) ^ (row & 7)) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(dst + ((2 * c + 1) ^ (row & 7)) * 16) = make_uint4(o[4], o[5], o[6], o[7]);
            }
          }
        }
        fence_proxy_async_smem();       // the MMAs read these stores through the async proxy
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (u == 0) { mbar_arrive(&kv_full[s]); mbar_arrive(&raw_empty[rs]); }
        ++kv_it;
        return true;
      };
      for (int i = 0; ok && i < w.ntiles; i += 3) {
        ok = tile_step(i, sl[0], sl[2]);
        if (ok && i + 1 < w.ntiles) ok = tile_step(i + 1, sl[1], sl[0]);
        if (ok && i + 2 < w.ntiles) ok = tile_step(i + 2, sl[2], sl[1]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue warps
    const int lq = warp & 3;           // TMEM lane quarter this warp may access
    const int li = lq * 32 + lane;     // row of the tile: token li / group, query head li % group
    const uint32_t lane_addr = static_cast<uint32_t>(lq * 32) << 16;
    uint32_t item_it = 0, tile_it = 0;
    bool ok = true;
    for (int it = blockIdx.x; ok && it < n_items; it += gridDim.x, ++item_it) {
      const GqaItem w = item_at(it);
      const int n_valid = w.nt * a.group;
      const bool warp_active = lq * 32 < n_valid;       // whole warp: rows past the chunk are never read
      const int tok = min(li / a.group, w.nt - 1);
      const int hi = a.pos[w.r0 + tok];
      const int lo = a.window > 0 ? max(0, hi - a.window + 1) : 0;
      float m = -1e30f, l = 0.f;
      for (int i = 0; i < w.ntiles; ++i) {
        const uint32_t ti = tile_it + i;
        if (!mbar_wait(&s_full[ti & 1], (ti >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGqa); ok = false; break; }
        tc_fence_after();
        if (warp_active) {
          uint32_t sv[64];
          tmem_ld32(tm_s + lane_addr + (ti & 1) * 64, sv);
          tmem_ld32(tm_s + lane_addr + (ti & 1) * 64 + 32, sv + 32);
          tmem_ld_wait();
          const int t0 = (w.tile0 + i) * kGqaPage;
          float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          // e4m3 cache: per-column factors of this tile's operand stage ([0,64): for S, [64,128): for P)
          const float* cf = col_fac + (ti % Cfg::kStages) * 128;
          if constexpr (KV8) {
            const float4* c4 = reinterpret_cast<const float4*>(cf);
            if (t0 >= lo && t0 + kGqaPage - 1 <= hi) {
#pragma unroll
              for (int j = 0; j < 64; j += 4) {
                const float4 c = c4[j >> 2];
                const float x0 = __uint_as_float(sv[j]) * c.x, x1 = __uint_as_float(sv[j + 1]) * c.y;
                const float x2 = __uint_as_float(sv[j + 2]) * c.z, x3 = __uint_as_float(sv[j + 3]) * c.w;
                sv[j] = __float_as_uint(x0); sv[j + 1] = __float_as_uint(x1);
                sv[j + 2] = __float_as_uint(x2); sv[j + 3] = __float_as_uint(x3);
                mxa[0] = fmaxf(mxa[0], x0); mxa[1] = fmaxf(mxa[1], x1); mxa[2] = fmaxf(mxa[2], x2); mxa[3] = fmaxf(mxa[3], x3);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 64; j += 4) {
                const float4 c = c4[j >> 2];
                const float cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int t = t0 + j + e;
                  const float x = (t >= lo && t <= hi) ? __uint_as_float(sv[j + e]) * cc[e] : -INFINITY;
                  sv[j + e] = __float_as_uint(x);
                  mxa[e] = fmaxf(mxa[e], x);
                }
              }
            }
          } else if (t0 >= lo && t0 + kGqaPage - 1 <= hi) {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              const float x = __uint_as_float(sv[j]) * a.scale_log2e;
              sv[j] = __float_as_uint(x);
              mxa[j & 3] = fmaxf(mxa[j & 3], x);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              const int t = t0 + j;
              const float x = (t >= lo && t <= hi) ? __uint_as_float(sv[j]) * a.scale_log2e : -INFINITY;
              sv[j] = __float_as_uint(x);
              mxa[j & 3] = fmaxf(mxa[j & 3], x);
            }
          }
          const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
          // lazy rescale: m only moves when a tile exceeds it by more than 2^kTau, so P <= 2^kTau
          // and the accumulator in TMEM is rarely touched
          constexpr float kTau = 7.0f;
          const bool up = mx > m + kTau;
          if (__any_sync(0xffffffffu, up)) {
            const float m_new = up ? mx : m;
            const float alpha = exp2f(m - m_new);
            l *= alpha;
            m = m_new;
            if (i > 0) {
              // the accumulator must be quiescent: P.V of the previous tile has retired
              if (!mbar_wait(&pv_done[(ti - 1) & 1], ((ti - 1) >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGqa); ok = false; break; }
              tc_fence_after();
#pragma unroll 1
              for (int c = 0; c < HD; c += 32) {
                uint32_t o[32];
                tmem_ld32(tm_o + lane_addr + c, o);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                tmem_st16(tm_o + lane_addr + c, o);
                tmem_st16(tm_o + lane_addr + c + 16, o + 16);
              }
              tmem_st_wait();
              tc_fence_before();
            }
          }
          float sa = 0.f, sb = 0.f;
          uint32_t pk[32];
          const float4* d4 = reinterpret_cast<const float4*>(cf + 64);
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            float e[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) e[q] = exp2f(__uint_as_float(sv[j + q]) - m);
            sa += e[0] + e[2]; sb += e[1] + e[3];
            if constexpr (KV8) {
              const float4 d = d4[j >> 2];
              e[0] *= d.x; e[1] *= d.y; e[2] *= d.z; e[3] *= d.w;
            }
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(e[0], e[1]), h1 = __floats2bfloat162_rn(e[2], e[3]);
            pk[j >> 1] = *reinterpret_cast<const uint32_t*>(&h0);
            pk[(j >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&h1);
          }
          l += sa + sb;
          tmem_st16(tm_s + lane_addr + (ti & 1) * 64, pk);
          tmem_st16(tm_s + lane_addr + (ti & 1) * 64 + 16, pk + 16);
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[ti & 1]);
      }
      if (!ok) break;
      // ---- finalize: O / l, written directly (one split) or as a partial with its log-sum-exp
      const uint32_t ti_last = tile_it + w.ntiles - 1;
      if (!mbar_wait(&pv_done[ti_last & 1], (ti_last >> 1) & 1, abort_flag)) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGqa); break; }
      tc_fence_after();
      if (warp_active) {
        const bool row_ok = li < n_valid;
        const int row = w.r0 + li / a.group;
        const int head = w.kvh * a.group + li % a.group;
        const float fin = (l > 0.f ? 1.0f / l : 0.f) * (KV8 ? 0x1p60f : 1.0f);    // e4m3 cache: the accumulator carries 2^-60
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          __syncwarp();
          tmem_ld32(tm_o + lane_addr + c, o);
          tmem_ld_wait();
          if (!row_ok) continue;
          if (w.ns == 1) {
            uint32_t h2[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * fin, __uint_as_float(o[2 * j + 1]) * fin);
              h2[j] = *reinterpret_cast<const uint32_t*>(&v);
            }
            uint4* dst = reinterpret_cast<uint4*>(a.out + (static_cast<size_t>(row) * a.nq + head) * HD + c);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_uint4(h2[4 * q], h2[4 * q + 1], h2[4 * q + 2], h2[4 * q + 3]);
          } else {
            float4* dst = reinterpret_cast<float4*>(a.opart + ((static_cast<size_t>(row) * a.nq + head) * a.max_splits + w.split) * HD + c);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              dst[q] = make_float4(__uint_as_float(o[4 * q]) * fin, __uint_as_float(o[4 * q + 1]) * fin,
                                   __uint_as_float(o[4 * q + 2]) * fin, __uint_as_float(o[4 * q + 3]) * fin);
          }
        }
        if (row_ok && w.ns > 1)
          a.lse[(static_cast<size_t>(row) * a.nq + head) * a.max_splits + w.split] = l > 0.f ? m + log2f(l) : -INFINITY;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
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
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::kTmemCols); }
}

// out[row][head][:] = sum_s 2^(lse_s - gm) opart_s / sum_s 2^(lse_s - gm) for rows that were split.
__global__ void gqa_merge_kernel(const float* opart, const float* lse, const int* row_ns, int nq, int max_splits,
                                 int hd, __nv_bfloat16* out) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int row = blockIdx.x, head = blockIdx.y;
  const int ns = row_ns[row];
  if (ns <= 1) return;
  const size_t base = (static_cast<size_t>(row) * nq + head) * max_splits;
  float gm = -INFINITY;
  for (int s = 0; s < ns; ++s) gm = fmaxf(gm, lse[base + s]);
  if (gm == -INFINITY) gm = 0.f;
  float wsum = 0.f;
  for (int s = 0; s < ns; ++s) wsum += exp2f(lse[base + s] - gm);
  const float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
  for (int c = threadIdx.x; c < hd; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < ns; ++s) acc += exp2f(lse[base + s] - gm) * opart[(base + s) * hd + c];
    out[(static_cast<size_t>(row) * nq + head) * hd + c] = __float2bfloat16(acc * inv);
  }
}

// ---------------------------------------------------------------------------------------------
// One warp per (row, head) of the fused qkv row: optional per-head RMSNorm, RoPE, then q goes to
// q_out[row][head][hd] and k / v go straight into their cache cells.
__global__ void rope_kv_kernel(__nv_bfloat16* q_out, const __nv_bfloat16* qkv, int ld_qkv, __nv_bfloat16* kc,
                               __nv_bfloat16* vc, const __nv_bfloat16* qn, const __nv_bfloat16* kn,
                               const float* rope_tab, const int* pos, const int* seq, const int* page_table,
                               int max_pages, int rows, int nq, int nkv, int hd, int rot, int pair_mode,
                               int plus_one, float eps, __nv_bfloat16* gate_out, float* kv_scale) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  extern __shared__ float rk_smem[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + wib;
  if (item >= static_cast<long long>(rows) * heads) return;
  const int r = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  const int p = pos[r];
  if (p < 0) return;
  float* buf = rk_smem + wib * hd;
  // gated attention: every query head is stored as [Q (hd) | gate (hd)]; K and V follow the 2*hd-wide query heads
  const int qw = gate_out ? 2 * hd : hd;
  const __nv_bfloat16* src = qkv + static_cast<size_t>(r) * ld_qkv +
                             (h < nq ? static_cast<size_t>(h) * qw : static_cast<size_t>(nq) * qw + static_cast<size_t>(h - nq) * hd);
  __nv_bfloat16* dst;
  const __nv_bfloat16* gamma = nullptr;
  const bool is_v = h >= nq + nkv;
  uint8_t* dst8 = nullptr;          // e4m3 cache cell (kv_scale given) and where its scale goes
  float* dst_scale = nullptr;
  if (h < nq) {
    dst = q_out + (static_cast<size_t>(r) * nq + h) * hd;
    gamma = qn;
    if (gate_out)
      for (int i = lane; i < hd / 8; i += 32)
        reinterpret_cast<uint4*>(gate_out + (static_cast<size_t>(r) * nq + h) * hd)[i] = reinterpret_cast<const uint4*>(src + hd)[i];
  } else {
    const int kh = is_v ? h - nq - nkv : h - nq;
    const int page = page_table[static_cast<size_t>(seq[r]) * max_pages + p / kGqaPage];
    const size_t cell = ((static_cast<size_t>(page) * kGqaPage + p % kGqaPage) * nkv + kh) * hd;
    dst = (is_v ? vc : kc) + cell;
    gamma = kn;
    if (kv_scale) {
      dst8 = reinterpret_cast<uint8_t*>(is_v ? vc : kc) + cell;
      dst_scale = kv_scale + (static_cast<size_t>(page) * kGqaPage + p % kGqaPage) * 2 * nkv + (is_v ? nkv : 0) + kh;
      dst = reinterpret_cast<__nv_bfloat16*>(buf);     // never dereferenced as a cache row below
    }
  }
  // e4m3 cell: the finished row (bf16-rounded, as the bf16 cache would hold it) scaled by amax / 448, one scale per cell
  auto store8 = [&]() {
    float amax = 0.f;
    for (int i = lane; i < hd; i += 32) amax = fmaxf(amax, fabsf(buf[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = fmaxf(amax, 1e-12f) / 448.0f, inv = 1.0f / sc;
    for (int i = lane; i < hd; i += 32)
      dst8[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(buf[i] * inv, __NV_SATFINITE, __NV_E4M3));
    if (lane == 0) *dst_scale = sc;
  };
  if (is_v) {
    if (dst8) {
      for (int i = lane; i < hd; i += 32) buf[i] = __bfloat162float(src[i]);
      __syncwarp();
      store8();
      return;
    }
    for (int i = lane; i < hd / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) { const float v = __bfloat162float(src[i]); buf[i] = v; ss += v * v; }
  if (gamma) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rs = rsqrtf(ss / hd + eps);
    __syncwarp();
    // the normalised value is rounded to bf16 before the rotation, as the unfused pair would do
    for (int i = lane; i < hd; i += 32) {
      const float g = __bfloat162float(gamma[i]);
      buf[i] = __bfloat162float(__float2bfloat16(buf[i] * rs * (plus_one ? 1.0f + g : g)));
    }
  }
  __syncwarp();
  const int half = rot / 2;
  const float* tab = rope_tab + static_cast<size_t>(p) * rot;
  if (dst8) {
    // rotate in place (each pair is owned by one lane), rounded to bf16 like the bf16 cache row, then quantise
    for (int i = lane; i < half; i += 32) {
      const int ia = pair_mode ? 2 * i : i, ib = pair_mode ? 2 * i + 1 : i + half;
      const float x = buf[ia], y = buf[ib], c = tab[i], s = tab[half + i];
      buf[ia] = __bfloat162float(__float2bfloat16(x * c - y * s));
      buf[ib] = __bfloat162float(__float2bfloat16(y * c + x * s));
    }
    for (int i = rot + lane; i < hd; i += 32) buf[i] = __bfloat162float(__float2bfloat16(buf[i]));
    __syncwarp();
    store8();
    return;
  }
  for (int i = lane; i < half; i += 32) {
    const int ia = pair_mode ? 2 * i : i, ib = pair_mode ? 2 * i + 1 : i + half;
    const float x = buf[ia], y = buf[ib], c = tab[i], s = tab[half + i];
    dst[ia] = __float2bfloat16(x * c - y * s);
    dst[ib] = __float2bfloat16(y * c + x * s);
  }
  for (int i = rot + lane; i < hd; i += 32) dst[i] = __float2bfloat16(buf[i]);
}

template <int HD>
int launch_gqa(const GqaArgs& a, const void* q, const void* kc, const void* vc, int64_t n_pages, int grid, cudaStream_t stream) {
  using Cfg = GqaCfg<HD, HD>;
  CUtensorMap tq, tk, tv;
  int r = make_tmap_3d(&tq, q, 2, HD, a.nq, a.rows, HD * 2, static_cast<uint64_t>(a.nq) * HD * 2, a.group, 128 / a.group, 128);
  if (r) return 1100 + r;
  r = make_tmap_3d(&tk, kc, 2, HD, a.nkv, static_cast<uint64_t>(n_pages) * kGqaPage, HD * 2, static_cast<uint64_t>(a.nkv) * HD * 2, 1, kGqaPage, 128);
  if (r) return 1200 + r;
  r = make_tmap_3d(&tv, vc, 2, HD, a.nkv, static_cast<uint64_t>(n_pages) * kGqaPage, HD * 2, static_cast<uint64_t>(a.nkv) * HD * 2, 1, kGqaPage, 128);
  if (r) return 1300 + r;
  static DeviceOnce attr;
  if (ensure_smem(attr, gqa_attn_kernel<HD, HD>, Cfg::kSmem) != cudaSuccess) return 3000;
  plow::launch_serial(gqa_attn_kernel<HD, HD>, dim3(grid), dim3(kGqaThreads), Cfg::kSmem, stream, a, tq, tk, tv, tk);
  return 0;
}

// e4m3 cache: kc / vc are bytes [n_pages*64][nkv][HD]; raw tiles of 128 bytes x 64 tokens per load.
template <int HD>
int launch_gqa8(const GqaArgs& a, const void* q, const void* kc, const void* vc, int64_t n_pages, int grid, cudaStream_t stream) {
  using Cfg = GqaCfg<HD, HD, true>;
  CUtensorMap tq, tk, tv;
  int r = make_tmap_3d(&tq, q, 2, HD, a.nq, a.rows, HD * 2, static_cast<uint64_t>(a.nq) * HD * 2, a.group, 128 / a.group, 128);
  if (r) return 1100 + r;
  r = make_tmap_3d(&tk, kc, 1, HD, a.nkv, static_cast<uint64_t>(n_pages) * kGqaPage, HD, static_cast<uint64_t>(a.nkv) * HD, 1, kGqaPage, 128);
  if (r) return 1200 + r;
  r = make_tmap_3d(&tv, vc, 1, HD, a.nkv, static_cast<uint64_t>(n_pages) * kGqaPage, HD, static_cast<uint64_t>(a.nkv) * HD, 1, kGqaPage, 128);
  if (r) return 1300 + r;
  static DeviceOnce attr;
  if (ensure_smem(attr, gqa_attn_kernel<HD, HD, true>, Cfg::kSmem) != cudaSuccess) return 3000;
  plow::launch_serial(gqa_attn_kernel<HD, HD, true>, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmem, stream, a, tq, tk, tv, tk);
  return 0;
}

// Materialised multi-head latent attention (prefill): q [rows][heads][192]; kvb [tokens][heads][256] = per head
// [128 no-position key dims | 128 value dims]; krope [tokens][64] shared by all heads.
int launch_mla_prefill(const GqaArgs& a, const void* q, const void* kvb, const void* krope, int64_t n_tokens, int grid, cudaStream_t stream) {
  using Cfg = GqaCfg<192, 128>;
  CUtensorMap tq, tk, tkr;
  int r = make_tmap_3d(&tq, q, 2, 192, a.nq, a.rows, 192 * 2, static_cast<uint64_t>(a.nq) * 192 * 2, 1, 128, 128);
  if (r) return 1100 + r;
  r = make_tmap_3d(&tk, kvb, 2, 256, a.nkv, static_cast<uint64_t>(n_tokens), 256 * 2, static_cast<uint64_t>(a.nkv) * 256 * 2, 1, kGqaPage, 128);
  if (r) return 1200 + r;
  r = make_tmap_3d(&tkr, krope, 2, 64, 1, static_cast<uint64_t>(n_tokens), 64 * 2, 64 * 2, 1, kGqaPage, 128);
  if (r) return 1300 + r;
  static DeviceOnce attr;
  if (ensure_smem(attr, gqa_attn_kernel<192, 128>, Cfg::kSmem) != cudaSuccess) return 3000;
  plow::launch_serial(gqa_attn_kernel<192, 128>, dim3(grid), dim3(kGqaThreads), Cfg::kSmem, stream, a, tq, tk, tk, tkr);
  return 0;
}

}  // namespace plow

extern "C" {

// q bf16 [rows][nq][hd]; kc / vc bf16 [n_pages][64][nkv][hd]; seq / pos int32 [rows] (pos < 0: inactive row);
// out bf16 [rows][nq*hd].  Scratch from the caller: items (8 ints each, capacity item_cap), n_items (1 int),
// row_ns int32 [rows], opart f32 [rows][nq][max_splits][hd], lse f32 [rows][nq][max_splits].
// kv_scale != null: kc / vc are e4m3 bytes with one f32 scale per (token, kv head) in kv_scale [n_pages][64][2*nkv]
// (k scales, then v scales); head dim 128 only.
int plow_gqa_attention(const void* q, const void* kc, const void* vc, int64_t n_pages, const int* page_table,
                       int max_pages, const int* seq, const int* pos, int rows, int nq, int nkv, int hd, int window,
                       int tiles_per_split, int max_splits, void* items, int item_cap, int* n_items, int* row_ns,
                       float* opart, float* lse, void* out, float softmax_scale, const float* kv_scale, int* status, void* stream_) {
  using namespace plow;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || max_splits <= 0 || tiles_per_split <= 0) return -1;
  const int group = nq / nkv;
  if (group > 128 || (group & (group - 1))) return -2;
  if (hd != 128 && hd != 256) return -3;
  if (kv_scale && hd != 128) return -4;
  const int tq = 128 / group;
  cudaMemsetAsync(n_items, 0, sizeof(int), stream);
  plow::launch_serial(gqa_build_items, dim3((rows + 255) / 256), dim3(256), 0, stream, seq, pos, rows, tq, nkv, window, tiles_per_split, max_splits,
                                                         static_cast<GqaItem*>(items), n_items, row_ns, item_cap, status);
  GqaArgs a;
  a.page_table = page_table; a.pos = pos; a.items = static_cast<const GqaItem*>(items); a.n_items = n_items;
  a.opart = opart; a.lse = lse; a.out = static_cast<__nv_bfloat16*>(out); a.status = status;
  a.rows = rows; a.nq = nq; a.nkv = nkv; a.group = group; a.max_pages = max_pages; a.max_splits = max_splits; a.window = window;
  a.scale_log2e = softmax_scale * 1.4426950408889634f;
  a.kr_slabs = 0; a.v_x0 = 0; a.head_major = 0; a.kv_scale = kv_scale;
  int grid = sm_count();
  if (item_cap < grid) grid = item_cap;
  int r = kv_scale ? launch_gqa8<128>(a, q, kc, vc, n_pages, grid, stream)
          : hd == 128 ? launch_gqa<128>(a, q, kc, vc, n_pages, grid, stream) : launch_gqa<256>(a, q, kc, vc, n_pages, grid, stream);
  if (r) return r;
  if (max_splits > 1)
    plow::launch_serial(gqa_merge_kernel, dim3(rows, nq), dim3(128), 0, stream, opart, lse, row_ns, nq, max_splits, hd, static_cast<__nv_bfloat16*>(out));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// Multi-head latent attention over materialised keys / values (prefill).  q bf16 [rows][heads][192] (rotary part
// already rotated); kvb bf16 [n_tokens][heads][256]; krope bf16 [n_tokens][64]; vpt int32 [n_slots][max_pages]: tile i
// of slot s covers tokens [64 vpt[s][i], 64 vpt[s][i] + 64) of kvb / krope; seq / pos int32 [rows] (pos < 0: the row is
// not attended here); out bf16 [rows][heads*128].  Scratch as for plow_gqa_attention (opart / lse with hd = 128).
int plow_mla_prefill_attention(const void* q, const void* kvb, const void* krope, int64_t n_tokens, const int* vpt, int max_pages,
                               const int* seq, const int* pos, int rows, int heads, int tiles_per_split, int max_splits,
                               void* items, int item_cap, int* n_items, int* row_ns, float* opart, float* lse, void* out,
                               float softmax_scale, int* status, void* stream_) {
  using namespace plow;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0 || heads <= 0 || max_splits <= 0 || tiles_per_split <= 0 || n_tokens <= 0) return -1;
  cudaMemsetAsync(n_items, 0, sizeof(int), stream);
  plow::launch_serial(gqa_build_items, dim3((rows + 255) / 256), dim3(256), 0, stream, seq, pos, rows, 128, heads, 0, tiles_per_split,
                      max_splits, static_cast<GqaItem*>(items), n_items, row_ns, item_cap, status);
  GqaArgs a;
  a.page_table = vpt; a.pos = pos; a.items = static_cast<const GqaItem*>(items); a.n_items = n_items;
  a.opart = opart; a.lse = lse; a.out = static_cast<__nv_bfloat16*>(out); a.status = status;
  a.rows = rows; a.nq = heads; a.nkv = heads; a.group = 1; a.max_pages = max_pages; a.max_splits = max_splits; a.window = 0;
  a.scale_log2e = softmax_scale * 1.4426950408889634f;
  a.kr_slabs = 1; a.v_x0 = 128; a.head_major = max_splits == 1 ? 1 : 0; a.kv_scale = nullptr;
  int grid = sm_count();
  if (item_cap < grid) grid = item_cap;
  int r = launch_mla_prefill(a, q, kvb, krope, n_tokens, grid, stream);
  if (r) return r;
  if (max_splits > 1)
    plow::launch_serial(gqa_merge_kernel, dim3(rows, heads), dim3(128), 0, stream, opart, lse, row_ns, heads, max_splits, 128, static_cast<__nv_bfloat16*>(out));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

// qkv bf16 [rows][ld_qkv] = [q heads | k heads | v heads]; qn / kn: optional per-head RMSNorm weights [hd];
// rope_tab f32 [max_pos][rot] = [cos(rot/2) | sin(rot/2)]; pair_mode 0 = half split, 1 = interleaved.
// kv_scale (optional) f32 [n_pages][64][2*nkv]: kc / vc are then e4m3 byte caches and every written cell gets its scale.
// gate_out (optional) bf16 [rows][nq*hd]: gated attention, query heads are then [Q | gate] pairs of width 2*hd.
int plow_rope_kv(void* q_out, const void* qkv, int ld_qkv, void* kc, void* vc, const void* qn, const void* kn,
                 const float* rope_tab, const int* pos, const int* seq, const int* page_table, int max_pages,
                 int rows, int nq, int nkv, int hd, int rot, int pair_mode, int plus_one, float eps, void* gate_out,
                 float* kv_scale, void* stream_) {
  using namespace plow;
  if (rows <= 0 || hd % 8 || rot > hd || rot % 2) return -1;
  const long long items = static_cast<long long>(rows) * (nq + 2 * nkv);
  const int wpb = 8;
  plow::launch_serial(rope_kv_kernel, dim3(static_cast<unsigned>((items + wpb - 1) / wpb)), dim3(wpb * 32), wpb * hd * sizeof(float), reinterpret_cast<cudaStream_t>(stream_), 
      static_cast<__nv_bfloat16*>(q_out), static_cast<const __nv_bfloat16*>(qkv), ld_qkv, static_cast<__nv_bfloat16*>(kc),
      static_cast<__nv_bfloat16*>(vc), static_cast<const __nv_bfloat16*>(qn), static_cast<const __nv_bfloat16*>(kn),
      rope_tab, pos, seq, page_table, max_pages, rows, nq, nkv, hd, rot, pair_mode, plus_one, eps,
      static_cast<__nv_bfloat16*>(gate_out), kv_scale);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
