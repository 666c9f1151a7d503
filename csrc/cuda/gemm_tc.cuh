// Persistent warp-specialised tcgen05 GEMM for sm_100a.
//
//   y[M, N] = x[M, K] * w[N, K]^T          (both operands K-major, fp32 accumulate in TMEM)
//
// One CTA per SM walks a static tile schedule.  Warp 0 issues TMA loads into a ring of
// 128-byte-swizzled shared-memory stages, one elected thread of warp 1 issues tcgen05.mma
// and commits completion to mbarriers, warps 2-5 read accumulators back with tcgen05.ld and
// run the epilogue.  Variants, all in this one template:
//   * bf16 inputs (kind::f16) or e4m3 inputs with 128x128 weight scales and 1x128 activation
//     scales (kind::f8f6f4).  fp32 block scales cannot be applied by the tensor core, so the
//     fp8 path accumulates one 128-wide K block per TMEM buffer and the epilogue warps fold
//     it into fp32 registers with the block's scale (two-level accumulation) while the MMA
//     warp runs the next block into the other buffer.
//   * SWAP: weights ride the 128 TMEM lanes and tokens the UMMA N dimension (16..128), so
//     small-M decode GEMMs stream weights at full tile efficiency.
//   * grouped (MoE): rows of x are sorted by expert, `grp_off[E+1]` gives each expert's row
//     range and w stacks the experts' matrices; tiles that run past an expert's rows are
//     masked at the store, so no padding of the token buffer is needed.
//   * DUAL: gate and up projections accumulate side by side and the epilogue writes
//     silu(gate) * up, optionally re-quantised to e4m3 with 1x128 scales for the next GEMM.
//
// Parity notes: the reference's prefill GEMM is a 128x128x32 mma.sync/wgmma tile loop with a
// GLU epilogue (runtime/nvidia/op_gemm.cuh:1218-1260, op_gemm_sm90.cuh) and its block-scaled
// fp8 decode GEMM is a swap-AB wgmma kernel with two-level accumulation
// (runtime/nvidia/op_gemm_fp8_block_sm90.cuh:77-91); grouped MoE tiles follow the
// (rowoff, cnt, tile_prefix) table of runtime/nvidia/op_moe.cuh.
#pragma once
#include "ptx.cuh"
#include "tmap.cuh"

namespace plow {

struct GemmArgs {
  const void* x;         // activations [rows, K]
  const void* w;         // weights [E * Nw, K], Nw = dual ? 2N : N
  void* y;               // output [rows, N] bf16 (or f32 when out_f32)
  const float* sx;       // fp8: activation scales, transposed [KB][ld_sx]
  const float* sw;       // fp8: weight scales [(E*Nw)/128][KB]
  const void* residual;  // optional bf16 [rows, N], added before the store
  void* yq;              // optional e4m3 output [rows, N]
  float* syq;            // its scales, transposed [N/128][ld_syq]
  const int* grp_off;    // grouped: [E+1] row offsets into x (device memory)
  const int* tile_prefix;// grouped, non-swap: [E+1] prefix of 128-row tile counts
  int* status;           // device status word (0 = ok)
  // optional arrival gate (expert-parallel dispatch): rows of x are written by peer GPUs; the
  // kernel starts reading them once *wait_ctr >= *wait_epoch * wait_mult (bounded wait)
  // split-K (dense swap mode): each tile is cut into `splits` K ranges run by different CTAs;
  // partials go to `ws` (fp32, [tile][split][128 lanes][cols]) and the CTA that arrives last on the
  // tile's counter sums them in split order and runs the epilogue (no CTA ever waits for another)
  float* ws;
  int* ws_ctr;
  int splits;
  // stream scheduling (swap mode): the linear (tile, K block) space is cut into equal contiguous ranges, one per
  // CTA, so every SM streams the same number of weight bytes whatever the tile count.  A tile whose K range is
  // shared is finished by the CTA that holds its first K blocks (the last thing that CTA does); the CTAs holding
  // the later K blocks run them first thing and publish fp32 partials to `ws` ([CTA][column][128 lanes]) with a
  // flag in `ws_ctr` ([CTA] x 32 ints), so the finishing CTA practically never waits.
  int stream;
  // fused all-reduce (tensor-parallel row-parallel GEMM, swap mode): this rank's partial tiles are
  // reduced through peer memory from inside the kernel, see the `ar_*` phase at the end of the kernel
  uint8_t* ar_peer[8];    // symmetric region of every rank (peer-mapped), NULL world = off
  unsigned long long ar_part_ofs, ar_flag_ofs, ar_done_ofs, ar_y_ofs;
  uint32_t* ar_epoch;     // device words: [0] launch counter, [1] arrivals on `done` seen so far (two-shot), [2] CTAs through (one-shot)
  int ar_world, ar_me;
  int ar_oneshot;          // 1: every rank pushes its partial to all ranks and reduces locally (decode sizes)
                           // 2: two-shot through NVSwitch multicast: multimem.ld_reduce by the tile's owner, multimem.st of the result
  uint8_t* ar_mc;          // multicast mapping of the symmetric region (mode 2)
  unsigned long long ar_tdone_ofs;   // mode 2: u32 [tiles] epoch word per tile, written to every rank when the tile has landed
  unsigned long long ar_half_bytes;   // one-shot: size of one parity half of the partial area
  long long* trace;       // clock64() phase stamps of CTA 0; only read by builds with -DPLOW_DEVICE_TRACE
  const uint32_t* wait_ctr;
  const uint32_t* wait_epoch;
  uint32_t wait_mult;
  uint32_t wait_deadline_ms;
  int M;                 // rows of x (upper bound when grouped)
  int N;                 // output features per expert
  int K;
  int ldy;               // elements
  int ld_sx;
  int ld_syq;
  int E;                 // 0 = dense
  int out_f32;
  float out_scale;       // multiplies the result (1.0 = none)
};

constexpr int kGemmThreads = 192;
constexpr int kStageBytesP = 128 * 128;

template <int BN, bool DUAL, bool SWAP, bool FP8 = false>
struct GemmCfg {
  static constexpr int kPT = (DUAL && SWAP) ? 2 : 1;    // 128-row tiles per stage
  static constexpr int kQT = (DUAL && !SWAP) ? 2 : 1;   // BN-row tiles per stage
  static constexpr int kStageBytes = kPT * kStageBytesP + kQT * BN * 128;
  static constexpr int kAccCols = BN * (DUAL ? 2 : 1);
  // Epilogue warps.  The block-scaled kernels at large M (tokens on the lanes) are bound by the promotion of the
  // per-K-block partials (one warp per scheduler, a latency chain of TMEM load -> wait -> FMAs kept the tensor pipe 45 %
  // busy): there two warps share each TMEM lane quarter and split the columns, so each sub-partition has two chains
  // to interleave and half the work per chain.
  static constexpr int kEpiWarps = (FP8 && !SWAP) ? 8 : 4;
  static constexpr int kHalves = kEpiWarps / 4;
  static constexpr int kCH = BN / kHalves;              // columns of each BN-wide block a warp owns
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  // accumulator buffers in TMEM: two for bf16 (tile i+1 runs while tile i drains); for fp8 as many K-block
  // partials as TMEM holds (up to eight), so the MMA warp keeps consuming stages while the promotion warps are
  // away writing a finished tile (measured: the end of a tile takes the four warps 2.5-9 us at decode shapes,
  // which four buffers could not cover: the tensor pipe and with it the weight stream stalled at every tile)
  static constexpr int kNBuf = !FP8 ? 2 : (8 * kAccCols <= 512 ? 8 : (4 * kAccCols <= 512 ? 4 : 2));
  static constexpr int kTmemCols =
      kNBuf * kAccCols <= 32 ? 32 : kNBuf * kAccCols <= 64 ? 64 : kNBuf * kAccCols <= 128 ? 128
                                                   : kNBuf * kAccCols <= 256 ? 256 : 512;
  static constexpr int kStages =
      (196 * 1024 / kStageBytes) > 10 ? 10 : (196 * 1024 / kStageBytes);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 2048 /*bars+scratch*/ + 4096 /*scale factors*/ +
                                    8192 /*two transpose buffers of the swap-mode store*/;
  static_assert(kNBuf * kAccCols <= 512, "accumulators exceed TMEM");
  static_assert(kStages >= 2, "tile too large for shared memory");
};

struct Tile {
  int tok0, tok_end;  // token rows (TMA coordinate, exclusive valid end)
  int wrow0;          // first weight row (absolute, in the stacked matrix)
  int feat0;          // first output feature of the tile within N
  int kb0, kb1;       // K-block range of this work item
  int tile_id, ks;    // split-K: output tile index and split index
  int contrib;        // stream scheduling: this piece only publishes its partial sums
  int n_follow;       // stream scheduling: CTAs after this one that hold later K blocks of the tile
};

template <int BN, bool DUAL, bool SWAP>
struct TileSched {
  const GemmArgs& a;
  int item, sub;
  int n_wt;  // weight tiles per expert
  int KB;
  // stream scheduling
  long long s_pos, s_hi;     // next iteration to hand out / end of this CTA's range (units of K blocks)
  long long s_per;           // iterations per CTA
  int s_e, s_pre;            // grouped: running expert and the number of work units before it
  __device__ int subtiles(int e) const { return (a.grp_off[e + 1] - a.grp_off[e] + BN - 1) / BN; }
  __device__ TileSched(const GemmArgs& a_, int KB_) : a(a_), item(blockIdx.x), sub(0), KB(KB_) {
    n_wt = SWAP ? (a.N + 127) / 128 : (a.N + BN - 1) / BN;
    s_pos = s_hi = 0; s_per = 1; s_e = 0; s_pre = 0;
    if (SWAP && a.stream) {
      long long units;
      if (a.E == 0) {
        units = static_cast<long long>((a.M + BN - 1) / BN) * n_wt;
      } else {
        units = 0;
        for (int e = 0; e < a.E; ++e) units += static_cast<long long>(subtiles(e)) * n_wt;
      }
      const long long iters = units * KB;
      s_per = (iters + gridDim.x - 1) / gridDim.x;
      if (s_per < 1) s_per = 1;
      s_pos = static_cast<long long>(blockIdx.x) * s_per;
      if (s_pos > iters) s_pos = iters;
      s_hi = s_pos + s_per < iters ? s_pos + s_per : iters;
    }
  }
  __device__ bool next_stream(Tile& t) {
    if (s_pos >= s_hi) return false;
    const int nw_per = DUAL ? 2 * a.N : a.N;
    const long long u = s_pos / KB;
    const long long u0 = u * KB;
    t.kb0 = static_cast<int>(s_pos - u0);
    t.kb1 = s_hi - u0 < KB ? static_cast<int>(s_hi - u0) : KB;
    s_pos = u0 + t.kb1;
    t.contrib = t.kb0 > 0;
    t.n_follow = 0;
    if (t.kb0 == 0 && t.kb1 < KB) t.n_follow = static_cast<int>((u0 + KB - 1) / s_per) - static_cast<int>(blockIdx.x);
    t.tile_id = 0; t.ks = 0;
    if (a.E == 0) {
      const int wt = static_cast<int>(u % n_wt), tt = static_cast<int>(u / n_wt);
      t.tok0 = tt * BN; t.tok_end = a.M; t.feat0 = wt * 128; t.wrow0 = t.feat0;
      return true;
    }
    // grouped: units are ordered expert, weight tile, token sub-tile; the running expert only moves forward
    int st = subtiles(s_e);
    while (u >= s_pre + static_cast<long long>(st) * n_wt) { s_pre += st * n_wt; ++s_e; st = subtiles(s_e); }
    const int local = static_cast<int>(u - s_pre);
    const int wt = local / st, sb = local % st;
    t.tok0 = a.grp_off[s_e] + sb * BN; t.tok_end = a.grp_off[s_e + 1];
    t.feat0 = wt * 128; t.wrow0 = s_e * nw_per + wt * 128;
    return true;
  }
  __device__ bool next(Tile& t) {
    const int nw_per = DUAL ? 2 * a.N : a.N;
    t.kb0 = 0; t.kb1 = KB; t.tile_id = 0; t.ks = 0; t.contrib = 0; t.n_follow = 0;
    if (SWAP && a.stream) return next_stream(t);
    if (a.E == 0) {
      const int n_tt = SWAP ? (a.M + BN - 1) / BN : (a.M + 127) / 128;
      const int S = (SWAP && a.splits > 1) ? a.splits : 1;
      // token tile fastest when SWAP (few token tiles), weight-tile-major otherwise so CTAs
      // running at the same time share one weight tile in L2
      if (item >= n_tt * n_wt * S) return false;
      int tt, wt;
      int tile = item;
      if (S > 1) {
        tile = item / S;
        t.ks = item % S;
        t.kb0 = t.ks * KB / S;
        t.kb1 = (t.ks + 1) * KB / S;
        t.tile_id = tile;
      }
      if (SWAP) { wt = tile % n_wt; tt = tile / n_wt; } else { tt = tile % n_tt; wt = tile / n_tt; }
      t.tok0 = tt * (SWAP ? BN : 128);
      t.tok_end = a.M;
      t.feat0 = wt * (SWAP ? 128 : BN);
      t.wrow0 = t.feat0;
      item += gridDim.x;
      return true;
    }
    if (SWAP) {
      while (true) {
        if (item >= a.E * n_wt) return false;
        const int e = item / n_wt, wt = item % n_wt;
        const int r0 = a.grp_off[e], r1 = a.grp_off[e + 1];
        const int tok = r0 + sub * BN;
        if (tok < r1) {
          t.tok0 = tok; t.tok_end = r1; t.feat0 = wt * 128; t.wrow0 = e * nw_per + wt * 128;
          ++sub;
          return true;
        }
        sub = 0;
        item += gridDim.x;
      }
    } else {
      // Expert-major order: the CTAs running at one time work on one or two experts, so an expert's weights are
      // read from HBM once and its token rows (a few MB) stay in L2 across the weight tiles.  (With the token tile
      // fastest over all experts, every wave of CTAs re-read the whole activation matrix, which at prefill sizes is
      // larger than L2.)  Within an expert the token tile is fastest: neighbours share one weight tile.
      const int n_mt = a.tile_prefix[a.E];
      if (item >= n_mt * n_wt) return false;
      int lo = 0, hi = a.E;  // largest e with tile_prefix[e] * n_wt <= item
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (a.tile_prefix[mid] * n_wt <= item) lo = mid; else hi = mid;
      }
      const int e = lo;
      const int st = a.tile_prefix[e + 1] - a.tile_prefix[e];
      const int local = item - a.tile_prefix[e] * n_wt;
      const int mt = local % st, wt = local / st;
      t.tok0 = a.grp_off[e] + mt * 128;
      t.tok_end = a.grp_off[e + 1];
      t.feat0 = wt * BN;
      t.wrow0 = e * nw_per + wt * BN;
      item += gridDim.x;
      return true;
    }
  }
};

// silu with the approximate reciprocal (2 ulp): the exact division cost the epilogue warps ~350 clocks per value
__device__ __forceinline__ float silu_f(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

template <int BN, bool FP8, bool DUAL, bool SWAP>
__global__ void __launch_bounds__((GemmCfg<BN, DUAL, SWAP, FP8>::kThreads), 1)
gemm_tc_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tm_x,
               const __grid_constant__ CUtensorMap tm_w) {
  using Cfg = GemmCfg<BN, DUAL, SWAP, FP8>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kAccCols = Cfg::kAccCols;
  constexpr int kNBuf = Cfg::kNBuf;
  constexpr int kEpiWarps = Cfg::kEpiWarps;
  constexpr int kCH = Cfg::kCH;
  constexpr int kKElems = FP8 ? 128 : 64;  // K elements per 128-byte stage row
  constexpr int kUmmaK = FP8 ? 32 : 16;
  constexpr int kUmmaN = SWAP ? BN : (DUAL ? 2 * BN : BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* ctrl = smem + kStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);        // [kStages]
  uint64_t* empty_bar = full_bar + kStages;                      // [kStages]
  uint64_t* acc_full = empty_bar + kStages;                      // [kNBuf]
  uint64_t* acc_empty = acc_full + kNBuf;                        // [kNBuf]
  uint64_t* drain_bar = acc_empty + kNBuf;                       // [1]
  uint64_t* xchg_bar = drain_bar + 1;                            // [2] epilogue-warp exchange
  uint64_t* pair_bar = xchg_bar + 2;                             // [4] the two warps of a lane quarter (8-warp epilogue)
  uint64_t* gate_bar = pair_bar + 4;                             // [1] producer -> epilogue warps: the arrival gate is open
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(gate_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* never_flag = abort_flag + 1;                     // stays 0
  float* red_scratch = reinterpret_cast<float*>(ctrl + 512);     // [2][4][16] quant amax exchange (+ split-K flag)
  float* fac_smem = reinterpret_cast<float*>(ctrl + 2048);       // [4 warps][256] fp8 block-scale factors
  uint8_t* tr_smem = ctrl + 2048 + 4096;                         // [2][4 KiB] token-major staging of a 128-feature x 16-token chunk

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int KB = (a.K + kKElems - 1) / kKElems;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < kNBuf; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kEpiWarps); }
    mbar_init(drain_bar, 1);
    mbar_init(&xchg_bar[0], kEpiWarps);
    mbar_init(&xchg_bar[1], kEpiWarps);
    for (int q = 0; q < 4; ++q) mbar_init(&pair_bar[q], 2);
    mbar_init(gate_bar, 1);
    *abort_flag = 0;
    *never_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const CUtensorMap* tm_p = SWAP ? &tm_w : &tm_x;  // operand on the 128 TMEM lanes
  const CUtensorMap* tm_q = SWAP ? &tm_x : &tm_w;  // operand on the UMMA N dimension

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      bool ok = true;
      // Dense swap mode: the weights ride the lanes and nothing on the device ever writes them, so the weight
      // halves of the first stages are requested before the dependency wait and stream in while the producing
      // kernel is still finishing; the activation halves of those stages follow right after the wait.
      const bool early = SWAP && a.E == 0;
      uint32_t npre = 0;
      auto run = [&](int phase) {
        TileSched<BN, DUAL, SWAP> sched(a, KB);
        Tile t;
        uint32_t it = 0;
        while (ok && sched.next(t)) {
          const int p_row = SWAP ? t.wrow0 : t.tok0;
          const int q_row = SWAP ? t.tok0 : t.wrow0;
          for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
            if (phase == 0 && it >= static_cast<uint32_t>(kStages)) return;
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            uint8_t* st = smem + s * Cfg::kStageBytes;
            const int kx = kb * kKElems;
            if (phase == 0 || it >= npre) {
              if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_STAGE_WAIT | kTagGemm); ok = false; break;
              }
              PLOW_TRACE(if (a.trace && blockIdx.x == 0 && it < 64) a.trace[it * 8 + 6] = clock64();)
              mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
              tma_load_2d(st, tm_p, kx, p_row, &full_bar[s]);
              if (DUAL && SWAP) tma_load_2d(st + kStageBytesP, tm_p, kx, p_row + a.N, &full_bar[s]);
              if (phase == 0) ++npre;
            }
            if (phase == 1) {
              uint8_t* sq = st + Cfg::kPT * kStageBytesP;
              tma_load_2d(sq, tm_q, kx, q_row, &full_bar[s]);
              if (DUAL && !SWAP) tma_load_2d(sq + BN * 128, tm_q, kx, q_row + a.N, &full_bar[s]);
            }
          }
        }
      };
      if (early) run(0);
      pdl_wait();
      if (a.wait_ctr) {
        // peers write the token rows with generic stores; after the acquire the async proxy (TMA)
        // must be ordered behind it too
        const uint32_t target = *a.wait_epoch * a.wait_mult;
        const unsigned long long t0 = globaltimer_ns();
        PLOW_TRACE(if (a.trace && blockIdx.x == 0) { a.trace[7] = static_cast<long long>(t0); a.trace[23] = ld_acquire_sys(a.wait_ctr); a.trace[31] = target; })
        while (ld_acquire_sys(a.wait_ctr) < target) {
          if (globaltimer_ns() - t0 > static_cast<unsigned long long>(a.wait_deadline_ms) * 1000000ull) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagGemm); ok = false; break;
          }
          __nanosleep(256);
        }
        PLOW_TRACE(if (a.trace && blockIdx.x == 0) a.trace[15] = static_cast<long long>(globaltimer_ns());)
        fence_proxy_async_all();
        mbar_arrive(gate_bar);      // the epilogue warps wait on this instead of polling the counter themselves
      }
      if (ok) run(1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      // grouped mode: the tile walk below reads grp_off / tile_prefix, which an earlier kernel of the step wrote
      // (a dense walk depends on the launch arguments only and needs no wait)
      if (a.E > 0) pdl_wait();
      TileSched<BN, DUAL, SWAP> sched(a, KB);
      Tile t;
      const uint32_t idesc = umma_idesc(128, kUmmaN, FP8 ? 0u : 1u, FP8 ? 0u : 1u);
      uint32_t it = 0;      // stage counter
      uint32_t accit = 0;   // accumulator-buffer counter (per tile for bf16, per K block for fp8)
      bool ok = true;
      while (ok && sched.next(t)) {
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          PLOW_TRACE(const bool tr = a.trace && blockIdx.x == 0 && it < 64;)
          PLOW_TRACE(if (tr) a.trace[it * 8 + 0] = clock64();)
          if (FP8 || kb == t.kb0) {
            const int b = accit % kNBuf;
            if (!mbar_wait(&acc_empty[b], ((accit / kNBuf) & 1) ^ 1, abort_flag)) {
              *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_FREE_WAIT | kTagGemm); ok = false; break;
            }
          }
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMA_WAIT | kTagGemm); ok = false; break;
          }
          tc_fence_after();
          PLOW_TRACE(if (tr) a.trace[it * 8 + 1] = clock64();)
          const int b = accit % kNBuf;
          const uint32_t d0 = tmem_base + b * kAccCols;
          const uint32_t sp = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t sq = sp + Cfg::kPT * kStageBytesP;
          const uint64_t pdesc = umma_desc_k128(sp);
          const uint64_t qdesc = umma_desc_k128(sq);
#pragma unroll
          for (int k4 = 0; k4 < 128 / (kUmmaK * (FP8 ? 1 : 2)); ++k4) {
            const uint32_t acc = FP8 ? (k4 > 0) : (kb > t.kb0 || k4 > 0);
            const uint64_t adv = static_cast<uint64_t>(k4 * 2);  // 32 bytes >> 4
            if (FP8) {
              tc_mma_f8(d0, pdesc + adv, qdesc + adv, idesc, acc);
              if (DUAL && SWAP)
                tc_mma_f8(d0 + BN, umma_desc_k128(sp + kStageBytesP) + adv, qdesc + adv, idesc, acc);
            } else {
              tc_mma_f16(d0, pdesc + adv, qdesc + adv, idesc, acc);
              if (DUAL && SWAP)
                tc_mma_f16(d0 + BN, umma_desc_k128(sp + kStageBytesP) + adv, qdesc + adv, idesc, acc);
            }
          }
          tc_commit(&empty_bar[s]);
          if (FP8 || kb == t.kb1 - 1) { tc_commit(&acc_full[accit % kNBuf]); ++accit; }
          PLOW_TRACE(if (tr) a.trace[it * 8 + 2] = clock64();)
        }
      }
      if (!ok) {  // drain whatever was issued before giving up
        tc_commit(drain_bar);
        mbar_wait(drain_bar, 0, never_flag);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5)
    pdl_wait();    // activation scales, residual, workspace counters and the epoch word below come from earlier kernels
    const uint32_t ar_ep = a.ar_world > 1 ? *a.ar_epoch + 1 : 0;   // this launch's all-reduce epoch
    if (a.wait_ctr) {
      // expert-parallel dispatch: the activation scales these warps prefetch are written by peer GPUs together with
      // the rows, so they too start only once everything has landed.  Only the producer thread polls the arrival
      // counter (one poller per CTA: the polled line is also the target of the peers' remote adds, and five pollers
      // per CTA on 148 CTAs kept that line busy); it opens this barrier when the gate is through.
      if (!mbar_wait(gate_bar, 0, abort_flag)) { /* the producer gave up (status recorded there) or the wait ran out */ }
    }
    const int lq = warp & 3;               // TMEM lane quarter this warp may read
    const int li = lq * 32 + lane;         // lane (row of D) owned by this thread
    const int half = (warp - 2) >> 2;      // which kCH columns of every BN-wide block this warp owns (0 with four warps)
    const int hc0 = half * kCH;
    const uint32_t lane_addr = static_cast<uint32_t>(lq * 32) << 16;
    TileSched<BN, DUAL, SWAP> sched(a, KB);
    Tile t;
    uint32_t accit = 0;
    uint32_t xchg_it = 0;
    uint32_t yq_it = 0;
    bool ok = true;
    constexpr int kAccRegs = FP8 ? kAccCols / Cfg::kHalves : 1;
    float acc[kAccRegs];
    const __nv_bfloat16* resid = reinterpret_cast<const __nv_bfloat16*>(a.residual);
    // The arrival gate is polled by the producer thread only: the epilogue warps touch the peers' rows
    // (their scales) after an accumulator-full barrier, which is ordered behind the producer's acquire.
    PLOW_TRACE(int tile_no = 0;)
    while (ok && sched.next(t)) {
      PLOW_TRACE(const bool trt = a.trace && blockIdx.x == 0 && li == 0 && tile_no < 2; if (trt) a.trace[(71 + tile_no) * 8 + 6] = clock64(); ++tile_no;)
      const int tok_i = t.tok0 + li;       // non-swap: this thread's token
      const int feat_i = t.feat0 + li;     // swap: this thread's feature
      if constexpr (FP8) {
#pragma unroll
        for (int i = 0; i < kAccRegs; ++i) acc[i] = 0.f;
        const int wblk_g = (t.wrow0 + hc0) >> 7;            // a 256-wide tile spans two 128-row scale blocks
        const int wblk_u = (t.wrow0 + hc0 + a.N) >> 7;
        // Scales are fetched two K blocks ahead so their latency hides behind the wait for
        // the partial.  SWAP: lane l fetches the activation scales of tokens tok0 + l + 32 i; per
        // K block the warp stages the BN combined factors (activation x weight scale) in its own
        // slice of shared memory and every lane reads them back as broadcast float4s.  Otherwise
        // each thread owns one token and needs a single factor.
        constexpr int kNS = SWAP ? (BN + 31) / 32 : 1;
        struct Sc { float sa[kNS]; float wg, wu; };
        auto fetch = [&](int kb, Sc& o) {
          if (kb >= KB) return;
          const float* sxr = a.sx + static_cast<size_t>(kb) * a.ld_sx;
#pragma unroll
          for (int i = 0; i < kNS; ++i)
            o.sa[i] = sxr[min(SWAP ? t.tok0 + i * 32 + lane : tok_i, a.M - 1)];
          o.wg = a.sw[static_cast<size_t>(wblk_g) * KB + kb];
          if constexpr (DUAL) o.wu = a.sw[static_cast<size_t>(wblk_u) * KB + kb];
        };
        float* fw = fac_smem + (warp - 2) * 256;   // [gate BN | up BN] factors of this warp
        Sc s0, s1, s2;
        fetch(t.kb0, s0);
        fetch(t.kb0 + 1, s1);
        PLOW_TRACE(if (trt) a.trace[(70 + tile_no) * 8 + 7] = clock64();)
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++accit) {
          fetch(kb + 2, s2);
          if constexpr (SWAP) {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < kNS; ++i) {
              fw[i * 32 + lane] = s0.sa[i] * s0.wg;
              if constexpr (DUAL) fw[128 + i * 32 + lane] = s0.sa[i] * s0.wu;
            }
            __syncwarp();
          }
          const int b = accit % kNBuf;
          PLOW_TRACE(const bool tre = a.trace && blockIdx.x == 0 && warp == 2 && lane == 0 && accit < 64;)
          PLOW_TRACE(if (tre) a.trace[accit * 8 + 3] = clock64();)
          if (!mbar_wait(&acc_full[b], (accit / kNBuf) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
          }
          tc_fence_after();
          PLOW_TRACE(if (tre) a.trace[accit * 8 + 4] = clock64();)
          const uint32_t tb = tmem_base + lane_addr + b * kAccCols + hc0;
          // acc index -> TMEM column: the warp's kCH columns of the gate block, then (dual) of the up block
#pragma unroll
          for (int c = 0; c < kAccRegs; c += 64) {
            // up to 64 columns per batch: all loads in flight, one wait
            uint32_t v[64];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (c + q * 16 < kAccRegs) tmem_ld16(tb + ((c + q * 16) / kCH) * BN + (c + q * 16) % kCH, v + q * 16);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (c + q * 16 < kAccRegs) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                  const int col = c + q * 16 + j;
                  float4 f;
                  if constexpr (SWAP) {
                    f = *reinterpret_cast<const float4*>(fw + (col < BN ? col : 128 + col - BN));
                  } else {
                    const float fs = s0.sa[0] * ((DUAL && col >= kCH) ? s0.wu : s0.wg);
                    f = make_float4(fs, fs, fs, fs);
                  }
                  acc[col] = fmaf(__uint_as_float(v[q * 16 + j]), f.x, acc[col]);
                  acc[col + 1] = fmaf(__uint_as_float(v[q * 16 + j + 1]), f.y, acc[col + 1]);
                  acc[col + 2] = fmaf(__uint_as_float(v[q * 16 + j + 2]), f.z, acc[col + 2]);
                  acc[col + 3] = fmaf(__uint_as_float(v[q * 16 + j + 3]), f.w, acc[col + 3]);
                }
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[b]);
          PLOW_TRACE(if (tre) a.trace[accit * 8 + 5] = clock64();)
          s0 = s1;
          s1 = s2;
        }
        if (!ok) break;
      } else {
        const int b = accit & 1;
        if (!mbar_wait(&acc_full[b], (accit >> 1) & 1, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
        }
        tc_fence_after();
      }
      const uint32_t tb = tmem_base + lane_addr + (accit & 1) * kAccCols;
      // raw accumulator columns [c, c + 16) of the kAccCols (gate | up) columns
      auto raw16 = [&](int c, float* r) {
        if constexpr (FP8) {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = acc[c + j];
        } else {
          uint32_t g[16];
          tmem_ld16(tb + c, g);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = __uint_as_float(g[j]);
        }
      };
      // stream scheduling: a piece that does not hold the first K blocks of its tile only publishes its partial
      // sums and moves on; the piece that does hold them adds the followers' partials before the epilogue.
      const float* fix = nullptr;     // partials of the CTAs that follow, [follower][column][128 lanes]
      int fix_n = 0;
      bool piece_done = false;
      if constexpr (SWAP) {
        if (a.stream && t.contrib) {
          float* wp = a.ws + static_cast<size_t>(blockIdx.x) * kAccCols * 128 + li;
#pragma unroll
          for (int c = 0; c < kAccCols; c += 16) {
            float r[16];
            raw16(c, r);
#pragma unroll
            for (int j = 0; j < 16; ++j) wp[static_cast<size_t>(c + j) * 128] = r[j];
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
          }
          ++xchg_it;
          if (li == 0) red_add_release_gpu(reinterpret_cast<uint32_t*>(a.ws_ctr) + blockIdx.x * 32, 1u);
          piece_done = true;
        } else if (a.stream && t.n_follow > 0) {
          if (lane == 0) {
            const unsigned long long t0 = globaltimer_ns();
            for (int f = 1; f <= t.n_follow; ++f) {
              const uint32_t* flag = reinterpret_cast<const uint32_t*>(a.ws_ctr) + (blockIdx.x + f) * 32;
              while (ld_acquire_gpu(flag) == 0u) {
                if (*abort_flag || globaltimer_ns() - t0 > kWaitDeadlineNs) {
                  *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_GRID_WAIT | kTagGemm); break;
                }
                __nanosleep(32);
              }
            }
          }
          __syncwarp();
          if (*abort_flag) { ok = false; break; }
          fix = a.ws + static_cast<size_t>(blockIdx.x + 1) * kAccCols * 128 + li;
          fix_n = t.n_follow;
        }
      }
      // split-K: publish this CTA's partial, wait (bounded) until the tile's other splits have
      // published theirs, then reduce and finish only this CTA's share of the token columns, so the
      // reduction traffic is spread over all the CTAs of the tile.  All tiles x splits CTAs are
      // resident at once (the launcher keeps the grid within one CTA per SM).
      int col_lo = 0, col_hi = BN;
      const float* ws_tile = nullptr;
      if constexpr (SWAP) {
        if (a.splits > 1 && a.E == 0) {
          PLOW_TRACE(const bool trs = a.trace && blockIdx.x == 0 && li == 0;)
          PLOW_TRACE(if (trs) a.trace[60 * 8 + 0] = clock64();)
          // workspace layout [tile][split][column][128 lanes]: a warp's 32 lanes touch 128 contiguous bytes
          float* wp = a.ws + (static_cast<size_t>(t.tile_id) * a.splits + t.ks) * kAccCols * 128 + li;
#pragma unroll
          for (int c = 0; c < kAccCols; c += 16) {
            float r[16];
            raw16(c, r);
#pragma unroll
            for (int j = 0; j < 16; ++j) wp[static_cast<size_t>(c + j) * 128] = r[j];
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
          }
          ++xchg_it;
          uint32_t* ctr = reinterpret_cast<uint32_t*>(a.ws_ctr) + t.tile_id * 32;   // one counter per 128-byte line
          PLOW_TRACE(if (trs) a.trace[60 * 8 + 1] = clock64();)
          if (li == 0) red_add_release_gpu(ctr, 1u);
          if (lane == 0) {
            const unsigned long long t0 = globaltimer_ns();
            while (ld_acquire_gpu(ctr) < static_cast<uint32_t>(a.splits)) {
              if (*abort_flag || globaltimer_ns() - t0 > kWaitDeadlineNs) {
                *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_GRID_WAIT | kTagGemm); break;
              }
              __nanosleep(32);
            }
          }
          __syncwarp();
          PLOW_TRACE(if (trs) a.trace[60 * 8 + 2] = clock64();)
          if (*abort_flag) { ok = false; break; }
          col_lo = t.ks * BN / a.splits;
          col_hi = (t.ks + 1) * BN / a.splits;
          ws_tile = a.ws + static_cast<size_t>(t.tile_id) * a.splits * kAccCols * 128 + li;
        }
      }
      // result of 16 columns starting at c (gate/up folded, out_scale applied)
      auto load16 = [&](int c, float* r) {
        if (ws_tile) {
          // partials are summed in split order (deterministic).  The 16 (or 32) loads of one split are
          // issued together before any add, so a split costs one L2 round trip, not one per column.
          float g[16], u[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) { g[j] = 0.f; u[j] = 0.f; }
          for (int ks = 0; ks < a.splits; ++ks) {
            const float* p = ws_tile + static_cast<size_t>(ks) * kAccCols * 128;
            float v[16], w2[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const bool in = c + j >= col_lo && c + j < col_hi;
              v[j] = in ? __ldcg(p + static_cast<size_t>(c + j) * 128) : 0.f;
              if constexpr (DUAL) w2[j] = in ? __ldcg(p + static_cast<size_t>(BN + c + j) * 128) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += v[j];
              if constexpr (DUAL) u[j] += w2[j];
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = DUAL ? silu_f(g[j]) * u[j] : g[j];
        } else if (fix_n > 0) {
          // this piece's own sums plus the followers' partials (follower order: deterministic)
          float g[16], u[16];
          raw16(c, g);
          if constexpr (DUAL) raw16(BN + c, u);
          for (int f = 0; f < fix_n; ++f) {
            const float* p = fix + static_cast<size_t>(f) * kAccCols * 128;
            float v[16], w2[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] = __ldcg(p + static_cast<size_t>(c + j) * 128);
              if constexpr (DUAL) w2[j] = __ldcg(p + static_cast<size_t>(BN + c + j) * 128);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += v[j];
              if constexpr (DUAL) u[j] += w2[j];
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = DUAL ? silu_f(g[j]) * u[j] : g[j];
        } else if constexpr (FP8) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if constexpr (DUAL) r[j] = silu_f(acc[c + j]) * acc[kCH + c + j];
            else r[j] = acc[c + j];
          }
        } else {
          uint32_t g[16];
          tmem_ld16(tb + c, g);
          if constexpr (DUAL) {
            uint32_t u[16];
            tmem_ld16(tb + BN + c, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = __uint_as_float(g[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] *= a.out_scale;
      };

      PLOW_TRACE(if (trt) a.trace[(70 + tile_no) * 8 + 0] = clock64();)
      if constexpr (SWAP) {
       if (!piece_done) {
        // thread = feature, columns = tokens
        const bool fok = feat_i < a.N;
#pragma unroll
        for (int c = 0; c < BN; c += 16) {
          if (t.tok0 + c >= t.tok_end) break;   // uniform across the CTA
          if (c + 16 <= col_lo || c >= col_hi) continue;
          float r[16];
          load16(c, r);
          PLOW_TRACE(if (trt && c == 0) a.trace[(70 + tile_no) * 8 + 1] = clock64();)
          if (a.ar_world > 1) {
            // fused all-reduce, phase 1: this rank's partial of the tile, bf16, [tile][feature][token]
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
              pk[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            if (a.ar_oneshot == 1) {
              // one-shot: the partial goes straight into every rank's [parity][tile][source rank][feature][token] slot
              const size_t po = a.ar_part_ofs + (ar_ep & 1) * a.ar_half_bytes +
                                (static_cast<size_t>(((t.feat0 >> 7) * a.ar_world + a.ar_me) * 128 + li) * BN + c) * 2;
              for (int p = 0; p < a.ar_world; ++p) {
                uint4* pp = reinterpret_cast<uint4*>(a.ar_peer[p] + po);
                pp[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                pp[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              }
              continue;
            }
            uint4* pp = reinterpret_cast<uint4*>(a.ar_peer[a.ar_me] + a.ar_part_ofs +
                                                 (static_cast<size_t>((t.feat0 >> 7) * 128 + li) * BN + c) * 2);
            pp[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            pp[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            continue;
          }
          // A thread holds one feature of 16 tokens, so a direct store is 16 scattered 2-byte writes per thread
          // (measured ~2300 clocks per chunk, which stalled the weight stream at every tile).  The common case goes
          // through shared memory instead: the chunk is laid out token-major and leaves as 16-byte row segments.
          const bool whole = !ws_tile && t.feat0 + 128 <= a.N && (a.ldy & 15) == 0;
          if (whole && a.y && !a.out_f32 && !resid) {
            __nv_bfloat16* tb16 = reinterpret_cast<__nv_bfloat16*>(tr_smem + (xchg_it & 1) * 4096);
#pragma unroll
            for (int j = 0; j < 16; ++j) tb16[j * 128 + li] = __float2bfloat16(r[j]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
            if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
              *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
            }
            ++xchg_it;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int u = li * 2 + q;                 // 256 units of 16 bytes: 16 per token row
              const int row = u >> 4, col = (u & 15) * 8;
              const int tok = t.tok0 + c + row;
              if (tok < t.tok_end)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y) + static_cast<size_t>(tok) * a.ldy + t.feat0 + col) =
                    *reinterpret_cast<const uint4*>(tb16 + row * 128 + col);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = t.tok0 + c + j;
              const bool ok_e = fok && tok < t.tok_end && c + j >= col_lo && c + j < col_hi;
              const size_t o = static_cast<size_t>(tok) * a.ldy + feat_i;
              if (ok_e && resid) r[j] += __bfloat162float(resid[o]);
              if (ok_e && a.y) {
                if (a.out_f32) reinterpret_cast<float*>(a.y)[o] = r[j];
                else reinterpret_cast<__nv_bfloat16*>(a.y)[o] = __float2bfloat16(r[j]);
              }
            }
          }
          if (a.yq) {
            // the 1x128 quant group of a token is the 128 lanes of this tile: reduce |r|
            // inside each warp, exchange the four warp maxima through shared memory
            float* scratch = red_scratch + (xchg_it & 1) * 64;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // |r| >= 0, so the float order is the order of its bit pattern: one warp-wide integer max per value
              const uint32_t vb = __reduce_max_sync(0xffffffffu, fok ? __float_as_uint(fabsf(r[j])) : 0u);
              if (lane == 0) scratch[lq * 16 + j] = __uint_as_float(vb);
            }
            PLOW_TRACE(if (trt && c == 0) a.trace[(70 + tile_no) * 8 + 2] = clock64();)
            __syncwarp();
            if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
            if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
              *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
            }
            ++xchg_it;
            PLOW_TRACE(if (trt && c == 0) a.trace[(70 + tile_no) * 8 + 3] = clock64();)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float m = fmaxf(fmaxf(scratch[j], scratch[16 + j]),
                                    fmaxf(scratch[32 + j], scratch[48 + j]));
              const float sc = fmaxf(m, 1e-10f) * (1.0f / 448.0f);
              const float inv = __fdividef(448.0f, fmaxf(m, 1e-10f));
              const int tok = t.tok0 + c + j;
              if (fok && tok < t.tok_end && c + j >= col_lo && c + j < col_hi) {
                reinterpret_cast<__nv_fp8_e4m3*>(a.yq)[static_cast<size_t>(tok) * a.ldy + feat_i] =
                    __nv_fp8_e4m3(r[j] * inv);
                if (li == 0) a.syq[static_cast<size_t>(t.feat0 >> 7) * a.ld_syq + tok] = sc;
              }
            }
          }
          PLOW_TRACE(if (trt && c == 0) a.trace[(70 + tile_no) * 8 + 4] = clock64();)
        }
        PLOW_TRACE(if (trt) a.trace[(70 + tile_no) * 8 + 5] = clock64();)
        if (!ok) break;
        if (a.ar_world > 1) {
          // tell the tile's owner (tile mod world) that this rank's partial is in place
          __threadfence_system();
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
          }
          ++xchg_it;
          const int tile = t.feat0 >> 7;
          if (a.ar_oneshot == 1) {
            // tell every rank, then reduce this tile from the local slots as soon as every rank's flag is here
            if (li < a.ar_world)
              st_release_sys(reinterpret_cast<uint32_t*>(a.ar_peer[li] + a.ar_flag_ofs) + tile * 8 + a.ar_me, ar_ep);
            if (li < a.ar_world) {
              const uint32_t* f = reinterpret_cast<const uint32_t*>(a.ar_peer[a.ar_me] + a.ar_flag_ofs) + tile * 8 + li;
              const unsigned long long t0 = globaltimer_ns();
              const unsigned long long dl = static_cast<unsigned long long>(a.wait_deadline_ms ? a.wait_deadline_ms : 2000) * 1000000ull;
              while (ld_acquire_sys(f) < ar_ep) {
                if (*abort_flag || globaltimer_ns() - t0 > dl) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagGemm); break; }
                __nanosleep(64);
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
            if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag) || *abort_flag) { ok = false; break; }
            ++xchg_it;
            const uint8_t* base = a.ar_peer[a.ar_me] + a.ar_part_ofs + (ar_ep & 1) * a.ar_half_bytes;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
              if (t.tok0 + c >= t.tok_end) break;
              float acc16[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) acc16[j] = 0.f;
              for (int r = 0; r < a.ar_world; ++r) {      // rank order: every rank forms the same sum, bit for bit
                const uint4* pp = reinterpret_cast<const uint4*>(base + (static_cast<size_t>((tile * a.ar_world + r) * 128 + li) * BN + c) * 2);
                const uint4 v0 = pp[0], v1 = pp[1];
                const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
                const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f0 = __bfloat1622float2(h0[j]), f1 = __bfloat1622float2(h1[j]);
                  acc16[2 * j] += f0.x; acc16[2 * j + 1] += f0.y; acc16[8 + 2 * j] += f1.x; acc16[8 + 2 * j + 1] += f1.y;
                }
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int tok = t.tok0 + c + j;
                if (fok && tok < t.tok_end) {
                  const size_t o = static_cast<size_t>(tok) * a.ldy + feat_i;
                  float v = acc16[j];
                  if (resid) v += __bfloat162float(resid[o]);
                  reinterpret_cast<__nv_bfloat16*>(a.y)[o] = __float2bfloat16(v);
                }
              }
            }
          } else if (li == 0) {
            if (a.ar_oneshot == 2)   // one multicast store puts this rank's flag of the tile on every rank
              multimem_st_u32(a.ar_mc + a.ar_flag_ofs + (static_cast<size_t>(tile) * 8 + a.ar_me) * 4, ar_ep);
            else
              st_release_sys(reinterpret_cast<uint32_t*>(a.ar_peer[tile % a.ar_world] + a.ar_flag_ofs) + tile * 8 + a.ar_me, ar_ep);
          }
        }
        if (ws_tile) {
          // the split that leaves last re-arms the tile's counters for the next launch
          PLOW_TRACE(if (a.trace && blockIdx.x == 0 && li == 0) a.trace[60 * 8 + 3] = clock64();)
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
          }
          ++xchg_it;
          if (li == 0) {
            int* done = a.ws_ctr + (256 + t.tile_id) * 32;
            if (atomicAdd(done, 1) == a.splits - 1) { *done = 0; a.ws_ctr[t.tile_id * 32] = 0; __threadfence(); }
          }
        }
        if (fix_n > 0) {
          // every warp is past its flag polls and its reads of the partials: re-arm the followers' flags
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
          }
          ++xchg_it;
          if (li < fix_n) reinterpret_cast<uint32_t*>(a.ws_ctr)[(blockIdx.x + 1 + li) * 32] = 0u;
        }
       }
      } else {
        // thread = token, columns = features (contiguous in memory); cl counts the warp's own columns
        const bool tok_ok = tok_i < t.tok_end;
        float amax = 0.f;
#pragma unroll
        for (int cl = 0; cl < kCH; cl += 16) {
          float r[16];
          load16(cl, r);
          const int f0 = t.feat0 + hc0 + cl;
          const size_t o = static_cast<size_t>(tok_i) * a.ldy + f0;
          if (tok_ok && resid) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f0 + j < a.N) r[j] += __bfloat162float(resid[o + j]);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(r[j]));
          if (tok_ok && a.y) {
            if (a.out_f32) {
              float* yp = reinterpret_cast<float*>(a.y) + o;
              if (f0 + 16 <= a.N && (a.ldy & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<float4*>(yp + j) = make_float4(r[j], r[j + 1], r[j + 2], r[j + 3]);
              } else {
                for (int j = 0; j < 16; ++j) if (f0 + j < a.N) yp[j] = r[j];
              }
            } else {
              __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(a.y) + o;
              if (f0 + 16 <= a.N && (a.ldy & 7) == 0) {
                uint32_t pk[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
                  pk[j] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(yp) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(yp + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              } else {
                for (int j = 0; j < 16; ++j) if (f0 + j < a.N) yp[j] = __float2bfloat16(r[j]);
              }
            }
          }
        }
        if constexpr (kCH * Cfg::kHalves == 128 || kCH == 128) {
          if (a.yq) {
            // the 1x128 group of a token is held by the thread (or by the two threads that share its lane): second
            // pass re-reads the accumulators
            if constexpr (kCH == 64) {
              // exchange the half maxima with the warp that owns the other columns of this lane quarter
              float* ex = fac_smem + (yq_it & 1) * 256;
              ex[half * 128 + li] = amax;
              __syncwarp();
              if (lane == 0) mbar_arrive(&pair_bar[lq]);
              if (!mbar_wait(&pair_bar[lq], yq_it & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_TMEM_WAIT | kTagGemm); ok = false; break;
              }
              amax = fmaxf(amax, ex[(half ^ 1) * 128 + li]);
              ++yq_it;
            }
            const float sc = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
            const float inv = 1.0f / sc;
#pragma unroll
            for (int cl = 0; cl < kCH; cl += 16) {
              float r[16];
              load16(cl, r);
              const int f0 = t.feat0 + hc0 + cl;
              if (tok_ok && resid) {
                const size_t o = static_cast<size_t>(tok_i) * a.ldy + f0;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (f0 + j < a.N) r[j] += __bfloat162float(resid[o + j]);
              }
              if (tok_ok && f0 + 16 <= a.N) {
                uint32_t pk[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_fp8x4_e4m3 q(make_float4(r[4 * j] * inv, r[4 * j + 1] * inv,
                                                r[4 * j + 2] * inv, r[4 * j + 3] * inv));
                  pk[j] = *reinterpret_cast<uint32_t*>(&q);
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.yq) +
                                          static_cast<size_t>(tok_i) * a.ldy + f0) =
                    make_uint4(pk[0], pk[1], pk[2], pk[3]);
              }
            }
            if (tok_ok && (kCH == 128 || half == 0)) a.syq[static_cast<size_t>((t.feat0 + (kCH == 128 ? hc0 : 0)) >> 7) * a.ld_syq + tok_i] = sc;
          }
        }
      }
      if constexpr (!FP8) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[accit & 1]);
        ++accit;
      }
    }
    // ---- fused all-reduce, phase 2 (swap mode): the owner of a tile (tile mod world) sums the ranks'
    // partials in rank order (f32, rounded to bf16 once, so every rank receives identical bits) and
    // stores the result into every rank's output; then one arrival per (tile, rank).  Reference
    // numerics: runtime/nvidia/op_collective.cuh:18-20.  Plain peer loads/stores, bounded waits.
    if constexpr (SWAP && !DUAL) {
      if (a.ar_world > 1 && ok && a.ar_oneshot == 1) {
        // the launch counter moves on once every CTA of this launch is through (ar_epoch[2] counts them)
        if (li == 0) {
          __threadfence();
          if (atomicAdd(&a.ar_epoch[2], 1u) == gridDim.x - 1) { a.ar_epoch[2] = 0; __threadfence(); a.ar_epoch[0] = ar_ep; }
        }
      }
      if (a.ar_world > 1 && ok && a.ar_oneshot != 1) {
        const bool mc = a.ar_oneshot == 2;
        const int W = a.ar_world;
        const int n_tiles = (a.N + 127) / 128;
        const unsigned long long dl = static_cast<unsigned long long>(a.wait_deadline_ms ? a.wait_deadline_ms : 2000) * 1000000ull;
        int idx = 0;
        for (int tile = a.ar_me; tile < n_tiles && ok; tile += W, ++idx) {
          if (idx % static_cast<int>(gridDim.x) != static_cast<int>(blockIdx.x)) continue;
          if (li < W) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(a.ar_peer[a.ar_me] + a.ar_flag_ofs) + tile * 8 + li;
            const unsigned long long t0 = globaltimer_ns();
            while (ld_acquire_sys(f) < ar_ep) {
              if (*abort_flag || globaltimer_ns() - t0 > dl) { *abort_flag = 1; atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagGemm); break; }
              __nanosleep(128);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag) || *abort_flag) { ok = false; break; }
          ++xchg_it;
          const int feat = tile * 128 + li;
#pragma unroll 1
          for (int c = 0; c < BN; c += 16) {
            if (c >= a.M) break;
            float acc16[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc16[j] = 0.f;
            for (int r = 0; r < (mc ? 1 : W); ++r) {
              const size_t po = a.ar_part_ofs + (static_cast<size_t>(tile * 128 + li) * BN + c) * 2;
              uint4 v0, v1;
              if (mc) {      // the switch sums the ranks' copies (f32 accumulation, one rounding)
                v0 = multimem_ld_reduce_bf16x8(a.ar_mc + po);
                v1 = multimem_ld_reduce_bf16x8(a.ar_mc + po + 16);
              } else {
                const uint4* pp = reinterpret_cast<const uint4*>(a.ar_peer[r] + po);
                v0 = pp[0]; v1 = pp[1];
              }
              const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
              const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f0 = __bfloat1622float2(h0[j]), f1 = __bfloat1622float2(h1[j]);
                acc16[2 * j] += f0.x; acc16[2 * j + 1] += f0.y; acc16[8 + 2 * j] += f1.x; acc16[8 + 2 * j + 1] += f1.y;
              }
            }
            // transpose the 128-feature x 16-token chunk through shared memory so every peer gets
            // whole 256-byte row segments (16-byte stores) instead of scattered 2-byte stores
            __nv_bfloat16* tsm = reinterpret_cast<__nv_bfloat16*>(fac_smem);       // [16 tokens][128 features]
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = acc16[j];
              if (resid && feat < a.N && c + j < a.M) v += __bfloat162float(resid[static_cast<size_t>(c + j) * a.ldy + feat]);
              tsm[j * 128 + li] = __float2bfloat16(v);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
            if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) { ok = false; break; }
            ++xchg_it;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int u = li * 2 + q;              // 256 units of 16 bytes
              const int row = u >> 4, col = (u & 15) * 8;
              if (c + row < a.M && tile * 128 + col + 8 <= a.N) {
                const uint4 v = *reinterpret_cast<const uint4*>(tsm + row * 128 + col);
                const size_t o = static_cast<size_t>(c + row) * a.ldy + tile * 128 + col;
                if (mc) multimem_st_bf16x8(a.ar_mc + a.ar_y_ofs + o * 2, v);
                else for (int p = 0; p < W; ++p) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.ar_peer[p] + a.ar_y_ofs) + o) = v;
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
            if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) { ok = false; break; }
            ++xchg_it;
          }
          if (!ok) break;
          __threadfence_system();
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (!mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) { ok = false; break; }
          ++xchg_it;
          if (mc) { if (li == 0) multimem_st_u32(a.ar_mc + a.ar_tdone_ofs + static_cast<size_t>(tile) * 4, ar_ep); }
          else if (li < W) red_add_release_sys(reinterpret_cast<uint32_t*>(a.ar_peer[li] + a.ar_done_ofs), 1u);
        }
        // the kernel ends on this rank only when every tile of this launch has landed here
        if (mc && blockIdx.x == 0) {
          // every tile's epoch word must have landed here (written by the tile's owner through the switch)
          const uint32_t* td = reinterpret_cast<const uint32_t*>(a.ar_peer[a.ar_me] + a.ar_tdone_ofs);
          const unsigned long long t0 = globaltimer_ns();
          for (int tile = li; tile < n_tiles; tile += 128) {
            while (ld_acquire_sys(td + tile) < ar_ep) {
              if (globaltimer_ns() - t0 > dl) { atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagGemm); break; }
              __nanosleep(128);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&xchg_bar[xchg_it & 1]);
          if (mbar_wait(&xchg_bar[xchg_it & 1], (xchg_it >> 1) & 1, abort_flag)) { ++xchg_it; if (li == 0) *a.ar_epoch = ar_ep; }
        } else if (mc) {
          // other CTAs have nothing left to do
        } else if (blockIdx.x == 0 && li == 0) {
          const uint32_t* d = reinterpret_cast<const uint32_t*>(a.ar_peer[a.ar_me] + a.ar_done_ofs);
          const unsigned long long t0 = globaltimer_ns();
          // ar_epoch[1] = arrivals seen by the launches before this one (shapes, hence tile counts, differ between
          // launches); no peer can be a launch ahead, because every tile needs this rank's partial of that launch
          const uint32_t target = a.ar_epoch[1] + static_cast<uint32_t>(n_tiles);
          while (ld_acquire_sys(d) - target > 0x7fffffffu) {      // wrap-safe "d < target"
            if (globaltimer_ns() - t0 > dl) { atomicCAS(a.status, 0, PLOW_ERR_PEER_WAIT | kTagGemm); break; }
            __nanosleep(128);
          }
          a.ar_epoch[1] = target;
          *a.ar_epoch = ar_ep;
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give TMA copies that were in flight when a role gave up time to land (bounded)
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {}
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool FP8, bool DUAL, bool SWAP>
int launch_gemm_tc(const GemmArgs& a, int ldx_elems, int ldw_elems, int64_t w_rows,
                   cudaStream_t stream) {
  using Cfg = GemmCfg<BN, DUAL, SWAP, FP8>;
  const int es = FP8 ? 1 : 2;
  CUtensorMap tm_x, tm_w;
  const uint32_t box_x = SWAP ? BN : 128;
  const uint32_t box_w = SWAP ? 128 : BN;
  int r = make_tmap_2d(&tm_x, a.x, es, a.M, a.K, static_cast<uint64_t>(ldx_elems) * es, box_x);
  if (r) return 1000 + r;
  r = make_tmap_2d(&tm_w, a.w, es, w_rows, a.K, static_cast<uint64_t>(ldw_elems) * es, box_w);
  if (r) return 2000 + r;
  auto kern = gemm_tc_kernel<BN, FP8, DUAL, SWAP>;
  static DeviceOnce attr_set;
  {
    cudaError_t e = ensure_smem(attr_set, kern, Cfg::kSmemBytes);
    if (e != cudaSuccess) return 3000 + static_cast<int>(e);
  }
  int grid = sm_count();
  if (SWAP && a.stream) {
    if (a.E == 0) {
      // at least two K blocks per CTA; the ranges are cut evenly over the grid
      const int kk = FP8 ? 128 : 64;
      const long long iters = static_cast<long long>((a.N + 127) / 128) * ((a.M + BN - 1) / BN) * ((a.K + kk - 1) / kk);
      if (iters / 2 < grid) grid = static_cast<int>(iters / 2 > 0 ? iters / 2 : 1);
    }
  } else if (a.E == 0) {
    const int n_wt = SWAP ? (a.N + 127) / 128 : (a.N + BN - 1) / BN;
    const int n_tt = SWAP ? (a.M + BN - 1) / BN : (a.M + 127) / 128;
    const long long tiles = static_cast<long long>(n_wt) * n_tt * (SWAP && a.splits > 1 ? a.splits : 1);
    if (tiles < grid) grid = static_cast<int>(tiles);
  }
  if (grid < 1) grid = 1;
  cudaError_t e = launch_pdl(kern, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, a, tm_x, tm_w);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // namespace plow
