// Fused forward + tangent attention for sm_100a, CTA-pair variant.
//
// Same algorithm, roles and tensor-memory layout as the dual pass of attn_fwd.cuh (P warps, G warps,
// one MMA-issuing warp, one TMA warp), but two CTAs of a cluster work on two neighbouring 128-row
// query tiles of the same (batch, head) and run every MMA together as one tcgen05.mma of M = 256
// with .cta_group::2:
//
//   * each CTA keeps its own query tile (A operand) and its own S / dS / P / O / T in tensor memory;
//   * the B operand is split between the two CTAs, so each CTA loads only HALF of every K/dK block
//     (64 of the 128 key rows) and HALF of every V/dV block (DPAD/2 of the head-dim columns).
//
// That halves the L2 -> shared-memory traffic per query tile (the single-CTA kernel re-reads all of
// K/dK/V/dV of a head for each of its query tiles) and the shared-memory footprint of the rings,
// which pays for a third ring stage.  Loads are plain per-CTA TMA loads (no cluster multicast); only
// tcgen05.commit fans its barrier arrival out to both CTAs.
//
// Barrier placement: "operand ready" barriers that the MMA warp waits on live in the LEADER CTA
// (rank 0) and are arrived on by both CTAs (TMA transaction bytes, softmax warps); barriers that
// a CTA's own warps wait on (S ready, dS ready, ring slot free, accumulators done ...) are local and
// are arrived on by the leader's tcgen05.commit with a two-CTA multicast mask.
//
// V column order.  CTA r holds DPAD/2 columns of V: columns [32r, 32r+32) and, when DPAD > 64, the
// e = DPAD/2 - 32 columns [64 + r e, 64 + r e + e).  Accumulator column t therefore maps to head-dim
// column   t            for t in [0, 32)
//          64 + t - 32  for t in [32, 32+e)
//          32 + t - h   for t in [h, h+32)        (h = DPAD/2)
//          64 + e + t - h - 32   for t in [h+32, DPAD)
// and the epilogue stores accordingly.
#pragma once

#include "attn_fwd.cuh"

namespace dmf {

// kShort: key sequences of at most kShortMaxBlocks blocks.  With so few blocks per tile the third V stage
// buys nothing, while writing the tile out is a large part of a tile's time: the shared memory goes to a
// second staging tile instead, so that o and to are staged and stored without waiting for the first
// store to have read its tile (behind the loads queued in the TMA unit that wait takes 2000 cycles).
template <int TAIL, bool kShort = false>
struct PairTraits {
  static_assert(TAIL == 0 || TAIL == 16 || TAIL == 32, "the pair kernel needs P in its own tensor-memory columns");
  static constexpr int kDPad = 64 + TAIL;
  static constexpr int kHalf = kDPad / 2;           // V / O columns per CTA
  static constexpr int kExtra = kHalf - 32;         // columns of the second V atom that are used
  // query tile (A operand), 128 rows
  static constexpr int kMainBytes = 128 * 128;
  static constexpr int kTailBytes = 128 * TAIL * 2;
  static constexpr int kTileBytes = kMainBytes + kTailBytes;
  static constexpr int kQGroupBytes = 2 * kTileBytes;
  // this CTA's half of a K / dK block, 64 rows
  static constexpr int kKMainBytes = 64 * 128;
  static constexpr int kKTailBytes = 64 * TAIL * 2;
  static constexpr int kKTileBytes = kKMainBytes + kKTailBytes;
  static constexpr int kKGroupBytes = 2 * kKTileBytes;
  // this CTA's half of a V / dV block: atoms of 32 columns x 128 rows, 64-byte swizzle
  static constexpr int kVAtoms = kExtra > 0 ? 2 : 1;
  static constexpr int kVAtomBytes = 128 * 64;
  static constexpr int kVTileBytes = kVAtoms * kVAtomBytes;
  static constexpr int kVGroupBytes = 2 * kVTileBytes;
  // Ring depths, output staging (one tile-shaped buffer each for o and to, or one shared by both) and
  // the number of query-tile buffers are what fits in 227 KB: head_dim 96 has room for two V stages
  // only; head_dim 64 has room for a second Q/dQ buffer, so that the query tiles of the next pair are
  // loaded a whole pair ahead (with one buffer that load can only start when the pair's last dS product
  // has run, and the tensor pipe waits for it: about 3400 cycles per pair).
  static constexpr int kStagesK = 3;
  static constexpr int kStagesV = (TAIL == 32 || kShort) ? 2 : 3;
  static constexpr int kOutBufs = (TAIL == 0 || (kShort && TAIL == 16)) ? 2 : 1;
  static constexpr int kQBufs = TAIL == 0 ? 2 : 1;
  static constexpr int kRingBytes = kQBufs * kQGroupBytes + kStagesK * kKGroupBytes + kStagesV * kVGroupBytes;
  static constexpr int kTileSmem = kRingBytes + kOutBufs * kTileBytes;
  static constexpr int kXchgBytes = 4096;
  // barriers
  static constexpr int kBarQFull = 0 /* one per Q buffer */, kBarQEmpty = 2 /* one per Q buffer */, kBarSFull = 4,
                       kBarPFull = 5, kBarGFull = 6, kBarXchg = 7, kBarSEmpty = 8, kBarPEmpty = 9, kBarPG = 10,
                       kBarAccEmpty = 11, kBarKFull = 12,
                       kBarKEmpty = kBarKFull + kStagesK, kBarVFull = kBarKEmpty + kStagesK,
                       kBarVEmpty = kBarVFull + kStagesV, kNumBars = kBarVEmpty + kStagesV;
  static constexpr int kSmemBytes = 1024 + kTileSmem + kXchgBytes + kNumBars * 8 + 16;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  // tensor memory columns (per CTA)
  static constexpr uint32_t kColS = 0, kColDS = 128, kColP = 256, kColO = 320, kColT = 320 + kDPad;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTailSwizzle = TAIL == 32 ? kSwizzle64 : kSwizzle32;
  static constexpr uint32_t kTailRowBytes = 2 * TAIL;
};

constexpr int kPairThreads = 320;
constexpr int kShortMaxBlocks = 2;  // see PairTraits

// head-dim column of accumulator column t (t a multiple of 8); see the header comment
template <typename TR>
__device__ __forceinline__ int pair_head_col(int t) {
  constexpr int h = TR::kHalf, e = TR::kExtra;
  if (t < 32) return t;
  if (t < h) return 64 + (t - 32);
  if (t < h + 32) return 32 + (t - h);
  return 64 + e + (t - h - 32);
}

// acc[256 x 128] (+)= A[256 x D] * B[128 x D]^T: each CTA's A tile has 128 rows, each CTA's B tile 64 rows
template <int TAIL, typename TR>
__device__ __forceinline__ void issue_qk_pair(bool leader, uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile,
                                              uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const uint64_t ad = make_smem_desc(a_tile + kk * 32, 16, 1024, kSwizzle128);
    const uint64_t bd = make_smem_desc(b_tile + kk * 32, 16, 1024, kSwizzle128);
    mma_ss_pair(d_tmem, ad, bd, idesc, (accumulate || kk > 0) ? 1u : 0u, leader);
  }
#pragma unroll
  for (int kk = 0; kk < TAIL / 16; ++kk) {
    const uint64_t ad = make_smem_desc(a_tile + TR::kMainBytes + kk * 32, 16, 8 * TR::kTailRowBytes, TR::kTailSwizzle);
    const uint64_t bd = make_smem_desc(b_tile + TR::kKMainBytes + kk * 32, 16, 8 * TR::kTailRowBytes, TR::kTailSwizzle);
    mma_ss_pair(d_tmem, ad, bd, idesc, 1u, leader);
  }
}

// acc[256 x DPAD] (+)= A[256 x 128] * V[128 x DPAD]; A from each CTA's tensor memory, each CTA's V tile
// holds DPAD/2 columns as 64-byte-swizzled atoms of 32 columns
template <typename TR>
__device__ __forceinline__ void issue_pv_pair(bool leader, uint32_t d_tmem, uint32_t a_tmem, uint32_t v_tile,
                                              uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < kBlockKV / 16; ++kk) {
    const uint64_t bd = make_smem_desc(v_tile + kk * (16 * 64), TR::kVAtomBytes, 8 * 64, kSwizzle64);
    mma_ts_pair(d_tmem, a_tmem + kk * 8, bd, idesc, (accumulate || kk > 0) ? 1u : 0u, leader);
  }
}

// ---- the kernel ---------------------------------------------------------------
// p.k_* maps have a box of 64 rows; p.num_tiles counts tile PAIRS; p.num_q_tiles is even.

// kDual = false is the plain forward on the same skeleton: no tangent tiles are loaded, no dS / P dV / G V
// products are issued, the G warps only do the epilogue.  Each softmax warp then has its scheduler to
// itself and a whole score row per thread (no row-max exchange between warpgroups as in the
// single-CTA plain forward).
//
// kF32Out (checking mode, not a production path): o and to leave the kernel as fp32, taken from the
// accumulators before the rounding to the 16-bit output type, with plain per-row global stores
// (p.o / p.to are then float tensors; their strides count floats).  Everything up to the epilogue
// is the same code except that all exponentials use the MUFU unit (see kPoly below), so what this mode
// shows is the error of the accumulation itself: the lazy rescale and the fp32 sums.
template <typename T, int TAIL, bool kDual, bool kShort, bool kF32Out = false>
__global__ void __launch_bounds__(kPairThreads, 1)
attn_fwd_pair_kernel(const __grid_constant__ FwdParams p) {
  using TR = PairTraits<TAIL, kShort>;
  constexpr int DPAD = TR::kDPad;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  // The checking mode evaluates every exponential on the MUFU unit.  The cubic (relative error up to 7.5e-5)
  // moves about one P element in 400 across a bf16 rounding boundary, and a single such element of a heavy
  // key shows up as 1e-3 in a max-norm comparison with an evaluation that rounds the exact exponential.
  constexpr int kPoly = kF32Out ? 0 : kPolyEvery;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_k = s_q + TR::kQBufs * TR::kQGroupBytes;
  const uint32_t s_v = s_k + TR::kStagesK * TR::kKGroupBytes;
  uint8_t* out_stage = smem + TR::kRingBytes;  // tile-shaped staging for the TMA stores of o and to
  float* xchg = reinterpret_cast<float*>(smem + TR::kTileSmem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::kTileSmem + TR::kXchgBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + TR::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) -> uint32_t { return bar0 + 8u * static_cast<uint32_t>(i); };       // this CTA's barrier
  auto lbar = [&](int i) -> uint32_t { return map_to_cta(bar(i), 0); };                      // the leader's barrier

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_kv_blocks = p.seqlen_kv / kBlockKV;
  const int pairs_per_bh = p.num_q_tiles >> 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < TR::kNumBars; ++i) {
      uint32_t count = 1;  // tcgen05.commit (multicast from the leader)
      if (i == TR::kBarQFull || i == TR::kBarQFull + 1 || (i >= TR::kBarKFull && i < TR::kBarKEmpty) || (i >= TR::kBarVFull && i < TR::kBarVEmpty))
        count = 2;  // one producer arrival (+ its transaction bytes) per CTA
      if (i == TR::kBarPFull || i == TR::kBarGFull || i == TR::kBarSEmpty || i == TR::kBarAccEmpty)
        count = 8;                         // 4 warps of each CTA
      if (i == TR::kBarXchg) count = 4;    // the 4 local P warps
      if (i == TR::kBarPG) count = 4;      // the 4 local P warps
      if (i == TR::kBarPEmpty) count = kDual ? 5 : 1;  // commit (+ the 4 local G warps, which read P too)
      mbar_init(bar(i), count);
    }
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc_pair(smem_u32(tmem_slot), TR::kTmemCols);
    tmem_relinquish_alloc_permit_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anybody arrives remotely
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // =========================== TMA producer (each CTA) ====================
    if (lane == 0) {
      prefetch_tensor_map(&p.q_main);
      prefetch_tensor_map(&p.k_main);
      prefetch_tensor_map(&p.v_map);
      uint32_t kcnt = 0, vcnt = 0, tcnt = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleProducer + b_);
      };
      // Q and dQ tile of pair number pp_ (the t-th pair of this cluster) into query buffer t % kQBufs
      auto load_q = [&](int pp_, uint32_t t) -> bool {
        const int bh_ = pp_ / pairs_per_bh;
        const int q0 = (2 * (pp_ % pairs_per_bh) + static_cast<int>(rank)) * kBlockQ;
        const int b_ = bh_ / p.heads, h_ = bh_ % p.heads;
        const int x_ = -column_shift(p, 0, b_, h_);
        const uint32_t qb = t % TR::kQBufs, dst = s_q + qb * TR::kQGroupBytes;
        if (!wait(TR::kBarQEmpty + qb, ((t / TR::kQBufs) & 1u) ^ 1u)) return false;
        const uint32_t qf = lbar(TR::kBarQFull + qb);
        mbar_arrive_expect_tx_cluster(qf, kDual ? TR::kQGroupBytes : TR::kTileBytes);
        tma_load_4d_pair(dst, &p.q_main, qf, x_, q0, h_, b_);
        if constexpr (kDual) tma_load_4d_pair(dst + TR::kTileBytes, &p.tq_main, qf, x_, q0, h_, b_);
        if constexpr (TAIL > 0) {
          tma_load_4d_pair(dst + TR::kMainBytes, &p.q_tail, qf, 64 + x_, q0, h_, b_);
          if constexpr (kDual)
            tma_load_4d_pair(dst + TR::kTileBytes + TR::kMainBytes, &p.tq_tail, qf, 64 + x_, q0, h_, b_);
        }
        return true;
      };
      for (int pp = cluster_id; ok && pp < p.num_tiles; pp += num_clusters, ++tcnt) {
        const int bh = pp / pairs_per_bh;
        const int b = bh / p.heads, h = bh % p.heads;
        const int xqk = -column_shift(p, 0, b, h);
        if (tcnt == 0u || TR::kQBufs == 1) ok = load_q(pp, tcnt);
        if (!ok) break;
        if (TR::kQBufs == 2 && pp + num_clusters < p.num_tiles) ok = load_q(pp + num_clusters, tcnt + 1u);
        if (!ok) break;
        for (int j = 0; j < num_kv_blocks; ++j) {
          const int kv0 = j * kBlockKV;
          {
            const uint32_t s = kcnt % TR::kStagesK, ph = (kcnt / TR::kStagesK) & 1u;
            ok = wait(TR::kBarKEmpty + s, ph ^ 1u);
            if (!ok) break;
            const uint32_t dst = s_k + s * TR::kKGroupBytes, fb = lbar(TR::kBarKFull + s);
            const int kr = kv0 + 64 * static_cast<int>(rank);  // this CTA's half of the key rows
            mbar_arrive_expect_tx_cluster(fb, kDual ? TR::kKGroupBytes : TR::kKTileBytes);
            tma_load_4d_pair(dst, &p.k_main, fb, xqk, kr, h, b);
            if constexpr (kDual) tma_load_4d_pair(dst + TR::kKTileBytes, &p.tk_main, fb, xqk, kr, h, b);
            if constexpr (TAIL > 0) {
              tma_load_4d_pair(dst + TR::kKMainBytes, &p.k_tail, fb, 64 + xqk, kr, h, b);
              if constexpr (kDual)
                tma_load_4d_pair(dst + TR::kKTileBytes + TR::kKMainBytes, &p.tk_tail, fb, 64 + xqk, kr, h, b);
            }
            ++kcnt;
          }
          {
            const uint32_t s = vcnt % TR::kStagesV, ph = (vcnt / TR::kStagesV) & 1u;
            ok = wait(TR::kBarVEmpty + s, ph ^ 1u);
            if (!ok) break;
            const uint32_t dst = s_v + s * TR::kVGroupBytes, fb = lbar(TR::kBarVFull + s);
            mbar_arrive_expect_tx_cluster(fb, kDual ? TR::kVGroupBytes : TR::kVTileBytes);
            const int x0 = 32 * static_cast<int>(rank);                   // columns [32r, 32r+32)
            tma_load_4d_pair(dst, &p.v_map, fb, x0, kv0, h, b);
            if constexpr (kDual) tma_load_4d_pair(dst + TR::kVTileBytes, &p.tv_map, fb, x0, kv0, h, b);
            if constexpr (TR::kVAtoms > 1) {
              const int x1 = 64 + TR::kExtra * static_cast<int>(rank);    // columns [64 + r e, ...): e of them used
              tma_load_4d_pair(dst + TR::kVAtomBytes, &p.v_map, fb, x1, kv0, h, b);
              if constexpr (kDual) tma_load_4d_pair(dst + TR::kVTileBytes + TR::kVAtomBytes, &p.tv_map, fb, x1, kv0, h, b);
            }
            ++vcnt;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA only) =======================
    // Warp-uniform control flow; one elected lane issues.  Every MMA is a .cta_group::2 instruction
    // that reads operands from, and writes accumulators to, both CTAs; every commit arrives on the
    // same-named barrier of both CTAs.
    if (rank == 0) {
      const bool leader = elect_one();
      auto commit = [&](int b_) { tc_commit_pair(bar(b_), leader); };
      constexpr uint32_t idesc_qk = make_idesc(kBf16, false, false, 256, 128);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, false, true, 256, DPAD);
      const uint32_t t_s = tmem + TR::kColS, t_ds = tmem + TR::kColDS, t_p = tmem + TR::kColP;
      const uint32_t t_o = tmem + TR::kColO, t_t = tmem + TR::kColT;
      uint32_t kcnt = 0, vcnt = 0, tcnt = 0, pcnt = 0, gcnt = 0, scnt = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleMma + b_);
      };
      for (int pp = cluster_id; ok && pp < p.num_tiles; pp += num_clusters, ++tcnt) {
        const uint32_t qb = tcnt % TR::kQBufs, q_tile = s_q + qb * TR::kQGroupBytes;
        ok = wait(TR::kBarQFull + qb, (tcnt / TR::kQBufs) & 1u);
        if (!ok) break;
        uint32_t sk = 0, kt = 0, s_in_tile = 0;
        // S of the next block: needs the softmax of BOTH CTAs to have read the current S, and the K halves
        auto issue_s = [&]() -> bool {
          sk = kcnt % TR::kStagesK;
          if (scnt > 0 && !wait(TR::kBarSEmpty, (scnt - 1u) & 1u)) return false;
          if (!wait(TR::kBarKFull + sk, (kcnt / TR::kStagesK) & 1u)) return false;
          tc_fence_after_sync();
          kt = s_k + sk * TR::kKGroupBytes;
          issue_qk_pair<TAIL, TR>(leader, t_s, q_tile, kt, idesc_qk, false);
          commit(TR::kBarSFull);
          if constexpr (!kDual) {  // nothing else reads this K block or, after the pair's last S, its query tile
            commit(TR::kBarKEmpty + sk);
            if (++s_in_tile == static_cast<uint32_t>(num_kv_blocks)) commit(TR::kBarQEmpty + qb);
          }
          ++scnt;
          ++kcnt;
          return true;
        };
        // Issue order per tile (S runs two blocks ahead of the P V products, which the three-stage K ring
        // allows):  S_0 dS_0 S_1 | P V_0, P dV_0, S_2, G V_0, dS_1 | P V_1, P dV_1, S_3, G V_1, dS_2 | ...
        // dS_j uses the K block that S_j used; S_{j+2} may only overwrite S_{j+1} once the softmax of both
        // CTAs has it in registers.
        uint32_t ds_sk = 0, ds_kt = 0;       // ring slot / address of the K block the next dS will use
        ok = issue_s();                      // S_0
        if (!ok) break;
        ds_sk = sk; ds_kt = kt;
        if constexpr (kDual) {
          issue_qk_pair<TAIL, TR>(leader, t_ds, q_tile + TR::kTileBytes, ds_kt, idesc_qk, false);   // dS_0
          issue_qk_pair<TAIL, TR>(leader, t_ds, q_tile, ds_kt + TR::kKTileBytes, idesc_qk, true);
          commit(TR::kBarKEmpty + ds_sk);  // "dS ready" for the G warps and "K slot free" in one
          if (num_kv_blocks == 1) commit(TR::kBarQEmpty + qb);
        }
        if (num_kv_blocks > 1) {
          ok = issue_s();                    // S_1
          if (!ok) break;
          ds_sk = sk; ds_kt = kt;            // dS_1 will use this K block
        }
        for (int j = 0; j < num_kv_blocks; ++j) {
          const uint32_t sv = vcnt % TR::kStagesV;
          const uint32_t vt = s_v + sv * TR::kVGroupBytes;
          ok = wait(TR::kBarVFull + sv, (vcnt / TR::kStagesV) & 1u);
          if (!ok) break;
          ok = wait(TR::kBarPFull, pcnt & 1u);
          if (!ok) break;
          ++pcnt;
          if (j == 0 && tcnt > 0) {  // the epilogue of the previous tile pair has read O and T (both CTAs)
            ok = wait(TR::kBarAccEmpty, (tcnt - 1u) & 1u);
            if (!ok) break;
          }
          tc_fence_after_sync();
          issue_pv_pair<TR>(leader, t_o, t_p, vt, idesc_pv, j > 0);                    // O += P V
          if constexpr (kDual) {
            issue_pv_pair<TR>(leader, t_t, t_p, vt + TR::kVTileBytes, idesc_pv, j > 0);  // T += P dV
            commit(TR::kBarPEmpty);
          } else {
            commit(TR::kBarVEmpty + sv);  // plain forward: V slot free, O up to date, P read, all in one
          }
          uint32_t nx_sk = 0, nx_kt = 0;
          const bool s_ahead = (j + 2 < num_kv_blocks);
          if (s_ahead) {
            ok = issue_s();                  // S_{j+2}
            if (!ok) break;
            nx_sk = sk; nx_kt = kt;
          }
          if constexpr (kDual) {
            ok = wait(TR::kBarGFull, gcnt & 1u);
            if (!ok) break;
            ++gcnt;
            tc_fence_after_sync();
            issue_pv_pair<TR>(leader, t_t, t_ds, vt, idesc_pv, true);                  // T += G V
          }
          if constexpr (kDual) commit(TR::kBarVEmpty + sv);  // "accumulators up to date" and "V slot free" in one
          ++vcnt;
          if (kDual && j + 1 < num_kv_blocks) {  // dS_{j+1}, on the K block S_{j+1} used
            issue_qk_pair<TAIL, TR>(leader, t_ds, q_tile + TR::kTileBytes, ds_kt, idesc_qk, false);
            issue_qk_pair<TAIL, TR>(leader, t_ds, q_tile, ds_kt + TR::kKTileBytes, idesc_qk, true);
            commit(TR::kBarKEmpty + ds_sk);
            if (j + 2 == num_kv_blocks) commit(TR::kBarQEmpty + qb);
          }
          ds_sk = nx_sk; ds_kt = nx_kt;
        }
      }
    }
  } else {
    // ===================== softmax / correction / epilogue (each CTA) ========
    // Identical to the role-split softmax of the single-CTA dual pass, on this CTA's own query tile and
    // tensor memory; only the arrivals the leader's MMA warp waits for go to the leader's barriers.
    {
      const bool p_role = warp < 6;
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t t_s = tmem + lane_base + TR::kColS, t_ds = tmem + lane_base + TR::kColDS;
      const uint32_t t_p = tmem + lane_base + TR::kColP, t_o = tmem + lane_base + TR::kColO;
      const float sl2 = p.scale_log2e;
      float* xalpha = xchg;        // [block parity][row]: factor the P warps applied to the accumulators
      float* xl = xchg + 256;      // [tile parity][row]: row sum l of the finished tile, for the G warps
      float* xm = xchg + 512;      // [tile parity][row]: running maximum of the finished tile
      uint32_t gblk = 0, tcnt = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
      };
      // Each tcgen05.commit costs the issuing thread about 120 cycles, so one commit serves two purposes:
      // the barrier that frees V ring slot g % kStagesV also says that O and T hold everything up to
      // block g, and the barrier that frees K ring slot g % kStagesK that dS of block g is ready
      // (blocks are counted through all tile pairs of this cluster, like the ring slots).
      auto wait_acc = [&](uint32_t g) -> bool {
        return wait(TR::kBarVEmpty + g % TR::kStagesV, (g / TR::kStagesV) & 1u);
      };
      for (int pp = cluster_id; ok && pp < p.num_tiles; pp += num_clusters, ++tcnt) {
        const int bh = pp / pairs_per_bh;
        const int q0 = (2 * (pp % pairs_per_bh) + static_cast<int>(rank)) * kBlockQ;
        const int b = bh / p.heads, h = bh % p.heads;
        float m_used = -CUDART_INF_F, l = 0.f, mu = 0.f;
        for (int j = 0; j < num_kv_blocks; ++j, ++gblk) {
          if (p_role) {
            // ---- S -> P ------------------------------------------------------
            ok = wait(TR::kBarSFull, gblk & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, r[c]);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive_warp_cluster(lbar(TR::kBarSEmpty));  // S is in registers (the leader waits for both CTAs)
            float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                mx0 = max3(mx0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                mx1 = max3(mx1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                mx2 = max3(mx2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
                mx3 = max3(mx3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
              }
            }
            const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
            float alpha = 1.f;
            if (j == 0) {
              m_used = m_blk;
            } else {
              const bool need = m_blk > m_used + kRescaleThreshold;
              if (__any_sync(0xffffffffu, need)) {
                // every MMA that accumulated into O / T for the previous blocks must be done: the
                // commit of block g-2 is complete (S of this block was issued after it), so the
                // barrier is at most one phase ahead
                ok = wait_acc(gblk - 1u);
                if (!ok) break;
                tc_fence_after_sync();
                if (need) {
                  alpha = fast_exp2(m_used - m_blk);
                  m_used = m_blk;
                }
                l *= alpha;
#pragma unroll 1
                for (int c = 0; c < 2 * DPAD / 16; ++c) {
                  uint32_t a[16];
                  tmem_ld_x16(t_o + c * 16, a);
                  tmem_wait_ld();
#pragma unroll
                  for (int i = 0; i < 16; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * alpha);
                  tmem_st_x16(t_o + c * 16, a);
                }
                tmem_wait_st();
              }
            }
            xalpha[(gblk & 1u) * 128 + row] = alpha;  // the G warps scale mu by the same factor
            const uint64_t sl2_2 = pack_f2(sl2, sl2), neg_m2 = pack_f2(-m_used, -m_used);
            uint64_t la = pack_f2(0.f, 0.f), lb = la;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float x0, x1, p2, p3;
                unpack_f2(fma2(pack_u2(r[c][i], r[c][i + 1]), sl2_2, neg_m2), x0, x1);
                const uint64_t xb = fma2(pack_u2(r[c][i + 2], r[c][i + 3]), sl2_2, neg_m2);
                if (kPoly > 0 && ((i / 4) % (kPoly > 0 ? kPoly : 1)) == (kPoly - 1)) {
                  poly_exp2_x2(xb, p2, p3);  // FMA-pipe cubic
                } else {
                  float x2, x3;
                  unpack_f2(xb, x2, x3);
                  p2 = fast_exp2(x2);
                  p3 = fast_exp2(x3);
                }
                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                la = add2(la, pack_f2(p0, p1));
                lb = add2(lb, pack_f2(p2, p3));
                r[c][i / 2] = Pack2<T>::pack(p0, p1);       // packed in place: word k holds elements 2k, 2k+1
                r[c][i / 2 + 1] = Pack2<T>::pack(p2, p3);
              }
            }
            {
              float s0, s1;
              unpack_f2(add2(la, lb), s0, s1);
              l += s0 + s1;
            }
            if (gblk > 0) {  // the P V products of the previous block and the G warps have read P
              ok = kDual ? wait(TR::kBarPEmpty, (gblk - 1u) & 1u) : wait_acc(gblk - 1u);
              if (!ok) break;
              tc_fence_after_sync();
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[i] = r[c][i];
              tmem_st_x16(t_p + c * 16, pk);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive_warp_cluster(lbar(TR::kBarPFull));  // for the MMA warp of the leader
            if constexpr (kDual) mbar_arrive_warp(bar(TR::kBarPG));  // for this CTA's G warps
          } else if constexpr (kDual) {
            // ---- G = P * dS * scale, mu += rowsum(G) ---------------------------
            // P first: it is ready long before dS, and once it sits in registers its columns can be
            // handed back to the P warps (they would otherwise wait for this whole block of G work).
            ok = wait(TR::kBarPG, gblk & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t pp[4][16];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_x16(t_p + c * 16, pp[c]);
            tmem_wait_ld();
            tc_fence_before_sync();
            mu *= xalpha[(gblk & 1u) * 128 + row];
            mbar_arrive_warp(bar(TR::kBarPEmpty));  // P has been read
            ok = wait(TR::kBarKEmpty + gblk % TR::kStagesK, (gblk / TR::kStagesK) & 1u);  // dS of this block
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t scale2 = pack_f2(p.scale, p.scale);
            uint64_t mua = pack_f2(0.f, 0.f), mub = mua;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t d[32];
              tmem_ld_x32(t_ds + c * 32, d);
              tmem_wait_ld();
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; i += 2) {
                const float2 pa = unpack2<T>(pp[c][i]), pb = unpack2<T>(pp[c][i + 1]);
                const uint64_t ga = mul2(pack_f2(pa.x, pa.y), mul2(pack_u2(d[2 * i], d[2 * i + 1]), scale2));
                const uint64_t gb = mul2(pack_f2(pb.x, pb.y), mul2(pack_u2(d[2 * i + 2], d[2 * i + 3]), scale2));
                mua = add2(mua, ga);
                mub = add2(mub, gb);
                float g0, g1, g2, g3;
                unpack_f2(ga, g0, g1);
                unpack_f2(gb, g2, g3);
                pk[i] = Pack2<T>::pack(g0, g1);
                pk[i + 1] = Pack2<T>::pack(g2, g3);
              }
              tmem_st_x16(t_ds + c * 16, pk);  // over dS columns this thread has already read
            }
            {
              float s0, s1;
              unpack_f2(add2(mua, mub), s0, s1);
              mu += s0 + s1;
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive_warp_cluster(lbar(TR::kBarGFull));
          }
        }
        // ---- end of the tile ------------------------------------------------------
        // The P warps hand l and the running maximum to the G warps and go straight on to the next
        // tile; the G warps alone normalise and store (they would otherwise idle until the first
        // P and dS of the next tile exist).
        if (p_role) {
          if (!ok) break;
          xl[(tcnt & 1u) * 128 + row] = l;
          xm[(tcnt & 1u) * 128 + row] = m_used;
          mbar_arrive_warp(bar(TR::kBarXchg));
          continue;
        }
        // A G warp only gets here after it has seen dS of the last block, which was issued after the
        // G V product of the block before, so the accumulator barrier is at most one phase ahead.
        if (ok) ok = wait(TR::kBarXchg, tcnt & 1u);
        if (ok) ok = wait_acc(gblk - 1u);
        // the staging tile of the previous pair must have been read by its store
        if (warp == 6 && lane == 0) tma_store_wait_read();
        ok = named_bar_and(1, 128, ok);  // every G warp arrives here, whatever happened to its waits
        if (!ok) break;
        tc_fence_after_sync();
        const float l_tot = xl[(tcnt & 1u) * 128 + row], mu_tot = mu;
        const float inv_l = 1.f / l_tot;
        const float mu_n = mu_tot * inv_l;
        const int64_t lq = q0 + row;
        p.lse[(static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q + lq] =
            (xm[(tcnt & 1u) * 128 + row] + __log2f(l_tot)) * 0.6931471805599453f;
        // Staging tiles have the layout of a TMA box pair: 64 columns with the 128-byte swizzle, then
        // TAIL columns with the tail's swizzle; 16-byte chunk c of row r sits at chunk c ^ f(r).
        uint8_t* st_o = out_stage;
        uint8_t* st_t = out_stage + (TR::kOutBufs - 1) * TR::kTileBytes;
        auto chunk_off = [&](int cc) -> uint32_t {  // cc: head-dim column, a multiple of 8
          if (cc < 64) return static_cast<uint32_t>(row * 128 + (((cc >> 3) ^ (row & 7)) << 4));
          const int ct = (cc - 64) >> 3;
          if constexpr (TAIL == 32)
            return static_cast<uint32_t>(TR::kMainBytes + row * 64 + ((ct ^ ((row >> 1) & 3)) << 4));
          else
            return static_cast<uint32_t>(TR::kMainBytes + row * 32 + ((ct ^ ((row >> 2) & 1)) << 4));
        };
        constexpr int kPasses = (!kF32Out && kDual && TR::kOutBufs == 1) ? 2 : 1;
#pragma unroll
        for (int pass = 0; pass < kPasses; ++pass) {
          const bool do_o = kF32Out || TR::kOutBufs == 2 || pass == 0;
          const bool do_t = kDual && (kF32Out || TR::kOutBufs == 2 || pass == 1);
#pragma unroll
          for (int c = 0; c < DPAD / 16; ++c) {
            uint32_t a[16], t[16];
            tmem_ld_x16(t_o + c * 16, a);
            if (do_t) tmem_ld_x16(t_o + DPAD + c * 16, t);
            tmem_wait_ld();
            if constexpr (kF32Out) {
              // fp32 results straight to global memory, 8 columns (two 16-byte stores) at a time
              float* go = static_cast<float*>(p.o) + static_cast<int64_t>(b) * p.o_sb + lq * p.o_sl + static_cast<int64_t>(h) * p.o_sh;
              float* gt = kDual ? static_cast<float*>(p.to) + static_cast<int64_t>(b) * p.to_sb + lq * p.to_sl + static_cast<int64_t>(h) * p.to_sh : nullptr;
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const int col = pair_head_col<TR>(c * 16 + hh * 8);
                if (col < p.head_dim) {  // accumulator columns past head_dim hold the zero padding
                  float fo[8], ft[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    fo[i] = __uint_as_float(a[hh * 8 + i]) * inv_l;
                    ft[i] = kDual ? fmaf(__uint_as_float(t[hh * 8 + i]), inv_l, -mu_n * fo[i]) : 0.f;
                  }
                  *reinterpret_cast<float4*>(go + col) = make_float4(fo[0], fo[1], fo[2], fo[3]);
                  *reinterpret_cast<float4*>(go + col + 4) = make_float4(fo[4], fo[5], fo[6], fo[7]);
                  if constexpr (kDual) {
                    *reinterpret_cast<float4*>(gt + col) = make_float4(ft[0], ft[1], ft[2], ft[3]);
                    *reinterpret_cast<float4*>(gt + col + 4) = make_float4(ft[4], ft[5], ft[6], ft[7]);
                  }
                }
              }
              continue;
            }
            uint32_t po[8], pt[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float o0 = __uint_as_float(a[2 * i]) * inv_l;
              const float o1 = __uint_as_float(a[2 * i + 1]) * inv_l;
              po[i] = Pack2<T>::pack(o0, o1);
              if (do_t) {
                const float t0 = fmaf(__uint_as_float(t[2 * i]), inv_l, -mu_n * o0);
                const float t1 = fmaf(__uint_as_float(t[2 * i + 1]), inv_l, -mu_n * o1);
                pt[i] = Pack2<T>::pack(t0, t1);
              }
            }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const uint32_t off = chunk_off(pair_head_col<TR>(c * 16 + hh * 8));  // accumulator -> head-dim column
              if (do_o)
                *reinterpret_cast<uint4*>(st_o + off) = make_uint4(po[4 * hh], po[4 * hh + 1], po[4 * hh + 2], po[4 * hh + 3]);
              if (do_t)
                *reinterpret_cast<uint4*>(st_t + off) = make_uint4(pt[4 * hh], pt[4 * hh + 1], pt[4 * hh + 2], pt[4 * hh + 3]);
            }
          }
          if (pass == kPasses - 1) {  // O and T are in registers / shared memory: the next tile may overwrite them
            tc_fence_before_sync();
            mbar_arrive_warp_cluster(lbar(TR::kBarAccEmpty));
          }
          if constexpr (kF32Out) continue;  // nothing was staged
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (warp == 6 && lane == 0) {
            if (do_o) {
              tma_store_4d(&p.o_main, smem_u32(st_o), 0, q0, h, b);
              if constexpr (TAIL > 0) tma_store_4d(&p.o_tail, smem_u32(st_o) + TR::kMainBytes, 64, q0, h, b);
            }
            if (do_t) {
              tma_store_4d(&p.to_main, smem_u32(st_t), 0, q0, h, b);
              if constexpr (TAIL > 0) tma_store_4d(&p.to_tail, smem_u32(st_t) + TR::kMainBytes, 64, q0, h, b);
            }
            tma_store_commit();
            if (kPasses == 2 && pass == 0) tma_store_wait_read();
          }
          if (kPasses == 2 && pass == 0) named_bar_sync(1, 128);  // the shared tile is free for T
        }
      }
      if (!p_role && warp == 6 && lane == 0) tma_store_wait_all();
    }
  }

  // ============================== teardown ==================================
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // nobody leaves (or frees tensor memory) while the other CTA may still touch this one
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc_pair(tmem, TR::kTmemCols);
}

}  // namespace dmf
