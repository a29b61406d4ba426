// Primal backward of attention for sm_100a, role-split variant (head_dim <= 96).
//
// Same two passes, operands and products as attn_bwd.cuh (see its header), but the per-block
// arithmetic is split between two groups of four warps that run side by side, the way the dual
// forward splits S -> P and dS -> G:
//
//   P warps (2-5)  S -> P = exp2(S*c - lse*log2e), 16-bit, into tensor-memory columns of its own
//   D warps (6-9)  dP, P -> dS = P * (dP - delta), 16-bit, over the dP columns; epilogue
//
// With P out of the S columns the next S can be issued as soon as the P warps hold the current one
// in registers, so S runs two blocks ahead of the accumulating products (three ring stages), and
// the P warps go on to the next tile while the D warps write the previous one out.
//
//   issue order per tile:  S_0 dP_0 S_1 | [dV += P_0^T dO_0] acc0 += dS_0 X_0, dP_1, S_2 | ...
//
// One tcgen05.commit costs the issuing thread about 120 cycles, so the commit that frees ring slot
// j % 3 also tells the D warps that the accumulators hold everything up to block j.
#pragma once

#include "attn_bwd.cuh"

namespace dmf {

constexpr int kBwdSplitThreads = 320;  // TMA warp, MMA warp, four P warps, four D warps

template <int TAIL>
struct BwdSplitTraits {
  static_assert(TAIL == 0 || TAIL == 16 || TAIL == 32, "P needs 64 tensor-memory columns of its own");
  static constexpr int kDPad = 64 + TAIL;
  static constexpr int kMainBytes = 128 * 128;
  static constexpr int kTailBytes = 128 * TAIL * 2;
  static constexpr int kTileBytes = kMainBytes + kTailBytes;
  static constexpr int kGroupBytes = 2 * kTileBytes;
  static constexpr int kStages = 3;
  static constexpr int kVecBytes = 2 * 128 * 4;  // per stage: -lse2[128], delta[128]
  static constexpr int kRingBytes = kGroupBytes * (1 + kStages);
  // One tile-shaped buffer stages the outputs for their TMA stores; the dQ pass has a second one for
  // the forward output o (delta = rowsum(dO * o) is computed from shared memory), or, where that does
  // not fit (head_dim 96), lets o share the staging tile.
  static constexpr bool kOwnOTile = TAIL < 32;
  static constexpr int kTileSmem = kRingBytes + kTileBytes * (kOwnOTile ? 2 : 1);
  static constexpr int kBarRFull = 0, kBarREmpty = 1, kBarSFull = 2, kBarDFull = 3, kBarPFull = 4, kBarGFull = 5,
                       kBarSEmpty = 6, kBarPEmpty = 7, kBarAccEmpty = 8, kBarOFull = 9, kBarOEmpty = 10, kBarDEmpty = 11,
                       kBarXFull = 12,
                       kBarXEmpty = kBarXFull + kStages, kNumBars = kBarXEmpty + kStages;
  static constexpr int kSmemBytes = 1024 + kTileSmem + kStages * kVecBytes + kNumBars * 8 + 16;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  static constexpr uint32_t kColS = 0, kColD = 128, kColAcc0 = 256, kColAcc1 = 256 + kDPad, kColP = 256 + 2 * kDPad;
  static_assert(kColP + 64 <= 512, "tensor memory");
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTailSwizzle = TAIL == 32 ? kSwizzle64 : kSwizzle32;
  static constexpr uint32_t kTailRowBytes = 2 * TAIL;
};

template <typename T, int TAIL, int kMode>
__global__ void __launch_bounds__(kBwdSplitThreads, 1)
attn_bwd_split_kernel(const __grid_constant__ BwdParams p) {
  using TR = BwdSplitTraits<TAIL>;
  constexpr int DPAD = TR::kDPad;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr bool kDKV = (kMode == kModeDKV);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_r = smem_u32(smem);
  const uint32_t s_x = s_r + TR::kGroupBytes;
  uint8_t* stage = smem + TR::kRingBytes;                                              // output staging tile
  uint8_t* o_tile = TR::kOwnOTile ? smem + TR::kRingBytes + TR::kTileBytes : stage;    // forward output o (dQ pass)
  float* vec = reinterpret_cast<float*>(smem + TR::kTileSmem);  // [stage][2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::kTileSmem + TR::kStages * TR::kVecBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + TR::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) -> uint32_t { return bar0 + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int J = p.inner_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < TR::kNumBars; ++i) {
      uint32_t count = 1;  // TMA transaction or tcgen05.commit
      if (i == TR::kBarPFull || i == TR::kBarGFull || i == TR::kBarSEmpty || i == TR::kBarAccEmpty ||
          i == TR::kBarDEmpty)
        count = 4;                                       // one arrival per warp of a group
      if (i == TR::kBarOEmpty && TR::kOwnOTile) count = 4;  // the D warps have read o (else: one thread, after the stores)
      if (i == TR::kBarPEmpty) count = kDKV ? 5u : 4u;   // the D warps (+ the commit behind dV += P^T dO)
      mbar_init(bar(i), count);
    }
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), TR::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // =========================== TMA producer ===============================
    if (lane == 0) {
      prefetch_tensor_map(&p.r0_main);
      prefetch_tensor_map(&p.x0_main);
      uint32_t xcnt = 0, tcnt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt) {
        const int bh = tile / p.tiles_per_bh;
        const int r0 = (tile % p.tiles_per_bh) * 128;
        const int b = bh / p.heads, h = bh % p.heads;
        ok = mbar_wait(bar(TR::kBarREmpty), (tcnt & 1u) ^ 1u, abort_flag, p.status_word,
                       kRoleProducer + TR::kBarREmpty);
        if (!ok) break;
        const uint32_t rf = bar(TR::kBarRFull);
        mbar_arrive_expect_tx(rf, TR::kGroupBytes);
        tma_load_4d(s_r, &p.r0_main, rf, 0, r0, h, b);
        tma_load_4d(s_r + TR::kTileBytes, &p.r1_main, rf, 0, r0, h, b);
        if constexpr (TAIL > 0) {
          tma_load_4d(s_r + TR::kMainBytes, &p.r0_tail, rf, 64, r0, h, b);
          tma_load_4d(s_r + TR::kTileBytes + TR::kMainBytes, &p.r1_tail, rf, 64, r0, h, b);
        }
        if constexpr (!kDKV) {  // the forward output of this query tile, for delta
          ok = mbar_wait(bar(TR::kBarOEmpty), (tcnt & 1u) ^ 1u, abort_flag, p.status_word,
                         kRoleProducer + TR::kBarOEmpty);
          if (!ok) break;
          const uint32_t of = bar(TR::kBarOFull), od = smem_u32(o_tile);
          mbar_arrive_expect_tx(of, TR::kTileBytes);
          tma_load_4d(od, &p.o_main, of, 0, r0, h, b);
          if constexpr (TAIL > 0) tma_load_4d(od + TR::kMainBytes, &p.o_tail, of, 64, r0, h, b);
        }
        for (int j = 0; j < J; ++j, ++xcnt) {
          const uint32_t s = xcnt % TR::kStages, ph = (xcnt / TR::kStages) & 1u;
          ok = mbar_wait(bar(TR::kBarXEmpty + s), ph ^ 1u, abort_flag, p.status_word,
                         kRoleProducer + TR::kBarXEmpty);
          if (!ok) break;
          const uint32_t dst = s_x + s * TR::kGroupBytes, fb = bar(TR::kBarXFull + s);
          mbar_arrive_expect_tx(fb, TR::kGroupBytes + (kDKV ? TR::kVecBytes : 0));
          tma_load_4d(dst, &p.x0_main, fb, 0, j * 128, h, b);
          tma_load_4d(dst + TR::kTileBytes, &p.x1_main, fb, 0, j * 128, h, b);
          if constexpr (TAIL > 0) {
            tma_load_4d(dst + TR::kMainBytes, &p.x0_tail, fb, 64, j * 128, h, b);
            tma_load_4d(dst + TR::kTileBytes + TR::kMainBytes, &p.x1_tail, fb, 64, j * 128, h, b);
          }
          if constexpr (kDKV) {
            const int64_t off = (static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q + j * 128;
            const uint32_t vdst = smem_u32(vec + s * 256);
            bulk_load_1d(vdst, p.ws_neg_lse2 + off, 512, fb);
            bulk_load_1d(vdst + 512, p.ws_delta + off, 512, fb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ================================
    // Warp-uniform control flow, one elected lane issues.  Blocks are counted through all tiles of
    // this CTA (g); block g sits in ring slot g % kStages.
    const bool leader = elect_one();
    auto commit = [&](int b_) { tc_commit(bar(b_), leader); };
    constexpr uint32_t idesc_qk = make_idesc(kBf16, false, false, 128, 128);
    constexpr uint32_t idesc_pv_main = make_idesc(kBf16, false, true, 128, 64);
    constexpr uint32_t idesc_pv_tail = make_idesc(kBf16, false, true, 128, TAIL > 0 ? TAIL : 16);
    const uint32_t t_s = tmem + TR::kColS, t_d = tmem + TR::kColD, t_p = tmem + TR::kColP;
    const uint32_t t_a0 = tmem + TR::kColAcc0, t_a1 = tmem + TR::kColAcc1;
    uint32_t g0 = 0, tcnt = 0;  // g0: number of the tile's first block
    bool ok = true;
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleMma + b_);
    };
    auto x_addr = [&](uint32_t g) -> uint32_t { return s_x + (g % TR::kStages) * TR::kGroupBytes; };
    // S of block g (g0 + j): the P warps hold the S before it in registers, the streamed tiles are there
    auto issue_s = [&](uint32_t g) -> bool {
      if (g > 0u && !wait(TR::kBarSEmpty, (g - 1u) & 1u)) return false;
      if (!wait(TR::kBarXFull + g % TR::kStages, (g / TR::kStages) & 1u)) return false;
      tc_fence_after_sync();
      issue_qk<TAIL, TR>(leader, t_s, s_r, x_addr(g), idesc_qk, false);  // S = R0 X0^T
      commit(TR::kBarSFull);
      return true;
    };
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt, g0 += static_cast<uint32_t>(J)) {
      ok = wait(TR::kBarRFull, tcnt & 1u);
      if (!ok) break;
      ok = issue_s(g0);
      if (!ok) break;
      issue_qk<TAIL, TR>(leader, t_d, s_r + TR::kTileBytes, x_addr(g0) + TR::kTileBytes, idesc_qk, false);  // dP = R1 X1^T
      commit(TR::kBarDFull);
      if (J == 1) commit(TR::kBarREmpty);
      if (J > 1) {
        ok = issue_s(g0 + 1u);
        if (!ok) break;
      }
      for (int j = 0; j < J; ++j) {
        const uint32_t g = g0 + static_cast<uint32_t>(j);
        const uint32_t xt = x_addr(g);
        if (j == 0 && tcnt > 0) {  // the epilogue of the previous tile has read the accumulators
          ok = wait(TR::kBarAccEmpty, (tcnt - 1u) & 1u);
          if (!ok) break;
        }
        if constexpr (kDKV) {  // dV += P^T dO
          ok = wait(TR::kBarPFull, g & 1u);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv<TAIL, TR>(leader, t_a1, t_p, xt + TR::kTileBytes, idesc_pv_main, idesc_pv_tail, j > 0);
          commit(TR::kBarPEmpty);
        }
        // dP of the next block (its streamed tiles were awaited for S).  In the dQ pass dS has columns of
        // its own (there is only one accumulator), so dP can be overwritten as soon as the D warps hold it
        // in registers and is computed while they work; in the dK/dV pass dS lives in the dP columns and
        // the next dP has to follow the product that reads it.
        auto issue_next_dp = [&]() {
          issue_qk<TAIL, TR>(leader, t_d, s_r + TR::kTileBytes, x_addr(g + 1u) + TR::kTileBytes, idesc_qk, false);
          commit(TR::kBarDFull);
          if (j + 2 == J) commit(TR::kBarREmpty);
        };
        if constexpr (!kDKV) {
          if (j + 1 < J) {
            ok = wait(TR::kBarDEmpty, g & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            issue_next_dp();
          }
        }
        ok = wait(TR::kBarGFull, g & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        issue_pv<TAIL, TR>(leader, t_a0, kDKV ? t_d : t_a1, xt, idesc_pv_main, idesc_pv_tail, j > 0);  // dQ += dS K  /  dK += dS^T Q
        commit(TR::kBarXEmpty + g % TR::kStages);  // slot free, and "accumulators hold block g" for the D warps
        if constexpr (kDKV) {
          if (j + 1 < J) issue_next_dp();
        }
        if (j + 2 < J) {
          ok = issue_s(g + 2u);
          if (!ok) break;
        }
      }
    }
  } else {
    // ====================== P warps and D warps =============================
    const bool p_role = warp < 6;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem + lane_base + TR::kColS, t_d = tmem + lane_base + TR::kColD;
    const uint32_t t_p = tmem + lane_base + TR::kColP, t_a0 = tmem + lane_base + TR::kColAcc0;
    const float sl2 = p.scale_log2e;
    uint32_t gblk = 0, tcnt = 0;
    bool ok = true;
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
    };
    // Tiles in shared memory have the layout of a TMA box pair: 64 columns with the 128-byte swizzle, then
    // TAIL columns with the tail's swizzle; 16-byte chunk k of row r sits at chunk k ^ f(r).
    auto chunk_off = [&](int cc) -> uint32_t {  // cc: head-dim column, a multiple of 8
      if (cc < 64) return static_cast<uint32_t>(row * 128 + (((cc >> 3) ^ (row & 7)) << 4));
      const int ct = (cc - 64) >> 3;
      if constexpr (TAIL == 32)
        return static_cast<uint32_t>(TR::kMainBytes + row * 64 + ((ct ^ ((row >> 1) & 3)) << 4));
      else
        return static_cast<uint32_t>(TR::kMainBytes + row * 32 + ((ct ^ ((row >> 2) & 1)) << 4));
    };
    const bool mover = (warp == 6 && lane == 0);  // issues the TMA stores
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt) {
      const int bh = tile / p.tiles_per_bh;
      const int r0 = (tile % p.tiles_per_bh) * 128;
      const int b = bh / p.heads, h = bh % p.heads;
      const int64_t lrow = r0 + row;
      float neg_lse2 = 0.f, delta = 0.f;
      if constexpr (!kDKV) {
        // per-row scalars of this query tile; also published for the dK/dV pass
        const int64_t vi = (static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q + lrow;
        if (p_role) {
          neg_lse2 = -p.lse[vi] * 1.4426950408889634f;
          p.ws_neg_lse2[vi] = neg_lse2;
        } else {
          // delta = rowsum(dO * o) from the two shared-memory tiles (dO is the resident tile R1): a thread
          // reads its own row, 16 bytes at a time, at the swizzled position of each chunk
          ok = wait(TR::kBarOFull, tcnt & 1u);
          if (ok) ok = wait(TR::kBarRFull, tcnt & 1u);
          const uint8_t* do_tile = smem + TR::kTileBytes;
          float acc = 0.f;
          if (ok) {  // (a failed wait skips the work, not the meeting at the tile's end)
#pragma unroll
          for (int c = 0; c < DPAD / 8; ++c) {
            const uint32_t off = chunk_off(c * 8);
            const uint4 ov = *reinterpret_cast<const uint4*>(o_tile + off);
            const uint4 dv = *reinterpret_cast<const uint4*>(do_tile + off);
            const uint32_t ou[4] = {ov.x, ov.y, ov.z, ov.w}, du[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 a = unpack2<T>(ou[i]), g = unpack2<T>(du[i]);
              acc = fmaf(a.x, g.x, acc);
              acc = fmaf(a.y, g.y, acc);
            }
          }
            if constexpr (TR::kOwnOTile) mbar_arrive_warp(bar(TR::kBarOEmpty));  // o has been read
            delta = acc;
            p.ws_delta[vi] = delta;
          }
        }
      }
      for (int j = 0; ok && j < J; ++j, ++gblk) {
        const float* vstage = vec + (gblk % TR::kStages) * 256;  // DKV: column vectors of this block
        if constexpr (kDKV) {
          // the vectors arrive with the streamed tiles: observe that barrier directly before reading them
          ok = wait(TR::kBarXFull + (gblk % TR::kStages), (gblk / TR::kStages) & 1u);
          if (!ok) break;
        }
        if (p_role) {
          // ---- P = exp2(S * c - lse2), 16-bit, into the P columns ----------------
          ok = wait(TR::kBarSFull, gblk & 1u);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t r[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, r[c]);
          tmem_wait_ld();
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarSEmpty));  // S is in registers
          const uint64_t sl2_2 = pack_f2(sl2, sl2);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              uint64_t na = pack_f2(neg_lse2, neg_lse2), nb = na;
              if constexpr (kDKV) {
                const float4 nv = *reinterpret_cast<const float4*>(vstage + c * 32 + i);
                na = pack_f2(nv.x, nv.y);
                nb = pack_f2(nv.z, nv.w);
              }
              float x0, x1, x2, x3;
              unpack_f2(fma2(pack_u2(r[c][i], r[c][i + 1]), sl2_2, na), x0, x1);
              unpack_f2(fma2(pack_u2(r[c][i + 2], r[c][i + 3]), sl2_2, nb), x2, x3);
              r[c][i / 2] = Pack2<T>::pack(fast_exp2(x0), fast_exp2(x1));  // packed in place: word k = elements 2k, 2k+1
              r[c][i / 2 + 1] = Pack2<T>::pack(fast_exp2(x2), fast_exp2(x3));
            }
          }
          if (gblk > 0) {  // the readers of the previous P are done with it
            ok = wait(TR::kBarPEmpty, (gblk - 1u) & 1u);
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
          mbar_arrive_warp(bar(TR::kBarPFull));
        } else {
          // ---- dS = P * (dP - delta), 16-bit ------------------------------------------
          if constexpr (kDKV) {
            // over the dP columns (no tensor-memory columns to spare): P first, then dP chunk by chunk
            ok = wait(TR::kBarPFull, gblk & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t pp[4][16];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_x16(t_p + c * 16, pp[c]);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive_warp(bar(TR::kBarPEmpty));  // P has been read
            ok = wait(TR::kBarDFull, gblk & 1u);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t d[32];
              tmem_ld_x32(t_d + c * 32, d);
              tmem_wait_ld();
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; i += 2) {
                const float4 dv = *reinterpret_cast<const float4*>(vstage + 128 + c * 32 + 2 * i);
                const float2 pa = unpack2<T>(pp[c][i]), pb = unpack2<T>(pp[c][i + 1]);
                const float g0 = pa.x * (__uint_as_float(d[2 * i]) - dv.x);
                const float g1 = pa.y * (__uint_as_float(d[2 * i + 1]) - dv.y);
                const float g2 = pb.x * (__uint_as_float(d[2 * i + 2]) - dv.z);
                const float g3 = pb.y * (__uint_as_float(d[2 * i + 3]) - dv.w);
                pk[i] = Pack2<T>::pack(g0, g1);
                pk[i + 1] = Pack2<T>::pack(g2, g3);
              }
              tmem_st_x16(t_d + c * 16, pk);  // over dP columns this thread has already read
            }
          } else {
            // into columns of its own (the second accumulator's, unused in this pass): all of dP goes to
            // registers first and is handed back, so that the next dP is computed during this block's work
            ok = wait(TR::kBarDFull, gblk & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t d[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_x32(t_d + c * 32, d[c]);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive_warp(bar(TR::kBarDEmpty));  // dP is in registers
            ok = wait(TR::kBarPFull, gblk & 1u);
            if (!ok) break;
            if (gblk > 0) {  // the product that read the previous dS is complete (its commit freed the ring slot)
              ok = wait(TR::kBarXEmpty + (gblk - 1u) % TR::kStages, ((gblk - 1u) / TR::kStages) & 1u);
              if (!ok) break;
            }
            tc_fence_after_sync();
            const uint32_t t_ds = tmem + lane_base + TR::kColAcc1;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pc[16];
              tmem_ld_x16(t_p + c * 16, pc);
              tmem_wait_ld();
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; i += 2) {
                const float2 pa = unpack2<T>(pc[i]), pb = unpack2<T>(pc[i + 1]);
                const float g0 = pa.x * (__uint_as_float(d[c][2 * i]) - delta);
                const float g1 = pa.y * (__uint_as_float(d[c][2 * i + 1]) - delta);
                const float g2 = pb.x * (__uint_as_float(d[c][2 * i + 2]) - delta);
                const float g3 = pb.y * (__uint_as_float(d[c][2 * i + 3]) - delta);
                pk[i] = Pack2<T>::pack(g0, g1);
                pk[i + 1] = Pack2<T>::pack(g2, g3);
              }
              tmem_st_x16(t_ds + c * 16, pk);
            }
            tc_fence_before_sync();
            mbar_arrive_warp(bar(TR::kBarPEmpty));  // P has been read
          }
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarGFull));
        }
      }
      if (p_role) {  // the P warps go straight on to the next tile (they take part in no hardware-barrier meeting)
        if (!ok) break;
        continue;
      }
      // a D warp whose wait gave up still goes to the meeting below, so that no other D warp is left alone there
      // ---- epilogue (D warps) -------------------------------------------------
      // the commit behind the last accumulating product of the tile also freed its ring slot
      if (ok) ok = wait(TR::kBarXEmpty + (gblk - 1u) % TR::kStages, ((gblk - 1u) / TR::kStages) & 1u);
      if (mover) tma_store_wait_read();  // the stores of the previous tile have read the staging tile
      ok = named_bar_and(1, 128, ok);    // every D warp arrives here, whatever happened to its waits
      if (!ok) break;
      tc_fence_after_sync();
      // out0 goes to the staging tile at once; out1 (dV) waits in registers until the store of out0 has read it
      uint32_t p1[kDKV ? DPAD / 2 : 1];
      const uint64_t scale2 = pack_f2(p.scale, p.scale);
#pragma unroll
      for (int c = 0; c < DPAD / 16; ++c) {
        uint32_t a[16], v[16];
        tmem_ld_x16(t_a0 + c * 16, a);
        if constexpr (kDKV) tmem_ld_x16(t_a0 + DPAD + c * 16, v);
        tmem_wait_ld();
        uint32_t p0[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float x0, x1;
          unpack_f2(mul2(pack_u2(a[2 * i], a[2 * i + 1]), scale2), x0, x1);
          p0[i] = Pack2<T>::pack(x0, x1);
          if constexpr (kDKV) p1[c * 8 + i] = Pack2<T>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          *reinterpret_cast<uint4*>(stage + chunk_off(c * 16 + hh * 8)) =
              make_uint4(p0[4 * hh], p0[4 * hh + 1], p0[4 * hh + 2], p0[4 * hh + 3]);
      }
      tc_fence_before_sync();
      mbar_arrive_warp(bar(TR::kBarAccEmpty));  // the next tile may overwrite the accumulators
      fence_proxy_async_smem();
      named_bar_sync(1, 128);  // out0 is staged
      const uint32_t stage_addr = smem_u32(stage);
      if (mover) {
        tma_store_4d(&p.out0_main, stage_addr, 0, r0, h, b);
        if constexpr (TAIL > 0) tma_store_4d(&p.out0_tail, stage_addr + TR::kMainBytes, 64, r0, h, b);
        tma_store_commit();
      }
      if constexpr (kDKV) {
        if (mover) tma_store_wait_read();
        named_bar_sync(1, 128);  // the store of out0 has read the tile
#pragma unroll
        for (int c = 0; c < DPAD / 16; ++c) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
            *reinterpret_cast<uint4*>(stage + chunk_off(c * 16 + hh * 8)) =
                make_uint4(p1[c * 8 + 4 * hh], p1[c * 8 + 4 * hh + 1], p1[c * 8 + 4 * hh + 2], p1[c * 8 + 4 * hh + 3]);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);  // out1 is staged
        if (mover) {
          tma_store_4d(&p.out1_main, stage_addr, 0, r0, h, b);
          if constexpr (TAIL > 0) tma_store_4d(&p.out1_tail, stage_addr + TR::kMainBytes, 64, r0, h, b);
          tma_store_commit();
        }
      } else if constexpr (!TR::kOwnOTile) {
        // o of the next tile is loaded into the staging tile: hand it to the producer once the store has read it
        if (mover) {
          tma_store_wait_read();
          mbar_arrive(bar(TR::kBarOEmpty));
        }
      }
    }
    if (mover) tma_store_wait_all();
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem, TR::kTmemCols);
}

}  // namespace dmf
