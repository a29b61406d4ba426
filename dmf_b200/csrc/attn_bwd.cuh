// Primal backward of attention for sm_100a: dq, dk, dv from dout, q, k, v, o, lse.
//
//   P  = exp(scale * Q K^T - lse)          delta = rowsum(dO * O)
//   dP = dO V^T                            dS = P * (dP - delta)
//   dV = P^T dO      dK = scale * dS^T Q      dQ = scale * dS K
//
// Two launches of one persistent warp-specialised kernel template, both built on
// the forward kernel's skeleton (TMA producer warp, one MMA-issuing thread, four
// softmax warps with thread = accumulator row, scores and their gradients in
// tensor memory):
//
//   kModeDQ   a tile is 128 query rows; (Q, dO) stay resident, (K, V) blocks stream.
//             S = Q K^T, dP = dO V^T, dQ += dS K.  It also computes delta and
//             -lse*log2(e) per row and stores both in the workspace.
//   kModeDKV  a tile is 128 key rows; (K, V) stay resident, (Q, dO) blocks stream
//             together with the matching workspace rows (delta, -lse*log2e).
//             S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q.
//
// Scores are recomputed in both passes (7 matrix products instead of the minimal 5);
// in exchange nothing is accumulated across CTAs: no atomics, no fp32 gradient
// buffer, bit-reproducible results.  The only scratch is the workspace of
// 2 * B * H * Lq floats.
#pragma once

#include "attn_fwd.cuh"

namespace dmf {

constexpr int kModeDQ = 0, kModeDKV = 1;
constexpr int kBwdThreads = 192;  // TMA warp, MMA warp, one softmax warpgroup

struct BwdParams {
  // resident / streamed operand maps, "main" = columns [0,64), "tail" = [64, 64+TAIL)
  CUtensorMap r0_main, r0_tail, r1_main, r1_tail;  // DQ: Q, dO      DKV: K, V
  CUtensorMap x0_main, x0_tail, x1_main, x1_tail;  // DQ: K, V       DKV: Q, dO
  // role-split kernel: the forward output as a TMA load map (DQ mode), the outputs as TMA store maps
  CUtensorMap o_main, o_tail, out0_main, out0_tail, out1_main, out1_tail;
  // DQ mode: rows of o and dout for delta, lse; outputs
  const void* o;
  const void* dout;
  int64_t o_sb, o_sl, o_sh;
  int64_t do_sb, do_sl, do_sh;
  const float* lse;
  float* ws_neg_lse2;  // workspace: -lse * log2(e), (B, H, Lq)
  float* ws_delta;     // workspace: rowsum(dO * O), (B, H, Lq)
  void* out0;          // DQ: dq   DKV: dk
  void* out1;          // DKV: dv
  int64_t out0_sb, out0_sl, out0_sh;
  int64_t out1_sb, out1_sl, out1_sh;
  int32_t* status_word;
  int batch, heads, seqlen_q, seqlen_kv, head_dim;
  int tiles_per_bh;   // tiles along the resident sequence
  int num_tiles;
  int inner_blocks;   // blocks along the streamed sequence
  float scale, scale_log2e;
};

template <int TAIL>
struct BwdTraits {
  static constexpr int kDPad = 64 + TAIL;
  static constexpr int kMainBytes = 128 * 128;
  static constexpr int kTailBytes = 128 * TAIL * 2;
  static constexpr int kTileBytes = kMainBytes + kTailBytes;
  static constexpr int kGroupBytes = 2 * kTileBytes;
  static constexpr int kStages = 2;
  static constexpr int kVecBytes = 2 * 128 * 4;  // per stage: -lse2[128], delta[128]
  static constexpr int kTileSmem = kGroupBytes * (1 + kStages);
  static constexpr int kBarRFull = 0, kBarREmpty = 1, kBarSFull = 2, kBarDFull = 3, kBarPFull = 4,
                       kBarGFull = 5, kBarAccFull = 6, kBarXFull = 7, kBarXEmpty = kBarXFull + kStages,
                       kNumBars = kBarXEmpty + kStages;
  static constexpr int kSmemBytes = 1024 + kTileSmem + kStages * kVecBytes + kNumBars * 8 + 16;
  static constexpr uint32_t kColS = 0, kColD = 128, kColAcc0 = 256, kColAcc1 = 256 + kDPad;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTailSwizzle = TAIL == 64 ? kSwizzle128 : (TAIL == 32 ? kSwizzle64 : kSwizzle32);
  static constexpr uint32_t kTailRowBytes = 2 * TAIL;
};

// 1-D bulk copy global -> shared, completion counted on an mbarrier (16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

template <typename T, int TAIL, int kMode>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ BwdParams p) {
  using TR = BwdTraits<TAIL>;
  constexpr int DPAD = TR::kDPad;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr bool kDKV = (kMode == kModeDKV);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_r = smem_u32(smem);
  const uint32_t s_x = s_r + TR::kGroupBytes;
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
    for (int i = 0; i < TR::kNumBars; ++i)
      mbar_init(bar(i), (i == TR::kBarPFull || i == TR::kBarGFull) ? 4u : 1u);  // one arrival per softmax warp
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
    {
      const bool leader = elect_one();
      auto commit = [&](int b_) { tc_commit(bar(b_), leader); };
      constexpr uint32_t idesc_qk = make_idesc(kBf16, false, false, 128, 128);
      constexpr uint32_t idesc_pv_main = make_idesc(kBf16, false, true, 128, 64);
      constexpr uint32_t idesc_pv_tail = make_idesc(kBf16, false, true, 128, TAIL > 0 ? TAIL : 16);
      const uint32_t t_s = tmem + TR::kColS, t_d = tmem + TR::kColD;
      const uint32_t t_a0 = tmem + TR::kColAcc0, t_a1 = tmem + TR::kColAcc1;
      uint32_t xcnt = 0, tcnt = 0, pcnt = 0, gcnt = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        // no vote: a lane can only disagree once the abort flag is up, and nothing below needs convergence
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleMma + b_);
      };
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt) {
        ok = wait(TR::kBarRFull, tcnt & 1u);
        if (!ok) break;
        uint32_t s = xcnt % TR::kStages;
        ok = wait(TR::kBarXFull + s, (xcnt / TR::kStages) & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t xt = s_x + s * TR::kGroupBytes;
        issue_qk<TAIL, TR>(leader, t_s, s_r, xt, idesc_qk, false);                                    // S  = R0 X0^T
        commit(TR::kBarSFull);
        issue_qk<TAIL, TR>(leader, t_d, s_r + TR::kTileBytes, xt + TR::kTileBytes, idesc_qk, false);  // dP = R1 X1^T
        commit(TR::kBarDFull);
        if (J == 1) commit(TR::kBarREmpty);
        for (int j = 0; j < J; ++j) {
          const uint32_t s_cur = s, xt_cur = xt;
          ok = wait(TR::kBarPFull, pcnt & 1u);
          if (!ok) break;
          ++pcnt;
          tc_fence_after_sync();
          if constexpr (kDKV)  // dV += P^T dO
            issue_pv<TAIL, TR>(leader, t_a1, t_s, xt_cur + TR::kTileBytes, idesc_pv_main, idesc_pv_tail, j > 0);
          const bool more = (j + 1 < J);
          if (more) {
            s = (xcnt + 1) % TR::kStages;
            ok = wait(TR::kBarXFull + s, ((xcnt + 1) / TR::kStages) & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            xt = s_x + s * TR::kGroupBytes;
            issue_qk<TAIL, TR>(leader, t_s, s_r, xt, idesc_qk, false);
            commit(TR::kBarSFull);
          }
          ok = wait(TR::kBarGFull, gcnt & 1u);
          if (!ok) break;
          ++gcnt;
          tc_fence_after_sync();
          issue_pv<TAIL, TR>(leader, t_a0, t_d, xt_cur, idesc_pv_main, idesc_pv_tail, j > 0);  // dQ += dS K   /   dK += dS^T Q
          commit(TR::kBarAccFull);
          commit(TR::kBarXEmpty + s_cur);
          ++xcnt;
          if (more) {
            issue_qk<TAIL, TR>(leader, t_d, s_r + TR::kTileBytes, xt + TR::kTileBytes, idesc_qk, false);
            commit(TR::kBarDFull);
            if (j + 2 == J) commit(TR::kBarREmpty);
          }
        }
      }
    }
  } else {
    // ============================ softmax warps =============================
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem + lane_base + TR::kColS, t_d = tmem + lane_base + TR::kColD;
    const uint32_t t_a0 = tmem + lane_base + TR::kColAcc0;
    const float sl2 = p.scale_log2e;
    uint32_t gblk = 0;
    bool ok = true;
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
    };
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      const int bh = tile / p.tiles_per_bh;
      const int r0 = (tile % p.tiles_per_bh) * 128;
      const int b = bh / p.heads, h = bh % p.heads;
      const int64_t lrow = r0 + row;
      float neg_lse2 = 0.f, delta = 0.f;
      if constexpr (!kDKV) {
        // per-row scalars of this query tile; also published for the dK/dV pass
        const int64_t vi = (static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q + lrow;
        neg_lse2 = -p.lse[vi] * 1.4426950408889634f;
        const uint4* o4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.o) + b * p.o_sb +
                                                         lrow * p.o_sl + h * p.o_sh);
        const uint4* d4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.dout) + b * p.do_sb +
                                                         lrow * p.do_sl + h * p.do_sh);
        float acc = 0.f;
        for (int c = 0; c < p.head_dim / 8; ++c) {
          const uint4 ov = __ldg(o4 + c), dv = __ldg(d4 + c);
          const uint32_t ou[4] = {ov.x, ov.y, ov.z, ov.w}, du[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 a = unpack2<T>(ou[i]), g = unpack2<T>(du[i]);
            acc = fmaf(a.x, g.x, acc);
            acc = fmaf(a.y, g.y, acc);
          }
        }
        delta = acc;
        p.ws_neg_lse2[vi] = neg_lse2;
        p.ws_delta[vi] = delta;
      }
      for (int j = 0; j < J; ++j, ++gblk) {
        const float* vstage = vec + (gblk % TR::kStages) * 256;  // DKV: column vectors of this block
        if constexpr (kDKV) {
          // the vectors arrive with the streamed tiles: observe that barrier directly before reading them
          ok = wait(TR::kBarXFull + (gblk % TR::kStages), (gblk / TR::kStages) & 1u);
          if (!ok) break;
        }
        // ---- part 1: P = exp2(S * c - lse2) ----------------------------------
        ok = wait(TR::kBarSFull, gblk & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, r[c]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float n0 = neg_lse2, n1 = neg_lse2, n2 = neg_lse2, n3 = neg_lse2;
            if constexpr (kDKV) {
              const float4 nv = *reinterpret_cast<const float4*>(vstage + c * 32 + i);
              n0 = nv.x; n1 = nv.y; n2 = nv.z; n3 = nv.w;
            }
            r[c][i] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r[c][i]), sl2, n0)));
            r[c][i + 1] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r[c][i + 1]), sl2, n1)));
            r[c][i + 2] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r[c][i + 2]), sl2, n2)));
            r[c][i + 3] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(r[c][i + 3]), sl2, n3)));
          }
        }
        if constexpr (kDKV) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pk[i] = Pack2<T>::pack(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
            tmem_st_x16(t_s + c * 16, pk);
          }
          tmem_wait_st();
        }
        tc_fence_before_sync();
        mbar_arrive_warp(bar(TR::kBarPFull));  // DQ: S has been read;  DKV: P^T is in tensor memory

        // ---- part 2: dS = P * (dP - delta) -----------------------------------
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
            float e0 = delta, e1 = delta, e2 = delta, e3 = delta;
            if constexpr (kDKV) {
              const float4 dv = *reinterpret_cast<const float4*>(vstage + 128 + c * 32 + 2 * i);
              e0 = dv.x; e1 = dv.y; e2 = dv.z; e3 = dv.w;
            }
            const float g0 = __uint_as_float(r[c][2 * i]) * (__uint_as_float(d[2 * i]) - e0);
            const float g1 = __uint_as_float(r[c][2 * i + 1]) * (__uint_as_float(d[2 * i + 1]) - e1);
            const float g2 = __uint_as_float(r[c][2 * i + 2]) * (__uint_as_float(d[2 * i + 2]) - e2);
            const float g3 = __uint_as_float(r[c][2 * i + 3]) * (__uint_as_float(d[2 * i + 3]) - e3);
            pk[i] = Pack2<T>::pack(g0, g1);
            pk[i + 1] = Pack2<T>::pack(g2, g3);
          }
          tmem_st_x16(t_d + c * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(bar(TR::kBarGFull));
      }
      if (!ok) break;
      // ---- epilogue --------------------------------------------------------
      ok = wait(TR::kBarAccFull, (gblk - 1u) & 1u);
      if (!ok) break;
      tc_fence_after_sync();
      T* out0_row = reinterpret_cast<T*>(p.out0) + b * p.out0_sb + lrow * p.out0_sl + h * p.out0_sh;
      T* out1_row = kDKV ? reinterpret_cast<T*>(p.out1) + b * p.out1_sb + lrow * p.out1_sl + h * p.out1_sh : nullptr;
#pragma unroll
      for (int c = 0; c < DPAD / 16; ++c) {
        uint32_t a[16], v[16];
        tmem_ld_x16(t_a0 + c * 16, a);
        if constexpr (kDKV) tmem_ld_x16(t_a0 + DPAD + c * 16, v);
        tmem_wait_ld();
        uint32_t p0[8], p1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p0[i] = Pack2<T>::pack(__uint_as_float(a[2 * i]) * p.scale, __uint_as_float(a[2 * i + 1]) * p.scale);
          if constexpr (kDKV) p1[i] = Pack2<T>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int col0 = c * 16 + hh * 8;
          if (col0 < p.head_dim) {
            *reinterpret_cast<uint4*>(out0_row + col0) = make_uint4(p0[4 * hh], p0[4 * hh + 1], p0[4 * hh + 2], p0[4 * hh + 3]);
            if constexpr (kDKV)
              *reinterpret_cast<uint4*>(out1_row + col0) = make_uint4(p1[4 * hh], p1[4 * hh + 1], p1[4 * hh + 2], p1[4 * hh + 3]);
          }
        }
      }
      tc_fence_before_sync();
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem, TR::kTmemCols);
}

}  // namespace dmf
