// Forward attention kernels for sm_100a: the fused forward + tangent ("dual")
// pass and the plain forward, one persistent warp-specialised kernel template.
//
// Work decomposition.  A tile is 128 consecutive query rows of one (batch, head).
// CTA i handles tiles i, i + gridDim.x, ... (one CTA per SM).  Inside a tile the
// KV sequence is walked in blocks of 128 rows with a single online softmax:
//
//   S  = Q K^T                    (tcgen05.mma, operands in shared memory)
//   dS = dQ K^T + Q dK^T          (two MMAs into one accumulator)
//   P  = exp2(S*c - m),  G = P * dS * scale        (softmax warps, registers)
//   O += P V,   T += P dV + G V   (tcgen05.mma, P / G read from tensor memory)
//
// running m (lazily updated max), l = sum P, mu = sum G; epilogue
//   o = O / l,   to = T / l - (mu / l) o,   lse = ln2 * (m + log2 l).
//
// Warp roles (320 threads):
//   warp 0     TMA producer: Q/dQ tile, then K/dK and V/dV blocks through two
//              shared-memory rings; also owns the tensor-memory allocation
//   warp 1     MMA issuer (warp-uniform control flow, one elected lane issues)
//   warps 2-9  softmax + correction + epilogue, two warpgroups: thread = one query
//              row (tensor-memory lane quarter = warp_id % 4) x one half of the
//              128 score columns
//
// Tensor memory columns (fp32 accumulators, 128 lanes):
//   [0,128)   S
//   [128,256) dS; G (16-bit) is written over its columns [0,32) and [64,96)
//   [256,320) P (16-bit), dual pass with DPAD <= 96; otherwise P is written over S like G over dS
//             (plain forward: [128,256) is the second S buffer)
//   then O (DPAD columns) and, dual only, T (DPAD columns)
//
// Head dim D is handled as a 64-column main part (128-byte swizzle) plus a tail
// of TAIL in {0,16,32,64} columns (swizzle of 2*TAIL bytes); columns past D in
// the tail are zero-filled by TMA and contribute nothing.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "sm100_ptx.cuh"

namespace dmf {

constexpr int kBlockQ = 128;
constexpr int kBlockKV = 128;
constexpr int kFwdThreads = 320;       // TMA warp, MMA warp, two softmax warpgroups
constexpr int kSoftmaxWarps = 8;
constexpr float kRescaleThreshold = 8.0f;
// Of every kPolyEvery groups of four score elements, one group computes two of its four exp2 on
// the FMA pipe (cubic) instead of the MUFU unit: 1 -> half of all exp2, 2 -> a quarter, 0 -> none.
#ifndef DMF_POLY_EVERY
#define DMF_POLY_EVERY 2
#endif
constexpr int kPolyEvery = DMF_POLY_EVERY;  // log2 units: P stays below 2^8

// Codes written to the status word when a wait gives up: role * 100 + barrier.
constexpr int kRoleProducer = 100, kRoleMma = 200, kRoleSoftmax = 300;

struct FwdParams {
  // TMA maps of (D, L, H, B) views; "main" = columns [0,64), "tail" = [64, 64+TAIL)
  CUtensorMap q_main, q_tail, k_main, k_tail;
  CUtensorMap tq_main, tq_tail, tk_main, tk_tail;
  // V and dV: boxes of 32 columns x 128 rows with 64-byte swizzle ("atoms"), see FwdTraits
  CUtensorMap v_map, tv_map;
  // outputs as TMA store maps (boxes of 128 rows; only the CTA-pair kernel stores through them)
  CUtensorMap o_main, o_tail, to_main, to_tail;
  void* o;
  void* to;
  float* lse;
  int64_t o_sb, o_sl, o_sh;
  int64_t to_sb, to_sl, to_sh;
  int32_t* status_word;
  int batch, heads, seqlen_q, seqlen_kv, head_dim;
  int num_q_tiles, num_tiles;
  float scale, scale_log2e;
  // Sector alignment of head rows (only used for head_dim 72, whose rows are 4.5 sectors of 32 B):
  // a row of (b, h) starts (align0 + b * align_b + h * align_h) mod 32 bytes into a sector.  When
  // that is 16, boxes are started 8 columns early (the 8 columns read as zeros) so that every box
  // begins on a sector boundary; otherwise each misaligned row drags in one or two extra sectors.
  // {qk, v}: the contraction group q, k, tq, tk and the group v, tv; enable = 0 turns a group off.
  int align_enable[2], align0[2], align_b[2], align_h[2];
};

// 8 when the rows of (b, h) start in the middle of a 32-byte sector and the group may be shifted.
__device__ __forceinline__ int column_shift(const FwdParams& p, int grp, int b, int h) {
  if (!p.align_enable[grp]) return 0;
  return (((p.align0[grp] + b * p.align_b[grp] + h * p.align_h[grp]) & 31) == 16) ? 8 : 0;
}

template <int TAIL, bool kDual>
struct FwdTraits {
  static constexpr int kDPad = 64 + TAIL;
  static constexpr int kMainBytes = 128 * 128;
  static constexpr int kTailBytes = 128 * TAIL * 2;
  static constexpr int kTileBytes = kMainBytes + kTailBytes;
  static constexpr int kGroup = kDual ? 2 : 1;  // primal (+ tangent) tile per ring slot
  static constexpr int kGroupBytes = kGroup * kTileBytes;
  static constexpr int kStagesK = 2;
  static constexpr int kStagesV = (kDual && TAIL == 32) ? 1 : 2;
  static constexpr int kStagesK_ = (kDual && TAIL == 64) ? 1 : kStagesK;
  static constexpr int kStagesV_ = (kDual && TAIL == 64) ? 1 : kStagesV;
  // V / dV blocks are the MN-major operand of the P V products.  They are stored as
  // ceil(DPAD/32) atoms of 32 columns x 128 rows (64-byte swizzle) so that one MMA of N = DPAD
  // covers the whole head dim; a split into a 64- and a 16-column MMA costs far more than the
  // 16 extra columns (a tcgen05.mma of N = 16 takes about as long as one of N = 128).
  static constexpr int kVAtoms = (kDPad + 31) / 32;
  static constexpr int kVAtomBytes = 128 * 64;
  static constexpr int kVTileBytes = kVAtoms * kVAtomBytes;
  static constexpr int kVGroupBytes = kGroup * kVTileBytes;
  // The plain forward stages its output tile in shared memory and writes it with TMA stores
  // (thread-per-row 16-byte global stores touch 32 lines per instruction and stall the LSU for
  // thousands of cycles per tile); the dual pass of this kernel has no room for that at head_dim 128.
  static constexpr bool kStageOut = !kDual;
  static constexpr int kRingBytes = kGroupBytes * (1 + kStagesK_) + kVGroupBytes * kStagesV_;
  static constexpr int kTileSmem = kRingBytes + (kStageOut ? kTileBytes : 0);
  // barriers
  static constexpr int kBarQFull = 0, kBarQEmpty = 1, kBarSFull = 2, kBarDSFull = 3, kBarPFull = 4,
                       kBarGFull = 5, kBarAccFull = 6 /* and 7 */, kBarXchg = 8, kBarSEmpty = 9, kBarPEmpty = 10,
                       kBarKFull = 11,
                       kBarKEmpty = kBarKFull + kStagesK_, kBarVFull = kBarKEmpty + kStagesK_,
                       kBarVEmpty = kBarVFull + kStagesV_, kNumBars = kBarVEmpty + kStagesV_;
  static constexpr int kXchgBytes = 4096;  // row max / row sum exchange between the softmax groups
  static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kTileSmem + kXchgBytes + kNumBars * 8 + 16;
  // tensor memory columns
  // Dual pass with room in tensor memory (DPAD <= 96): P gets columns of its own, so S of the
  // next block can be issued as soon as the softmax has read the current S, instead of behind the
  // P V products that read P.  Otherwise P is written over S.
  static constexpr bool kSepP = kDual && (kDPad <= 96);
  // With P in its own columns the two softmax warpgroups split by role instead of by column:
  // one turns S into P (all 128 columns of its row), the other turns dS and P into G.
  static constexpr bool kRoleSplit = kSepP;
  static constexpr uint32_t kColS = 0, kColDS = 128, kColP = 256, kColO = kSepP ? 320 : 256,
                            kColT = kColO + kDPad;
  static constexpr uint32_t kTmemCols = 512;
  // swizzle of the tail part
  static constexpr uint32_t kTailSwizzle = TAIL == 64 ? kSwizzle128 : (TAIL == 32 ? kSwizzle64 : kSwizzle32);
  static constexpr uint32_t kTailRowBytes = 2 * TAIL;
};

// ---- MMA issue helpers: executed by the whole MMA warp, the instruction itself by its leader lane ----

// acc[128 x 128] (+)= A[128 x D] * B[128 x D]^T, both operands K-major in shared memory.
template <int TAIL, typename TR>
__device__ __forceinline__ void issue_qk(bool leader, uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile,
                                         uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const uint64_t ad = make_smem_desc(a_tile + kk * 32, 16, 1024, kSwizzle128);
    const uint64_t bd = make_smem_desc(b_tile + kk * 32, 16, 1024, kSwizzle128);
    mma_ss(d_tmem, ad, bd, idesc, (accumulate || kk > 0) ? 1u : 0u, leader);
  }
#pragma unroll
  for (int kk = 0; kk < TAIL / 16; ++kk) {
    const uint64_t ad = make_smem_desc(a_tile + TR::kMainBytes + kk * 32, 16, 8 * TR::kTailRowBytes,
                                       TR::kTailSwizzle);
    const uint64_t bd = make_smem_desc(b_tile + TR::kMainBytes + kk * 32, 16, 8 * TR::kTailRowBytes,
                                       TR::kTailSwizzle);
    mma_ss(d_tmem, ad, bd, idesc, 1u, leader);
  }
}

// acc[128 x DPAD] (+)= A[128 x 128] * V[128 x DPAD]; A is 16-bit in tensor memory
// (two elements per column), V is MN-major (row = kv index, D contiguous) in shared memory.
template <int TAIL, typename TR>
__device__ __forceinline__ void issue_pv(bool leader, uint32_t d_tmem, uint32_t a_tmem, uint32_t v_tile,
                                         uint32_t idesc_main, uint32_t idesc_tail, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < kBlockKV / 16; ++kk) {
    const uint32_t acc = (accumulate || kk > 0) ? 1u : 0u;
    const uint64_t bd = make_smem_desc(v_tile + kk * (16 * 128), 8192, 1024, kSwizzle128);
    mma_ts(d_tmem, a_tmem + kk * 8, bd, idesc_main, acc, leader);
    if constexpr (TAIL > 0) {
      const uint64_t bt = make_smem_desc(v_tile + TR::kMainBytes + kk * (16 * TR::kTailRowBytes),
                                         TR::kTailBytes, 8 * TR::kTailRowBytes, TR::kTailSwizzle);
      mma_ts(d_tmem + 64, a_tmem + kk * 8, bt, idesc_tail, acc, leader);
    }
  }
}

// Same product with V stored as 64-byte-swizzled atoms of 32 columns: one MMA of N = DPAD per K-step.
// kSplitA: the 16-bit A operand was written over a 128-column fp32 buffer by the two softmax
// groups, k-steps 0-3 in columns [0,32) and k-steps 4-7 in [64,96); otherwise it is contiguous.
template <typename TR, bool kSplitA>
__device__ __forceinline__ void issue_pv_atoms(bool leader, uint32_t d_tmem, uint32_t a_tmem, uint32_t v_tile,
                                               uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < kBlockKV / 16; ++kk) {
    // leading-dim offset = next 32-column atom, stride offset = next group of 8 kv rows
    const uint64_t bd = make_smem_desc(v_tile + kk * (16 * 64), TR::kVAtomBytes, 8 * 64, kSwizzle64);
    const uint32_t a_col = kSplitA ? (kk >> 2) * 64 + (kk & 3) * 8 : kk * 8;
    mma_ts(d_tmem, a_tmem + a_col, bd, idesc, (accumulate || kk > 0) ? 1u : 0u, leader);
  }
}

// ---- the kernel ---------------------------------------------------------------

template <typename T, int TAIL, bool kDual>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ FwdParams p) {
  using TR = FwdTraits<TAIL, kDual>;
  constexpr int DPAD = TR::kDPad;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_k = s_q + TR::kGroupBytes;
  const uint32_t s_v = s_k + TR::kStagesK_ * TR::kGroupBytes;
  float* xchg = reinterpret_cast<float*>(smem + TR::kTileSmem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::kTileSmem + TR::kXchgBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + TR::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) -> uint32_t { return bar0 + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kv_blocks = p.seqlen_kv / kBlockKV;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < TR::kNumBars; ++i) {
      // arrivals: softmax warps arrive once per warp; tcgen05.commit and the TMA producer arrive once
      uint32_t count = 1;
      if (i == TR::kBarXchg) count = kSoftmaxWarps;
      if (i == TR::kBarPFull || i == TR::kBarGFull || i == TR::kBarSEmpty)
        count = TR::kRoleSplit ? kSoftmaxWarps / 2 : kSoftmaxWarps;
      if (i == TR::kBarPEmpty && TR::kRoleSplit) count = 1 + kSoftmaxWarps / 2;  // commit + the G warps
      if (!kDual && i == TR::kBarGFull) count = kSoftmaxWarps;  // plain pass: second "P ready" barrier
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
      prefetch_tensor_map(&p.q_main);
      prefetch_tensor_map(&p.k_main);
      prefetch_tensor_map(&p.v_map);
      uint32_t kcnt = 0, vcnt = 0, tcnt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt) {
        const int bh = tile / p.num_q_tiles;
        const int q0 = (tile % p.num_q_tiles) * kBlockQ;
        const int b = bh / p.heads, h = bh % p.heads;
        ok = mbar_wait(bar(TR::kBarQEmpty), (tcnt & 1u) ^ 1u, abort_flag, p.status_word,
                       kRoleProducer + TR::kBarQEmpty);
        if (!ok) break;
        const int xqk = -column_shift(p, 0, b, h), xv = -column_shift(p, 1, b, h);
        mbar_arrive_expect_tx(bar(TR::kBarQFull), TR::kGroupBytes);
        tma_load_4d(s_q, &p.q_main, bar(TR::kBarQFull), xqk, q0, h, b);
        if constexpr (TAIL > 0) tma_load_4d(s_q + TR::kMainBytes, &p.q_tail, bar(TR::kBarQFull), 64 + xqk, q0, h, b);
        if constexpr (kDual) {
          tma_load_4d(s_q + TR::kTileBytes, &p.tq_main, bar(TR::kBarQFull), xqk, q0, h, b);
          if constexpr (TAIL > 0)
            tma_load_4d(s_q + TR::kTileBytes + TR::kMainBytes, &p.tq_tail, bar(TR::kBarQFull), 64 + xqk, q0, h, b);
        }
        for (int j = 0; j < num_kv_blocks; ++j) {
          const int kv0 = j * kBlockKV;
          {
            const uint32_t s = kcnt % TR::kStagesK_, ph = (kcnt / TR::kStagesK_) & 1u;
            ok = mbar_wait(bar(TR::kBarKEmpty + s), ph ^ 1u, abort_flag, p.status_word,
                           kRoleProducer + TR::kBarKEmpty);
            if (!ok) break;
            const uint32_t dst = s_k + s * TR::kGroupBytes, fb = bar(TR::kBarKFull + s);
            mbar_arrive_expect_tx(fb, TR::kGroupBytes);
            tma_load_4d(dst, &p.k_main, fb, xqk, kv0, h, b);
            if constexpr (TAIL > 0) tma_load_4d(dst + TR::kMainBytes, &p.k_tail, fb, 64 + xqk, kv0, h, b);
            if constexpr (kDual) {
              tma_load_4d(dst + TR::kTileBytes, &p.tk_main, fb, xqk, kv0, h, b);
              if constexpr (TAIL > 0)
                tma_load_4d(dst + TR::kTileBytes + TR::kMainBytes, &p.tk_tail, fb, 64 + xqk, kv0, h, b);
            }
            ++kcnt;
          }
          {
            const uint32_t s = vcnt % TR::kStagesV_, ph = (vcnt / TR::kStagesV_) & 1u;
            ok = mbar_wait(bar(TR::kBarVEmpty + s), ph ^ 1u, abort_flag, p.status_word,
                           kRoleProducer + TR::kBarVEmpty);
            if (!ok) break;
            const uint32_t dst = s_v + s * TR::kVGroupBytes, fb = bar(TR::kBarVFull + s);
            mbar_arrive_expect_tx(fb, TR::kVGroupBytes);
#pragma unroll
            for (int a = 0; a < TR::kVAtoms; ++a) {
              tma_load_4d(dst + a * TR::kVAtomBytes, &p.v_map, fb, a * 32 + xv, kv0, h, b);
              if constexpr (kDual)
                tma_load_4d(dst + TR::kVTileBytes + a * TR::kVAtomBytes, &p.tv_map, fb, a * 32 + xv, kv0, h, b);
            }
            ++vcnt;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ================================
    // The whole warp runs the loops and waits (warp-uniform control flow keeps descriptors in
    // uniform registers); only the elected lane executes tcgen05.mma / tcgen05.commit.
    {
      const bool leader = elect_one();
      auto commit = [&](int b_) { tc_commit(bar(b_), leader); };
      constexpr uint32_t idesc_qk = make_idesc(kBf16, false, false, 128, 128);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, false, true, 128, DPAD);
      const uint32_t t_s = tmem + TR::kColS, t_ds = tmem + TR::kColDS;
      const uint32_t t_o = tmem + TR::kColO, t_t = tmem + TR::kColT;
      uint32_t kcnt = 0, vcnt = 0, tcnt = 0, pcnt = 0, gcnt = 0, scnt = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        // no vote: a lane can only disagree once the abort flag is up, and nothing below needs convergence
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleMma + b_);
      };
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt) {
        ok = wait(TR::kBarQFull, tcnt & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        if constexpr (kDual) {
          constexpr bool kSepP = TR::kSepP;
          const uint32_t t_p = kSepP ? tmem + TR::kColP : t_s;
          // block 0: S and dS
          uint32_t sk = kcnt % TR::kStagesK_;
          if constexpr (kSepP) {
            // S is about to be overwritten: the softmax must have read the previous block's S
            if (scnt > 0) {
              ok = wait(TR::kBarSEmpty, (scnt - 1u) & 1u);
              if (!ok) break;
            }
          }
          ok = wait(TR::kBarKFull + sk, (kcnt / TR::kStagesK_) & 1u);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t kt = s_k + sk * TR::kGroupBytes;
          issue_qk<TAIL, TR>(leader, t_s, s_q, kt, idesc_qk, false);
          commit(TR::kBarSFull);
          ++scnt;
          issue_qk<TAIL, TR>(leader, t_ds, s_q + TR::kTileBytes, kt, idesc_qk, false);
          issue_qk<TAIL, TR>(leader, t_ds, s_q, kt + TR::kTileBytes, idesc_qk, true);
          commit(TR::kBarDSFull);
          commit(TR::kBarKEmpty + sk);
          ++kcnt;
          if (num_kv_blocks == 1) commit(TR::kBarQEmpty);
          for (int j = 0; j < num_kv_blocks; ++j) {
            const uint32_t sv = vcnt % TR::kStagesV_;
            const uint32_t vt = s_v + sv * TR::kVGroupBytes;
            const bool more = (j + 1 < num_kv_blocks);
            // S of the next block.  With a separate P buffer it goes first (the tensor pipe computes
            // it while the softmax of this block runs); with P over S it must follow the readers of P.
            auto issue_next_s = [&]() -> bool {
              sk = kcnt % TR::kStagesK_;
              if constexpr (kSepP) {
                if (!wait(TR::kBarSEmpty, (scnt - 1u) & 1u)) return false;
              }
              if (!wait(TR::kBarKFull + sk, (kcnt / TR::kStagesK_) & 1u)) return false;
              tc_fence_after_sync();
              kt = s_k + sk * TR::kGroupBytes;
              issue_qk<TAIL, TR>(leader, t_s, s_q, kt, idesc_qk, false);
              commit(TR::kBarSFull);
              ++scnt;
              return true;
            };
            if constexpr (kSepP) {
              if (more) {
                ok = issue_next_s();
                if (!ok) break;
              }
            }
            ok = wait(TR::kBarVFull + sv, (vcnt / TR::kStagesV_) & 1u);
            if (!ok) break;
            ok = wait(TR::kBarPFull, pcnt & 1u);
            if (!ok) break;
            ++pcnt;
            tc_fence_after_sync();
            issue_pv_atoms<TR, !kSepP>(leader, t_o, t_p, vt, idesc_pv, j > 0);                    // O += P V
            issue_pv_atoms<TR, !kSepP>(leader, t_t, t_p, vt + TR::kVTileBytes, idesc_pv, j > 0);  // T += P dV
            if constexpr (kSepP) {
              commit(TR::kBarPEmpty);
            } else {
              if (more) {
                ok = issue_next_s();
                if (!ok) break;
              }
            }
            ok = wait(TR::kBarGFull, gcnt & 1u);
            if (!ok) break;
            ++gcnt;
            tc_fence_after_sync();
            issue_pv_atoms<TR, !TR::kRoleSplit>(leader, t_t, t_ds, vt, idesc_pv, true);  // T += G V
            commit(TR::kBarAccFull);
            commit(TR::kBarVEmpty + sv);
            ++vcnt;
            if (more) {
              issue_qk<TAIL, TR>(leader, t_ds, s_q + TR::kTileBytes, kt, idesc_qk, false);
              issue_qk<TAIL, TR>(leader, t_ds, s_q, kt + TR::kTileBytes, idesc_qk, true);
              commit(TR::kBarDSFull);
              commit(TR::kBarKEmpty + sk);
              ++kcnt;
              if (j + 2 == num_kv_blocks) commit(TR::kBarQEmpty);
            }
          }
        } else {
          // plain forward: S double-buffered in the S / dS columns.  Each buffer has its own
          // "S ready" and "P ready" barrier (the dS / G barriers of the dual pass), because S of
          // block g+1 is issued before P of block g is awaited: one barrier shared by both
          // buffers could run two phases ahead of its waiter, which a parity wait cannot express.
          auto issue_s = [&]() -> bool {
            const uint32_t sk = kcnt % TR::kStagesK_;
            if (!wait(TR::kBarKFull + sk, (kcnt / TR::kStagesK_) & 1u)) return false;
            tc_fence_after_sync();
            issue_qk<TAIL, TR>(leader, (scnt & 1u) ? t_ds : t_s, s_q, s_k + sk * TR::kGroupBytes, idesc_qk, false);
            commit(TR::kBarSFull + (scnt & 1u));
            commit(TR::kBarKEmpty + sk);
            ++kcnt;
            ++scnt;
            return true;
          };
          ok = issue_s();
          if (!ok) break;
          if (num_kv_blocks == 1) commit(TR::kBarQEmpty);
          for (int j = 0; j < num_kv_blocks; ++j) {
            if (j + 1 < num_kv_blocks) {
              ok = issue_s();
              if (!ok) break;
              if (j + 2 == num_kv_blocks) commit(TR::kBarQEmpty);
            }
            const uint32_t sv = vcnt % TR::kStagesV_;
            ok = wait(TR::kBarVFull + sv, (vcnt / TR::kStagesV_) & 1u);
            if (!ok) break;
            ok = wait(TR::kBarPFull + (pcnt & 1u), (pcnt >> 1) & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            issue_pv_atoms<TR, true>(leader, t_o, (pcnt & 1u) ? t_ds : t_s, s_v + sv * TR::kVGroupBytes, idesc_pv, j > 0);
            commit(TR::kBarAccFull + (pcnt & 1u));
            ++pcnt;
            commit(TR::kBarVEmpty + sv);
            ++vcnt;
          }
        }
      }
    }
  } else {
    // ===================== softmax / correction / epilogue ==================
    if constexpr (TR::kRoleSplit) {
      // Role split (dual pass, P in its own tensor-memory columns).  Both warpgroups map thread ->
      // query row (lane quarter = warp % 4).  Warps 2-5 ("P warps") turn S into P: row max, lazy
      // rescale of the accumulators, exp2, row sum l.  Warps 6-9 ("G warps") turn dS and the
      // 16-bit P into G = P * dS * scale and keep mu = rowsum(G).  They meet once per tile, in the
      // epilogue, to combine l and mu.  No per-block exchange, and the two halves of the softmax
      // work run concurrently instead of one after the other.
      const bool p_role = warp < 6;
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t t_s = tmem + lane_base + TR::kColS, t_ds = tmem + lane_base + TR::kColDS;
      const uint32_t t_p = tmem + lane_base + TR::kColP, t_o = tmem + lane_base + TR::kColO;
      const float sl2 = p.scale_log2e;
      float* xalpha = xchg;        // [block parity][row]: factor the P warps applied to the accumulators
      float* xsum = xchg + 256;    // [l | mu][row]
      uint32_t gblk = 0, xuse = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
      };
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        const int bh = tile / p.num_q_tiles;
        const int q0 = (tile % p.num_q_tiles) * kBlockQ;
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
            mbar_arrive_warp(bar(TR::kBarSEmpty));  // S is in registers: the next S may be computed
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
                ok = wait(TR::kBarAccFull, (gblk - 1u) & 1u);
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
                if (kPolyEvery > 0 && ((i / 4) % (kPolyEvery > 0 ? kPolyEvery : 1)) == (kPolyEvery - 1)) {
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
            // ---- G = P * dS * scale, mu += rowsum(G) ---------------------------
            // P first: it is ready long before dS, and once it sits in registers its columns can be
            // handed back to the P warps (they would otherwise wait for this whole block of G work).
            ok = wait(TR::kBarPFull, gblk & 1u);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t pp[4][16];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_x16(t_p + c * 16, pp[c]);
            tmem_wait_ld();
            tc_fence_before_sync();
            mu *= xalpha[(gblk & 1u) * 128 + row];
            mbar_arrive_warp(bar(TR::kBarPEmpty));  // P has been read
            ok = wait(TR::kBarDSFull, gblk & 1u);
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
            mbar_arrive_warp(bar(TR::kBarGFull));
          }
        }
        if (!ok) break;
        // ---- epilogue: combine l and mu, normalise, write o, to, lse --------------
        // The meeting comes first: a G warp only gets here after it has seen dS of the last block,
        // which was issued after the G V product of the block before, so once everybody has met the
        // accumulator barrier is at most one phase ahead of any waiter.
        xsum[(p_role ? 0 : 128) + row] = p_role ? l : mu;
        mbar_arrive_warp(bar(TR::kBarXchg));
        ok = wait(TR::kBarXchg, xuse & 1u);
        ++xuse;
        if (!ok) break;
        ok = wait(TR::kBarAccFull, (gblk - 1u) & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        const float l_tot = xsum[row], mu_tot = xsum[128 + row];
        const float inv_l = 1.f / l_tot;
        const float mu_n = mu_tot * inv_l;
        const int vshift = column_shift(p, 1, b, h);
        const int64_t lq = q0 + row;
        T* o_row = reinterpret_cast<T*>(p.o) + b * p.o_sb + lq * p.o_sl + h * p.o_sh;
        T* to_row = reinterpret_cast<T*>(p.to) + b * p.to_sb + lq * p.to_sl + h * p.to_sh;
#pragma unroll
        for (int c = 0; c < DPAD / 16; ++c) {
          if ((c & 1) != (p_role ? 0 : 1)) continue;  // the two groups alternate 16-column chunks
          uint32_t a[16], t[16];
          tmem_ld_x16(t_o + c * 16, a);
          tmem_ld_x16(t_o + DPAD + c * 16, t);
          tmem_wait_ld();
          uint32_t po[8], pt[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float o0 = __uint_as_float(a[2 * i]) * inv_l;
            const float o1 = __uint_as_float(a[2 * i + 1]) * inv_l;
            po[i] = Pack2<T>::pack(o0, o1);
            const float t0 = fmaf(__uint_as_float(t[2 * i]), inv_l, -mu_n * o0);
            const float t1 = fmaf(__uint_as_float(t[2 * i + 1]), inv_l, -mu_n * o1);
            pt[i] = Pack2<T>::pack(t0, t1);
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int cc = c * 16 + hh * 8 - vshift;
            if (cc >= 0 && cc < p.head_dim) {
              *reinterpret_cast<uint4*>(o_row + cc) = make_uint4(po[4 * hh], po[4 * hh + 1], po[4 * hh + 2], po[4 * hh + 3]);
              *reinterpret_cast<uint4*>(to_row + cc) = make_uint4(pt[4 * hh], pt[4 * hh + 1], pt[4 * hh + 2], pt[4 * hh + 3]);
            }
          }
        }
        if (p_role)
          p.lse[(static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q + lq] =
              (m_used + __log2f(l_tot)) * 0.6931471805599453f;
        tc_fence_before_sync();
      }
    } else {
    // Column split (plain forward, and the dual pass when P has to share columns with S).
    // Two warpgroups (warps 2-5 and 6-9).  A thread owns one query row (tensor-memory lane
    // = 32 * (warp % 4) + lane) and one half of the 128 score columns: group g reads S / dS
    // columns [64g, 64g+64) and writes its 16-bit P / G back over the first 32 of those columns
    // (so no thread ever overwrites a column another thread still has to read).  The row max and,
    // in the epilogue, the row sums are combined through shared memory.
    const int grp = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t col0 = 64u * static_cast<uint32_t>(grp);
    const uint32_t t_s = tmem + lane_base + TR::kColS + col0, t_ds = tmem + lane_base + TR::kColDS + col0;
    const uint32_t t_o = tmem + lane_base + TR::kColO;
    const float sl2 = p.scale_log2e;
    float* xmax = xchg;         // [block parity][group][row]
    float* xsum = xchg + 512;   // [l | mu][group][row]
    uint32_t gblk = 0;  // blocks processed so far by this CTA (all tiles)
    uint32_t xuse = 0;  // uses of the exchange barrier
    bool ok = true;
    // warp-uniform result: the warp-wide votes and .sync.aligned instructions below need all 32 lanes
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
    };
    // Wait until the MMAs that accumulate block `blk` into O / T are complete.  A parity wait
    // only works while the barrier is at most one phase ahead of the waiter.  Dual pass: one
    // barrier, one commit per block; by the time this is called for block c the commit of c-1
    // is known complete (the dS of block c, awaited in part 2, was issued after it).  Plain
    // pass: the softmax can run a block ahead of the P V products, so even and odd blocks
    // commit to separate barriers; the commit of c-2 is complete once S of block c has arrived.
    auto wait_acc = [&](uint32_t blk) -> bool {
      return kDual ? wait(TR::kBarAccFull, blk & 1u) : wait(TR::kBarAccFull + (blk & 1u), (blk >> 1) & 1u);
    };
    // All 256 softmax threads meet (bounded, like every other wait); shared-memory writes made
    // before it are visible after it.
    auto exchange = [&]() -> bool {
      mbar_arrive_warp(bar(TR::kBarXchg));
      const bool r_ = wait(TR::kBarXchg, xuse & 1u);
      ++xuse;
      return r_;
    };
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
      const int bh = tile / p.num_q_tiles;
      const int q0 = (tile % p.num_q_tiles) * kBlockQ;
      const int b = bh / p.heads, h = bh % p.heads;
      float m_used = -CUDART_INF_F, l = 0.f, mu = 0.f;  // l, mu: this thread's columns only
      for (int j = 0; j < num_kv_blocks; ++j, ++gblk) {
        // ---- part 1: S -> P ------------------------------------------------
        const uint32_t buf = kDual ? 0u : (gblk & 1u);
        ok = wait(TR::kBarSFull + buf, kDual ? (gblk & 1u) : ((gblk >> 1) & 1u));
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t t_sb = buf ? t_ds : t_s;
        uint32_t r[2][32];
        tmem_ld_x32(t_sb, r[0]);
        tmem_ld_x32(t_sb + 32, r[1]);
        tmem_wait_ld();
        if constexpr (TR::kSepP) {  // S is in registers: the MMA warp may overwrite it with the next block's S
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarSEmpty));
        }
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            mx0 = max3(mx0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
            mx1 = max3(mx1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
            mx2 = max3(mx2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
            mx3 = max3(mx3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
          }
        }
        const float m_loc = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        float* xm = xmax + (gblk & 1u) * 256;
        xm[grp * 128 + row] = m_loc;
        ok = exchange();
        if (!ok) break;
        const float m_blk = fmaxf(m_loc, xm[(1 - grp) * 128 + row]) * sl2;
        if (j == 0) {
          m_used = m_blk;
        } else {
          const bool need = m_blk > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            // every MMA that accumulates into O / T for the previous blocks must be done
            ok = wait_acc(gblk - 1u);
            if (!ok) break;
            tc_fence_after_sync();
            const float alpha = need ? fast_exp2(m_used - m_blk) : 1.f;
            if (need) m_used = m_blk;
            l *= alpha;
            mu *= alpha;
            constexpr int kAccCols = kDual ? 2 * DPAD : DPAD;
#pragma unroll 1
            for (int c = grp; c < kAccCols / 16; c += 2) {  // the two groups share the columns
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
        // P = exp2(S * c - m), two elements per fp32 instruction
        const uint64_t sl2_2 = pack_f2(sl2, sl2), neg_m2 = pack_f2(-m_used, -m_used);
        uint64_t la = pack_f2(0.f, 0.f), lb = la;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float x0, x1, x2, x3;
            unpack_f2(fma2(pack_u2(r[c][i], r[c][i + 1]), sl2_2, neg_m2), x0, x1);
            unpack_f2(fma2(pack_u2(r[c][i + 2], r[c][i + 3]), sl2_2, neg_m2), x2, x3);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
            la = add2(la, pack_f2(p0, p1));
            lb = add2(lb, pack_f2(p2, p3));
            r[c][i] = __float_as_uint(p0);
            r[c][i + 1] = __float_as_uint(p1);
            r[c][i + 2] = __float_as_uint(p2);
            r[c][i + 3] = __float_as_uint(p3);
          }
        }
        {
          float s0, s1;
          unpack_f2(add2(la, lb), s0, s1);
          l += s0 + s1;
        }
        uint32_t t_pst = t_sb;  // P over this thread's own S columns ...
        if constexpr (TR::kSepP) {
          // ... or into the P buffer, once the P V products of the previous block have read it
          t_pst = tmem + lane_base + TR::kColP + 32u * static_cast<uint32_t>(grp);
          if (gblk > 0) {
            ok = wait(TR::kBarPEmpty, (gblk - 1u) & 1u);
            if (!ok) break;
            tc_fence_after_sync();
          }
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pk[i] = Pack2<T>::pack(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
          tmem_st_x16(t_pst + c * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(bar(TR::kBarPFull + buf));

        if constexpr (kDual) {
          // ---- part 2: G = P * dS * scale, mu += rowsum(G) ------------------
          ok = wait(TR::kBarDSFull, gblk & 1u);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t scale2 = pack_f2(p.scale, p.scale);
          uint64_t mua = pack_f2(0.f, 0.f), mub = mua;
          uint32_t d[2][32];
          tmem_ld_x32(t_ds, d[0]);
          tmem_ld_x32(t_ds + 32, d[1]);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const uint64_t ga = mul2(pack_u2(r[c][2 * i], r[c][2 * i + 1]),
                                       mul2(pack_u2(d[c][2 * i], d[c][2 * i + 1]), scale2));
              const uint64_t gb = mul2(pack_u2(r[c][2 * i + 2], r[c][2 * i + 3]),
                                       mul2(pack_u2(d[c][2 * i + 2], d[c][2 * i + 3]), scale2));
              mua = add2(mua, ga);
              mub = add2(mub, gb);
              float g0, g1, g2, g3;
              unpack_f2(ga, g0, g1);
              unpack_f2(gb, g2, g3);
              pk[i] = Pack2<T>::pack(g0, g1);
              pk[i + 1] = Pack2<T>::pack(g2, g3);
            }
            tmem_st_x16(t_ds + c * 16, pk);
          }
          {
            float s0, s1;
            unpack_f2(add2(mua, mub), s0, s1);
            mu += s0 + s1;
          }
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarGFull));
        }
      }
      if (!ok) break;
      // ---- epilogue: normalise and write o, to, lse -------------------------
      ok = wait_acc(gblk - 1u);
      if (!ok) break;
      tc_fence_after_sync();
      xsum[grp * 128 + row] = l;
      xsum[256 + grp * 128 + row] = mu;
      // the staging tile of the previous tile must have been read by its store before anybody meets
      if (TR::kStageOut && warp == 2 && lane == 0) tma_store_wait_read();
      ok = exchange();
      if (!ok) break;
      const float l_tot = l + xsum[(1 - grp) * 128 + row];
      const float mu_tot = mu + xsum[256 + (1 - grp) * 128 + row];
      const float inv_l = 1.f / l_tot;
      const float mu_n = mu_tot * inv_l;
      const int vshift = column_shift(p, 1, b, h);  // V columns (hence O / T columns) were loaded 8 early
      const int64_t lq = q0 + row;
      T* o_row = reinterpret_cast<T*>(p.o) + b * p.o_sb + lq * p.o_sl + h * p.o_sh;
      T* to_row = kDual ? reinterpret_cast<T*>(p.to) + b * p.to_sb + lq * p.to_sl + h * p.to_sh : nullptr;
#pragma unroll
      for (int c = 0; c < DPAD / 16; ++c) {
        if ((c & 1) != grp) continue;  // the two groups alternate 16-column chunks
        uint32_t a[16], t[16];
        tmem_ld_x16(t_o + c * 16, a);
        if constexpr (kDual) tmem_ld_x16(t_o + DPAD + c * 16, t);
        tmem_wait_ld();
        uint32_t po[8], pt[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float o0 = __uint_as_float(a[2 * i]) * inv_l;
          const float o1 = __uint_as_float(a[2 * i + 1]) * inv_l;
          po[i] = Pack2<T>::pack(o0, o1);
          if constexpr (kDual) {
            const float t0 = fmaf(__uint_as_float(t[2 * i]), inv_l, -mu_n * o0);
            const float t1 = fmaf(__uint_as_float(t[2 * i + 1]), inv_l, -mu_n * o1);
            pt[i] = Pack2<T>::pack(t0, t1);
          }
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int cc = c * 16 + hh * 8 - vshift;  // accumulator column -> head-dim column
          if (cc >= 0 && cc < p.head_dim) {
            if constexpr (TR::kStageOut) {
              // Staging tile in the layout of a TMA box pair: 64 columns with the 128-byte swizzle, then
              // TAIL columns with the tail's swizzle; 16-byte chunk k of row r sits at chunk k ^ f(r).
              uint32_t off;
              if (cc < 64) {
                off = static_cast<uint32_t>(row * 128 + (((cc >> 3) ^ (row & 7)) << 4));
              } else {
                const int ct = (cc - 64) >> 3;
                const int fx = TAIL == 64 ? (row & 7) : (TAIL == 32 ? ((row >> 1) & 3) : ((row >> 2) & 1));
                off = static_cast<uint32_t>(TR::kMainBytes + row * (2 * TAIL) + ((ct ^ fx) << 4));
              }
              *reinterpret_cast<uint4*>(smem + TR::kRingBytes + off) =
                  make_uint4(po[4 * hh], po[4 * hh + 1], po[4 * hh + 2], po[4 * hh + 3]);
            } else {
              *reinterpret_cast<uint4*>(o_row + cc) = make_uint4(po[4 * hh], po[4 * hh + 1], po[4 * hh + 2], po[4 * hh + 3]);
              if constexpr (kDual)
                *reinterpret_cast<uint4*>(to_row + cc) = make_uint4(pt[4 * hh], pt[4 * hh + 1], pt[4 * hh + 2], pt[4 * hh + 3]);
            }
          }
        }
      }
      if (grp == 0)
        p.lse[(static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q + lq] =
            (m_used + __log2f(l_tot)) * 0.6931471805599453f;
      if constexpr (TR::kStageOut) {
        fence_proxy_async_smem();
        ok = exchange();  // the tile is staged
        if (!ok) break;
        if (warp == 2 && lane == 0) {
          const uint32_t st = s_q + TR::kRingBytes;
          tma_store_4d(&p.o_main, st, 0, q0, h, b);
          if constexpr (TAIL > 0) tma_store_4d(&p.o_tail, st + TR::kMainBytes, 64, q0, h, b);
          tma_store_commit();
        }
      }
      // the accumulator reads above must be complete before the next tile's first MMA overwrites O / T
      tc_fence_before_sync();
    }
    if (TR::kStageOut && warp == 2 && lane == 0) tma_store_wait_all();
    }  // column split
  }

  // ============================== teardown ==================================
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem, TR::kTmemCols);
}

}  // namespace dmf
