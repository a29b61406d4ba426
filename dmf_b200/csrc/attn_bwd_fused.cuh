// Primal backward of attention for sm_100a in ONE pass, for sequences of two 128-row tiles
// (seqlen_q == seqlen_kv == 256, head_dim <= 80): the shape every block of the 256-pixel models trains at.
//
// The two-launch backward (attn_bwd_split.cuh) recomputes the scores in both of its passes (7 matrix
// products) and, with only two key blocks per query tile, never reaches a steady state.  Here a cluster
// of two CTAs owns a whole (batch, head); nothing is recomputed (5 products) and every input tile is
// read from L2 once per CTA:
//
//   CTA r keeps key tile r (K_r, V_r) resident and walks the two query tiles i, the partner's first:
//     S^T  = K_r Q_i^T                      rows = keys, columns = queries (tensor memory)
//     dP^T = V_r dO_i^T
//     P^T  = exp2(S^T c - lse_i log2 e)     P warps, 16-bit, tensor-memory columns of its own
//     dS^T = P^T * (dP^T - delta_i)         D warps, 16-bit, into SHARED memory (row = key, 128 queries)
//     dV_r += P^T dO_i                      A from tensor memory, B = dO_i read MN-major
//     dK_r += dS^T Q_i                      A = the dS^T tile read K-major, B = Q_i read MN-major
//     dQ_i partial = dS K_r                 A = the same dS^T tile read MN-major (i.e. transposed),
//                                           B = K_r read MN-major; rows = queries
//   dQ_i is the sum of the two CTAs' partials.  The partial for the PARTNER's query tile is computed
//   first, staged as fp32 in local shared memory and moved into the partner's shared memory by ONE
//   bulk asynchronous copy (cp.async.bulk shared::cta -> shared::cluster, completion counted on the
//   partner's barrier; thread-issued remote stores of the same 40 KB took 7600 cycles).  It lands in
//   the partner's slot of the step-0 tiles, which are dead by then (both CTAs' step-0 products commit
//   to one barrier of each CTA with a multicast tcgen05.commit, so "the partner's slot is dead" costs
//   no software handshake).  The receiver moves the partial from shared memory into the S columns of
//   its tensor memory, and its own partial, computed second, is ACCUMULATED onto it by the tensor
//   core (partner + own, a fixed order); the owner then scales, rounds and stores dQ_i.  No atomics,
//   no workspace, bit-reproducible.
//
//   -lse_i log2 e is formed by the P warps from the lse row that travels with the tiles; delta_i =
//   rowsum(dO_i * O_i) by the D warps from shared-memory tiles while the P warps turn S into P (the
//   forward output O_i is loaded for that alone).
//
// Both dQ partials use the S columns (free once the second S has been read): the one for the partner is
// drained from there, the partner's is written there, the own one is accumulated there.  Tensor memory:
// S 128 | dP 128 | P 64 | dK DPAD | dV DPAD = 480 columns at head_dim 72.
//
// Warp roles (352 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 P warps (S -> P; the dQ
// partials: exchange, final tile), warps 6-9 D warps (delta; dP, P -> dS; dK / dV tiles), warp 10 issues
// the TMA stores of the three staged output tiles (an issuing thread stalls for a thousand cycles and more
// when the TMA queue is full of the next head's loads; in a warp of its own that stalls nobody else).
#pragma once

#include "attn_bwd.cuh"

namespace dmf {

constexpr int kBwdFusedThreads = 352;  // TMA warp, MMA warp, four P warps, four D warps, store warp
constexpr int kBwdFusedSeqlen = 256;  // the only sequence length this kernel takes (two tiles)

struct BwdFusedParams {
  // load maps, boxes of 128 rows: "main" = columns [0,64), "tail" = [64, 64+TAIL)
  CUtensorMap q_main, q_tail, do_main, do_tail, k_main, k_tail, v_main, v_tail, o_main, o_tail;
  // store maps
  CUtensorMap dq_main, dq_tail, dk_main, dk_tail, dv_main, dv_tail;
  const float* lse;  // (B, H, 256) fp32, 16-byte aligned
  int32_t* status_word;
  int batch, heads, head_dim;
  int num_heads_total;  // batch * heads
  float scale, scale_log2e;
};

template <int TAIL>
struct BwdFusedTraits {
  static_assert(TAIL == 0 || TAIL == 16, "shared memory holds the tiles of a head only up to head_dim 80");
  static constexpr int kDPad = 64 + TAIL;
  static constexpr int kMainBytes = 128 * 128;
  static constexpr int kTailBytes = 128 * TAIL * 2;
  static constexpr int kTileBytes = kMainBytes + kTailBytes;
  static constexpr int kGroupBytes = 2 * kTileBytes;  // (K, V) or (Q_i, dO_i)
  static constexpr int kStages = 2;                   // one per step of a head
  static constexpr int kDsBytes = 128 * 128 * 2;      // dS^T: two atoms of 64 query columns, 128-byte rows
  static constexpr int kXchgBytes = 128 * kDPad * 4;  // an fp32 dQ partial: [column / 4][row][4]
  static constexpr int kVecBytes = 2 * 128 * 4;       // per step: -lse*log2e[128], delta[128]
  static_assert(kTileBytes <= kDsBytes && 2 * kTileBytes <= kXchgBytes, "output staging aliases these buffers");
  static_assert(kXchgBytes <= kGroupBytes, "the partner's partial is received in the slot of the step-0 tiles");
  // offsets from the 1024-byte aligned base
  static constexpr int kOffKV = 0;
  static constexpr int kOffX = kOffKV + kGroupBytes;
  static constexpr int kOffO = kOffX + kStages * kGroupBytes;
  static constexpr int kOffDs = kOffO + kTileBytes;
  static constexpr int kOffXchg = kOffDs + kDsBytes;
  static constexpr int kOffLse = kOffXchg + kXchgBytes;          // raw lse rows as loaded, per stage
  static constexpr int kOffVec = kOffLse + kStages * 512;
  static constexpr int kOffBars = kOffVec + kStages * kVecBytes;
  static constexpr int kBarKFull = 0, kBarXFull = 1 /* +stage */, kBarXEmpty = 3 /* +stage */, kBarOFull = 5,
                       kBarOEmpty = 6, kBarSFull = 7, kBarSEmpty = 8, kBarDFull = 9, kBarPFull = 10, kBarPEmpty = 11,
                       kBarGFull = 12, kBarRecvInTmem = 15, kBarAccEmpty = 16,
                       kBarXchgFull = 17, kBarX0Both = 18, kBarSendDone = 19, kBarX0Free = 20, kBarQStaged = 21,
                       kBarKVStaged = 22, kBarStageFree = 13, kBarVFull = 23, kNumBars = 24;
  static constexpr int kSmemBytes = 1024 + kOffBars + kNumBars * 8 + 16;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  static constexpr uint32_t kColS = 0, kColD = 128, kColP = 256, kColDK = 320, kColDV = 320 + kDPad;
  static_assert(kColDV + kDPad <= 512, "tensor memory");
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTailSwizzle = kSwizzle32;
  static constexpr uint32_t kTailRowBytes = 2 * TAIL;
};

// ---- cluster helpers used only here ----

// Arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once every tcgen05 operation issued
// so far by this thread (a cta_group::1 issuer) has completed.
__device__ __forceinline__ void tc_commit_both(uint32_t bar, bool issue) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      ".reg .b16 m;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "mov.b16 m, 3;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t"
      "}"
      ::"r"(bar), "r"(static_cast<uint32_t>(issue))
      : "memory");
}

// Bulk asynchronous copy of `bytes` (a multiple of 16) from this CTA's shared memory into another CTA's; the
// transaction bytes are counted on a barrier of the destination CTA.  Both destination operands are
// shared::cluster addresses (mapa).  Not a multicast copy, and not a load from global memory.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster, uint32_t src_smem, uint32_t bytes,
                                                 uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(src_smem), "r"(bytes), "r"(bar_cluster)
               : "memory");
}

// acc[128 x (64 + TAIL)] (+)= A[128 x 128] * B[128 x (64 + TAIL)], A 16-bit in SHARED memory as two atoms of
// 64 columns (128-byte rows, 128-byte swizzle, 16 KB apart), B a (row = k index, head-dim contiguous) tile read
// MN-major.  kTransA = false: A rows are the tile's rows (K-major read).  kTransA = true: A is the transpose
// of the stored tile (MN-major read): row m of A is column m of the tile, the k index runs over the tile's rows.
template <int TAIL, typename TR, bool kTransA>
__device__ __forceinline__ void issue_smem_a_pv(bool leader, uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile,
                                                uint32_t idesc_main, uint32_t idesc_tail, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t acc = (accumulate || kk > 0) ? 1u : 0u;
    // K-major: k-step kk = 16 columns = 32 bytes inside atom kk / 4; 8-row groups 1024 bytes apart.
    // MN-major: k-step kk = 16 tile rows = 2048 bytes; the two 64-column atoms (M 0..63, 64..127) 16 KB apart.
    const uint64_t ad = kTransA ? make_smem_desc(a_tile + kk * 2048, 16384, 1024, kSwizzle128)
                                : make_smem_desc(a_tile + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, kSwizzle128);
    const uint64_t bd = make_smem_desc(b_tile + kk * (16 * 128), 8192, 1024, kSwizzle128);
    mma_ss(d_tmem, ad, bd, idesc_main, acc, leader);
    if constexpr (TAIL > 0) {
      const uint64_t bt = make_smem_desc(b_tile + TR::kMainBytes + kk * (16 * TR::kTailRowBytes), TR::kTailBytes,
                                         8 * TR::kTailRowBytes, TR::kTailSwizzle);
      mma_ss(d_tmem + 64, ad, bt, idesc_tail, acc, leader);
    }
  }
}


constexpr int kRoleStore = 500;  // status codes of the store warp's waits (role * 100 + barrier, like the others)

// In-kernel timeline, compiled in only with -DDMF_TRACE (diagnostic builds): the first thread of each role in
// cluster 0 appends (SM cycle counter << 8 | event id) to a per-CTA, per-role list in device memory, which a
// diagnostic export copies out.  Without the define the macro is empty and the kernel carries nothing of this.
#ifdef DMF_TRACE
constexpr int kTraceRoles = 4, kTraceEvents = 512;
__device__ unsigned long long g_bwd_fused_trace[2][kTraceRoles][kTraceEvents];
#define DMF_TRACE_DECL unsigned trace_n = 0;
#define DMF_TRACE_EVENT(role, id)                                                                        \
  do {                                                                                                   \
    if (cluster_id == 0 && lane == 0 && trace_n < kTraceEvents)                                          \
      g_bwd_fused_trace[rank][role][trace_n++] = (static_cast<unsigned long long>(clock64()) << 8) | (id); \
  } while (0)
#else
#define DMF_TRACE_DECL
#define DMF_TRACE_EVENT(role, id) do { } while (0)
#endif

template <typename T, int TAIL>
__global__ void __launch_bounds__(kBwdFusedThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ BwdFusedParams p) {
  using TR = BwdFusedTraits<TAIL>;
  constexpr int DPAD = TR::kDPad;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_kv = s_base + TR::kOffKV, s_x = s_base + TR::kOffX, s_o = s_base + TR::kOffO;
  const uint32_t s_ds = s_base + TR::kOffDs, s_xchg = s_base + TR::kOffXchg, s_lse = s_base + TR::kOffLse;
  uint8_t* ds_tile = smem + TR::kOffDs;      // dS^T of the current step; between heads: staging of dK, dV
  uint8_t* send = smem + TR::kOffXchg;       // this CTA's dQ partial for the partner; at the end of a head: staging of dQ, dV
  const uint8_t* recv = smem + TR::kOffX;    // the partner's dQ partial for this CTA, in the slot of the step-0 tiles
  const float* lse_raw = reinterpret_cast<const float*>(smem + TR::kOffLse);   // [stage][128]
  float* vec = reinterpret_cast<float*>(smem + TR::kOffVec);                   // [stage][2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::kOffBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + TR::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) -> uint32_t { return bar0 + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t peer = rank ^ 1u;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  // step 0 works on the partner's query tile, step 1 on this CTA's own
  auto q_tile_of = [&](int step) -> int { return step == 0 ? static_cast<int>(peer) : static_cast<int>(rank); };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < TR::kNumBars; ++i) {
      uint32_t count = 1;  // TMA transaction or tcgen05.commit
      if (i == TR::kBarOEmpty || i == TR::kBarSEmpty || i == TR::kBarPFull || i == TR::kBarGFull ||
          i == TR::kBarRecvInTmem || i == TR::kBarAccEmpty || i == TR::kBarX0Free || i == TR::kBarQStaged ||
          i == TR::kBarKVStaged)
        count = 4;                                  // one arrival per warp of a group
      if (i == TR::kBarPEmpty) count = 5;           // the commit behind dV += P^T dO, and the four D warps
      if (i == TR::kBarX0Both) count = 2;           // the step-0 commits of both CTAs (multicast)
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
  cluster_sync_all();  // both CTAs' barriers exist before anybody arrives remotely
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // =========================== TMA producer ===============================
    if (lane == 0) {
      prefetch_tensor_map(&p.q_main);
      prefetch_tensor_map(&p.do_main);
      prefetch_tensor_map(&p.k_main);
      prefetch_tensor_map(&p.v_main);
      prefetch_tensor_map(&p.o_main);
      uint32_t hcnt = 0;
      bool ok = true;
      DMF_TRACE_DECL
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleProducer + b_);
      };
      for (int bh = cluster_id; ok && bh < p.num_heads_total; bh += num_clusters, ++hcnt) {
        const int b = bh / p.heads, h = bh % p.heads;
        const uint32_t ph = hcnt & 1u;   // every barrier below completes once per head (O: once per step)
#pragma unroll 1
        for (int step = 0; ok && step < 2; ++step) {
          const int q0 = q_tile_of(step) * 128;
          // (Q_i, dO_i) and the lse row of the tile.  Slot 1 is freed by the last product of the previous head;
          // slot 0 receives the partner's dQ partial in the second half of a head and is free once the P warps
          // have read that
          ok = wait(step == 0 ? TR::kBarX0Free : TR::kBarXEmpty + 1, ph ^ 1u);
          if (!ok) break;
          {
            const uint32_t dst = s_x + step * TR::kGroupBytes, fb = bar(TR::kBarXFull + step);
            mbar_arrive_expect_tx(fb, TR::kGroupBytes + 512);
            tma_load_4d(dst, &p.q_main, fb, 0, q0, h, b);
            tma_load_4d(dst + TR::kTileBytes, &p.do_main, fb, 0, q0, h, b);
            if constexpr (TAIL > 0) {
              tma_load_4d(dst + TR::kMainBytes, &p.q_tail, fb, 64, q0, h, b);
              tma_load_4d(dst + TR::kTileBytes + TR::kMainBytes, &p.do_tail, fb, 64, q0, h, b);
            }
            const int64_t off = (static_cast<int64_t>(b) * p.heads + h) * kBwdFusedSeqlen + q0;
            bulk_load_1d(s_lse + step * 512, p.lse + off, 512, fb);
            DMF_TRACE_EVENT(0, 1 + 3 * step);
          }
          if (step == 0) {
            // K_r, V_r next (the first product of the head needs K and the step-0 query tile; the forward output, for
            // delta, is needed two thousand cycles later): free when the last products of the previous head are complete
            ok = wait(TR::kBarXEmpty + 1, ph ^ 1u);
            if (!ok) break;
            // K on a barrier of its own, ahead of V: the head's first product needs only K
            const uint32_t fk = bar(TR::kBarKFull), fv = bar(TR::kBarVFull);
            const int k0 = static_cast<int>(rank) * 128;
            mbar_arrive_expect_tx(fk, TR::kTileBytes);
            tma_load_4d(s_kv, &p.k_main, fk, 0, k0, h, b);
            if constexpr (TAIL > 0) tma_load_4d(s_kv + TR::kMainBytes, &p.k_tail, fk, 64, k0, h, b);
            mbar_arrive_expect_tx(fv, TR::kTileBytes);
            tma_load_4d(s_kv + TR::kTileBytes, &p.v_main, fv, 0, k0, h, b);
            if constexpr (TAIL > 0) tma_load_4d(s_kv + TR::kTileBytes + TR::kMainBytes, &p.v_tail, fv, 64, k0, h, b);
            DMF_TRACE_EVENT(0, 3);
          }
          // the forward output of the tile, for delta (one buffer: freed when the P warps have read it)
          ok = wait(TR::kBarOEmpty, ((2u * hcnt + static_cast<uint32_t>(step)) & 1u) ^ 1u);
          if (!ok) break;
          {
            const uint32_t of = bar(TR::kBarOFull);
            mbar_arrive_expect_tx(of, TR::kTileBytes);
            tma_load_4d(s_o, &p.o_main, of, 0, q0, h, b);
            if constexpr (TAIL > 0) tma_load_4d(s_o + TR::kMainBytes, &p.o_tail, of, 64, q0, h, b);
            DMF_TRACE_EVENT(0, 2 + 3 * step);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ================================
    const bool leader = elect_one();
    auto commit = [&](int b_) { tc_commit(bar(b_), leader); };
    constexpr uint32_t idesc_qk = make_idesc(kBf16, false, false, 128, 128);
    constexpr uint32_t idesc_pv_main = make_idesc(kBf16, false, true, 128, 64);
    constexpr uint32_t idesc_pv_tail = make_idesc(kBf16, false, true, 128, TAIL > 0 ? TAIL : 16);
    constexpr uint32_t idesc_tr_main = make_idesc(kBf16, true, true, 128, 64);   // A read transposed
    constexpr uint32_t idesc_tr_tail = make_idesc(kBf16, true, true, 128, TAIL > 0 ? TAIL : 16);
    const uint32_t t_s = tmem + TR::kColS, t_d = tmem + TR::kColD, t_p = tmem + TR::kColP;
    const uint32_t t_dk = tmem + TR::kColDK, t_dv = tmem + TR::kColDV;
    const uint32_t k_tile = s_kv, v_tile = s_kv + TR::kTileBytes;
    uint32_t hcnt = 0;
    bool ok = true;
    DMF_TRACE_DECL
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleMma + b_);
    };
    // The S columns are handed back by the P warps three times per head: S_0 read, S_1 read, the first dQ
    // partial read.  n counts those hand-backs from the start of the kernel.
    auto wait_s_empty = [&](uint32_t n) -> bool { return wait(TR::kBarSEmpty, n & 1u); };
    for (int bh = cluster_id; ok && bh < p.num_heads_total; bh += num_clusters, ++hcnt) {
      const uint32_t ph = hcnt & 1u;
      const uint32_t g0 = 2u * hcnt;  // number of the head's first step
      const uint32_t q0_tile = s_x, do0_tile = s_x + TR::kTileBytes;
      const uint32_t q1_tile = s_x + TR::kGroupBytes, do1_tile = q1_tile + TR::kTileBytes;
      // ---- S_0, dP_0, S_1 ----
      ok = wait(TR::kBarKFull, ph) && wait(TR::kBarXFull + 0, ph);
      if (ok && hcnt > 0) ok = wait_s_empty(3u * hcnt - 1u);   // the previous head's first dQ partial has been read
      if (!ok) break;
      tc_fence_after_sync();
      DMF_TRACE_EVENT(1, 10);
      issue_qk<TAIL, TR>(leader, t_s, k_tile, q0_tile, idesc_qk, false);     // S_0^T = K Q_0^T
      commit(TR::kBarSFull);
      DMF_TRACE_EVENT(1, 11);
      // (the dP columns are free: the D warps had read dP_1 of the previous head before its last products were issued)
      ok = wait(TR::kBarVFull, ph);
      if (!ok) break;
      tc_fence_after_sync();
      issue_qk<TAIL, TR>(leader, t_d, v_tile, do0_tile, idesc_qk, false);    // dP_0^T = V dO_0^T
      commit(TR::kBarDFull);
      DMF_TRACE_EVENT(1, 12);
      ok = wait(TR::kBarXFull + 1, ph) && wait_s_empty(3u * hcnt);           // S_0 is in the P warps' registers
      if (!ok) break;
      tc_fence_after_sync();
      issue_qk<TAIL, TR>(leader, t_s, k_tile, q1_tile, idesc_qk, false);     // S_1^T
      commit(TR::kBarSFull);
      DMF_TRACE_EVENT(1, 13);
      // ---- step 0: dV = P_0^T dO_0, dK = dS_0^T Q_0, dQ partial of the partner's tile ----
      ok = wait(TR::kBarPFull, g0 & 1u);
      if (ok && hcnt > 0) ok = wait(TR::kBarAccEmpty, (hcnt - 1u) & 1u);     // the previous head's dK, dV have been read
      if (!ok) break;
      tc_fence_after_sync();
      DMF_TRACE_EVENT(1, 14);
      issue_pv<TAIL, TR>(leader, t_dv, t_p, do0_tile, idesc_pv_main, idesc_pv_tail, false);
      commit(TR::kBarPEmpty);
      DMF_TRACE_EVENT(1, 15);
      ok = wait(TR::kBarGFull, g0 & 1u) && wait_s_empty(3u * hcnt + 1u);     // dS_0 in shared memory; S_1 read
      if (!ok) break;
      tc_fence_after_sync();
      DMF_TRACE_EVENT(1, 16);
      issue_smem_a_pv<TAIL, TR, false>(leader, t_dk, s_ds, q0_tile, idesc_pv_main, idesc_pv_tail, false);
      issue_smem_a_pv<TAIL, TR, true>(leader, t_s, s_ds, k_tile, idesc_tr_main, idesc_tr_tail, false);
      commit(TR::kBarXEmpty + 0);  // dS buffer free; the first dQ partial is complete
      tc_commit_both(bar(TR::kBarX0Both), leader);  // ... in both CTAs: each CTA's slot 0 can receive the other's partial
      // ---- step 1 ----
      issue_qk<TAIL, TR>(leader, t_d, v_tile, do1_tile, idesc_qk, false);    // dP_1^T (dP_0 was read before dS_0 was signalled)
      commit(TR::kBarDFull);
      DMF_TRACE_EVENT(1, 17);
      ok = wait(TR::kBarPFull, (g0 + 1u) & 1u);
      if (!ok) break;
      tc_fence_after_sync();
      DMF_TRACE_EVENT(1, 18);
      issue_pv<TAIL, TR>(leader, t_dv, t_p, do1_tile, idesc_pv_main, idesc_pv_tail, true);
      commit(TR::kBarPEmpty);
      ok = wait(TR::kBarGFull, (g0 + 1u) & 1u);
      if (!ok) break;
      tc_fence_after_sync();
      DMF_TRACE_EVENT(1, 19);
      issue_smem_a_pv<TAIL, TR, false>(leader, t_dk, s_ds, q1_tile, idesc_pv_main, idesc_pv_tail, true);
      ok = wait(TR::kBarRecvInTmem, ph);            // the partner's partial of this CTA's dQ tile sits in the S columns
      if (!ok) break;
      tc_fence_after_sync();
      issue_smem_a_pv<TAIL, TR, true>(leader, t_s, s_ds, k_tile, idesc_tr_main, idesc_tr_tail, true);  // += dS_1 K
      commit(TR::kBarXEmpty + 1);  // slot 1, K/V and the dS buffer free; dK, dV and the second dQ partial complete
      DMF_TRACE_EVENT(1, 20);
    }
  } else if (warp == 10) {
    // ============================== store warp ==============================
    if (lane == 0) {
      uint32_t hcnt = 0;
      bool ok = true;
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleStore + b_);
      };
      for (int bh = cluster_id; ok && bh < p.num_heads_total; bh += num_clusters, ++hcnt) {
        const int b = bh / p.heads, h = bh % p.heads;
        const uint32_t ph = hcnt & 1u;
        const int r0 = static_cast<int>(rank) * 128;   // this CTA's query tile and key tile
        ok = wait(TR::kBarQStaged, ph);
        if (!ok) break;
        tma_store_4d(&p.dq_main, s_xchg, 0, r0, h, b);
        if constexpr (TAIL > 0) tma_store_4d(&p.dq_tail, s_xchg + TR::kMainBytes, 64, r0, h, b);
        tma_store_commit();
        ok = wait(TR::kBarKVStaged, ph);
        if (!ok) break;
        tma_store_4d(&p.dk_main, s_ds, 0, r0, h, b);
        if constexpr (TAIL > 0) tma_store_4d(&p.dk_tail, s_ds + TR::kMainBytes, 64, r0, h, b);
        tma_store_4d(&p.dv_main, s_xchg + TR::kTileBytes, 0, r0, h, b);
        if constexpr (TAIL > 0) tma_store_4d(&p.dv_tail, s_xchg + TR::kTileBytes + TR::kMainBytes, 64, r0, h, b);
        tma_store_commit();
        tma_store_wait_read();                 // all three staging tiles have been read
        mbar_arrive(bar(TR::kBarStageFree));
      }
      tma_store_wait_all();
    }
  } else {
    // ====================== P warps and D warps =============================
    const bool p_role = warp < 6;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem + lane_base + TR::kColS, t_d = tmem + lane_base + TR::kColD;
    const uint32_t t_p = tmem + lane_base + TR::kColP, t_dk = tmem + lane_base + TR::kColDK;
    const float sl2 = p.scale_log2e;
    uint32_t hcnt = 0;
    bool ok = true;
    DMF_TRACE_DECL
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
    };
    // 16-byte chunk of head-dim column cc (a multiple of 8) of this thread's row in a tile-shaped buffer
    auto chunk_off = [&](int cc) -> uint32_t {
      if (cc < 64) return static_cast<uint32_t>(row * 128 + (((cc >> 3) ^ (row & 7)) << 4));
      const int ct = (cc - 64) >> 3;
      return static_cast<uint32_t>(TR::kMainBytes + row * 32 + ((ct ^ ((row >> 2) & 1)) << 4));
    };
    const int bar_id = p_role ? 2 : 1;  // hardware barrier of the role's 128 threads
    const bool mover = (lane == 0) && (warp == 2);  // the P warps' thread for one-per-CTA actions

    // Failure handling: a wait that gives up makes `ok` false.  From then on a warp skips all work but still walks
    // through every hardware-barrier meeting of the head (they AND everybody's `ok`, so the whole role agrees),
    // and leaves the head loop only at its end: no warp is ever left alone at a meeting.
    for (int bh = cluster_id; ok && bh < p.num_heads_total; bh += num_clusters, ++hcnt) {
      const int b = bh / p.heads, h = bh % p.heads;
      const uint32_t ph = hcnt & 1u;
      if (p_role) {
        // ================================ P warps ================================
#pragma unroll 1
        for (int step = 0; step < 2; ++step) {
          const uint32_t g = 2u * hcnt + static_cast<uint32_t>(step);
          float* vstage = vec + step * 256;
          // ---- -lse * log2e of the step's 128 queries (the lse row arrives with the step's tiles) ----
          if (ok) ok = wait(TR::kBarXFull + step, ph);
          if (warp == 2) DMF_TRACE_EVENT(2, 30);
          if (ok) vstage[row] = -lse_raw[step * 128 + row] * 1.4426950408889634f;
          ok = named_bar_and(bar_id, 128, ok);  // all 128 values are visible to the P warps
          if (warp == 2) DMF_TRACE_EVENT(2, 31);
          // ---- P^T = exp2(S^T * c - lse2), 16-bit, into the P columns ----
          if (ok) ok = wait(TR::kBarSFull, g & 1u);
          if (ok) {
            tc_fence_after_sync();
            if (warp == 2) DMF_TRACE_EVENT(2, 32);
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
                const float4 nv = *reinterpret_cast<const float4*>(vstage + c * 32 + i);
                float x0, x1, x2, x3;
                unpack_f2(fma2(pack_u2(r[c][i], r[c][i + 1]), sl2_2, pack_f2(nv.x, nv.y)), x0, x1);
                unpack_f2(fma2(pack_u2(r[c][i + 2], r[c][i + 3]), sl2_2, pack_f2(nv.z, nv.w)), x2, x3);
                r[c][i / 2] = Pack2<T>::pack(fast_exp2(x0), fast_exp2(x1));
                r[c][i / 2 + 1] = Pack2<T>::pack(fast_exp2(x2), fast_exp2(x3));
              }
            }
            if (warp == 2) DMF_TRACE_EVENT(2, 33);
            // the readers of the previous P (the dV product and the D warps) are done with it
            if (g > 0) ok = wait(TR::kBarPEmpty, (g - 1u) & 1u);
            if (ok) {
              tc_fence_after_sync();
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
              if (warp == 2) DMF_TRACE_EVENT(2, 34);
            }
          }
        }
        // ---- the partner's dQ partial (step 0, in the S columns): staged as fp32, one bulk copy to the partner ----
        // both CTAs' step-0 products are complete: the partial is there, and the step-0 tiles of BOTH CTAs are dead
        if (ok) ok = wait(TR::kBarX0Both, ph);
        // the completion of the partner's copy into this CTA's slot 0 is counted here
        if (ok && mover) mbar_arrive_expect_tx(bar(TR::kBarXchgFull), TR::kXchgBytes);
        // the stores of the previous head's dQ and dV tiles have read the region the partial is staged in
        if (ok && hcnt > 0) ok = wait(TR::kBarStageFree, (hcnt - 1u) & 1u);
        if (ok) {
          tc_fence_after_sync();
          if (warp == 2) DMF_TRACE_EVENT(2, 35);
#pragma unroll
          for (int c = 0; c < DPAD / 16; ++c) {
            uint32_t a[16];
            tmem_ld_x16(t_s + c * 16, a);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(send + ((c * 4 + i) * 128 + row) * 16) = make_uint4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
          }
          fence_proxy_async_smem();
        }
        ok = named_bar_and(bar_id, 128, ok);         // all 128 rows are staged
        if (ok && mover) {
          bulk_copy_to_cta(map_to_cta(s_x, peer), s_xchg, TR::kXchgBytes, map_to_cta(bar(TR::kBarXchgFull), peer));
          DMF_TRACE_EVENT(2, 36);
        }
        // ---- the partner's partial of this CTA's own dQ tile: shared memory -> the S columns ----
        if (ok)
          ok = wait(TR::kBarXchgFull, ph);             // (transaction bytes of an asynchronous copy, like a TMA load)
        if (ok) {
          if (warp == 2) DMF_TRACE_EVENT(2, 37);
#pragma unroll
          for (int c = 0; c < DPAD / 16; ++c) {
            uint32_t a[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 o4 = *reinterpret_cast<const uint4*>(recv + ((c * 4 + i) * 128 + row) * 16);
              a[4 * i] = o4.x; a[4 * i + 1] = o4.y; a[4 * i + 2] = o4.z; a[4 * i + 3] = o4.w;
            }
            tmem_st_x16(t_s + c * 16, a);
          }
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarRecvInTmem)); // the own partial can be accumulated onto it
          mbar_arrive_warp(bar(TR::kBarX0Free));     // slot 0 is free for the next head's step-0 tiles
          // tell the partner that its copy has arrived (its staging region is free again).  Nothing this thread
          // wrote is read by the partner on the strength of this arrival, so it carries no cluster-scope release
          // (such a release costs thousands of cycles here)
          if (warp == 5 && lane == 0) mbar_arrive_cluster(map_to_cta(bar(TR::kBarSendDone), peer));
          if (warp == 2) DMF_TRACE_EVENT(2, 40);
        }
        // ---- this CTA's own dQ tile: partner's partial + own (accumulated by the tensor core), scaled, stored ----
        if (ok) ok = wait(TR::kBarXEmpty + 1, ph);
        uint32_t packed[DPAD / 2];
        if (ok) {
          tc_fence_after_sync();
          if (warp == 2) DMF_TRACE_EVENT(2, 41);
          const uint64_t scale2 = pack_f2(p.scale, p.scale);
#pragma unroll
          for (int c = 0; c < DPAD / 16; ++c) {
            uint32_t a[16];
            tmem_ld_x16(t_s + c * 16, a);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float x0, x1;
              unpack_f2(mul2(pack_u2(a[2 * i], a[2 * i + 1]), scale2), x0, x1);
              packed[c * 8 + i] = Pack2<T>::pack(x0, x1);
            }
          }
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarSEmpty));     // the S columns are free for the next head
          // this CTA's own copy has arrived at the partner (signalled long ago): the staging region can take the dQ tile
          ok = wait(TR::kBarSendDone, ph);
        }
        if (ok) {
#pragma unroll
          for (int c = 0; c < DPAD / 8; ++c)
            *reinterpret_cast<uint4*>(send + chunk_off(c * 8)) =
                make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
          fence_proxy_async_smem();
          mbar_arrive_warp(bar(TR::kBarQStaged));    // for the store warp
        }
        if (warp == 2) DMF_TRACE_EVENT(2, 38);
      } else {
        // ================================ D warps ================================
#pragma unroll 1
        for (int step = 0; step < 2; ++step) {
          const uint32_t g = 2u * hcnt + static_cast<uint32_t>(step);
          float* vstage = vec + step * 256;
          // ---- delta = rowsum(dO * O) of the step's 128 queries, one query row per thread, from the shared-memory
          // tiles (this role would otherwise sit idle until the first P of the step exists) ----
          if (ok) ok = wait(TR::kBarXFull + step, ph);
          if (ok) ok = wait(TR::kBarOFull, g & 1u);
          if (ok) {
            const uint8_t* do_tile = smem + TR::kOffX + step * TR::kGroupBytes + TR::kTileBytes;
            const uint8_t* o_tile = smem + TR::kOffO;
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < DPAD / 8; ++c) {
              const uint32_t off = chunk_off(c * 8);
              const uint4 ov = *reinterpret_cast<const uint4*>(o_tile + off);
              const uint4 dv = *reinterpret_cast<const uint4*>(do_tile + off);
              const uint32_t ou[4] = {ov.x, ov.y, ov.z, ov.w}, du[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 a = unpack2<T>(ou[i]), g2 = unpack2<T>(du[i]);
                acc = fmaf(a.x, g2.x, acc);
                acc = fmaf(a.y, g2.y, acc);
              }
            }
            vstage[128 + row] = acc;
            mbar_arrive_warp(bar(TR::kBarOEmpty));  // o has been read
          }
          if (warp == 6) DMF_TRACE_EVENT(3, 56);
          if (ok) ok = wait(TR::kBarPFull, g & 1u);
          if (ok) ok = wait(TR::kBarDFull, g & 1u);
          // the dS buffer: free when the products of the step before (this head's step 0) are done with it, or the
          // store of the previous head's dK tile, which was staged there
          if (ok && step == 1) ok = wait(TR::kBarXEmpty + 0, ph);
          if (ok && step == 0 && hcnt > 0) ok = wait(TR::kBarStageFree, (hcnt - 1u) & 1u);
          ok = named_bar_and(bar_id, 128, ok);       // (delta of all 128 queries is visible to the D warps)
          if (warp == 6) DMF_TRACE_EVENT(3, 50);
          if (ok) {
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t d[32], pc[16];
              tmem_ld_x32(t_d + c * 32, d);
              tmem_ld_x16(t_p + c * 16, pc);
              tmem_wait_ld();
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; i += 2) {
                const float4 dv = *reinterpret_cast<const float4*>(vstage + 128 + c * 32 + 2 * i);
                const float2 pa = unpack2<T>(pc[i]), pb = unpack2<T>(pc[i + 1]);
                const float g0 = pa.x * (__uint_as_float(d[2 * i]) - dv.x);
                const float g1 = pa.y * (__uint_as_float(d[2 * i + 1]) - dv.y);
                const float g2 = pb.x * (__uint_as_float(d[2 * i + 2]) - dv.z);
                const float g3 = pb.y * (__uint_as_float(d[2 * i + 3]) - dv.w);
                pk[i] = Pack2<T>::pack(g0, g1);
                pk[i + 1] = Pack2<T>::pack(g2, g3);
              }
              // query columns 32c .. 32c+31 of this key row: atom c / 2, 16-byte chunks 4 (c % 2) .. + 3
              uint8_t* dst = ds_tile + (c >> 1) * 16384 + row * 128;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                *reinterpret_cast<uint4*>(dst + ((((c & 1) * 4 + k) ^ (row & 7)) << 4)) =
                    make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
            }
            tc_fence_before_sync();
            mbar_arrive_warp(bar(TR::kBarPEmpty));  // P has been read (dP too: its columns may take a dQ partial)
            fence_proxy_async_smem();
            mbar_arrive_warp(bar(TR::kBarGFull));   // dS^T is in shared memory
            if (warp == 6) DMF_TRACE_EVENT(3, 51);
          }
        }
        // ---- epilogue: dK (scaled) staged in the dS buffer, dV in the second half of the send region ----
        if (ok) ok = wait(TR::kBarXEmpty + 1, ph);  // every product of the head is complete
        // the send region: this CTA's copy to the partner has arrived there
        if (ok)
          ok = wait(TR::kBarSendDone, ph);
        ok = named_bar_and(bar_id, 128, ok);
        if (warp == 6) DMF_TRACE_EVENT(3, 52);
        if (ok) {
          tc_fence_after_sync();
          uint8_t* dv_stage = send + TR::kTileBytes;
          const uint64_t scale2 = pack_f2(p.scale, p.scale);
#pragma unroll
          for (int c = 0; c < DPAD / 16; ++c) {
            uint32_t a[16], v[16];
            tmem_ld_x16(t_dk + c * 16, a);
            tmem_ld_x16(t_dk + DPAD + c * 16, v);
            tmem_wait_ld();
            uint32_t p0[8], p1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float x0, x1;
              unpack_f2(mul2(pack_u2(a[2 * i], a[2 * i + 1]), scale2), x0, x1);
              p0[i] = Pack2<T>::pack(x0, x1);
              p1[i] = Pack2<T>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const uint32_t off = chunk_off(c * 16 + hh * 8);
              *reinterpret_cast<uint4*>(ds_tile + off) = make_uint4(p0[4 * hh], p0[4 * hh + 1], p0[4 * hh + 2], p0[4 * hh + 3]);
              *reinterpret_cast<uint4*>(dv_stage + off) = make_uint4(p1[4 * hh], p1[4 * hh + 1], p1[4 * hh + 2], p1[4 * hh + 3]);
            }
          }
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarAccEmpty));  // the next head may overwrite dK, dV
          fence_proxy_async_smem();
          mbar_arrive_warp(bar(TR::kBarKVStaged));  // for the store warp
        }
        if (warp == 6) DMF_TRACE_EVENT(3, 53);
      }
    }
  }

  // ============================== teardown ==================================
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the partner may still write this CTA's shared memory or barriers
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem, TR::kTmemCols);
}

}  // namespace dmf
