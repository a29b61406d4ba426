// Primal backward of attention for sm_100a in one pass over the scores, for LONG sequences (any multiple of 128
// in both lengths; head_dim <= 80): a key tile stays resident, the query tiles stream past it, and dQ is summed in
// an fp32 buffer of the caller's workspace with vector atomics.
//
// The two-launch backward (attn_bwd_split.cuh) recomputes S and dP in both of its passes (7 matrix products per
// 128 x 128 block).  Here every block is visited once (5 products):
//
//   CTA owns key tile j of one (batch, head): K_j, V_j resident; for each query tile i (a "step"):
//     S^T  = K_j Q_i^T,  dP^T = V_j dO_i^T        rows = keys, columns = queries (tensor memory)
//     P^T  = exp2(S^T c - lse_i log2 e)           16-bit, tensor-memory columns of its own
//     dS^T = P^T * (dP^T - delta_i)               16-bit, into shared memory (two buffers)
//     dV_j += P^T dO_i,   dK_j += dS^T Q_i        accumulated in tensor memory over the steps
//     dQ_i partial = dS K_j                        into the dP columns (dP has been read by then) -> registers ->
//                                                  red.global.add.v4.f32 into the fp32 accumulator tile of
//                                                  (batch, head, i)
//   delta = rowsum(dO * O) and -lse log2 e come from a small kernel that runs first (two rows of 512 bytes per
//   step here instead of a 20 KB tile of O), the conversion of the accumulator to the 16-bit dQ from one that runs
//   last.
//
// The sum over the key tiles of a query tile is taken in whatever order the CTAs get there: like the
// FlashAttention backward the reference calls (deterministic=False), and unlike the other backward kernels of
// this library, the last bits of dQ can differ from run to run.  dK and dV are reproducible.
//
// Rings: Q_i (+ its two rows) three slots, dO_i two slots, dS^T two buffers; shared memory at head_dim 72: K,V
// 40 KB + Q 60 KB + dO 40 KB + dS^T 64 KB = 204 KB.  What bounds a step is the traffic between the SMs and L2:
// every 128 x 128 block brings a Q and a dO tile in (40 KB) and sends a dQ partial out (36 KB of atomics); the
// five products of a block take about half of a step's time when timed alone.  The dQ partial goes to global
// memory from registers: staging it in shared memory for a bulk reduction (cp.reduce.async.bulk) was no faster
// and cost 16 KB of shared memory.
// Tensor memory: S 128 | P 64 | dP, then the dQ partial 128 | dK | dV.
//
// Warp roles (448 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 the elementwise warps (two per
// lane quarter, 64 query columns each: S -> P, then dP, P -> dS), warps 10-13 the drain warps (dQ partial ->
// atomics each step; dK / dV tiles -> shared memory -> TMA stores at the end of a key tile).
#pragma once

#include "attn_bwd_fused.cuh"

namespace dmf {

constexpr int kBwdStreamThreads = 448;

struct BwdStreamParams {
  CUtensorMap q, dout, k, v;   // loads: boxes of 16 head-dim columns x 128 rows, 32-byte swizzle
  CUtensorMap dk, dv;          // stores, same boxes
  const float* nlse2;   // (B, H, Lq) fp32: -lse * log2(e), in the workspace, written by bwd_delta_kernel
  const float* ndelta;  // (B, H, Lq) fp32: -rowsum(dO * O), in the workspace, written by bwd_delta_kernel
  float* dq_acc;        // workspace: per (b, h, query tile) 128 x head_dim floats as [column / 4][row][4]
  int32_t* status_word;
  int batch, heads, head_dim, seqlen_q, seqlen_kv;
  // Heads whose rows start in the middle of a 32-byte sector (head_dim 72: rows of 144 bytes, every other head)
  // are loaded 8 columns early, so that every 32-byte box is one sector instead of two halves: group 0 = q and k,
  // group 1 = v and dout; (align0 + b * align_b + h * align_h) % 32 is the byte offset of the head's rows.
  int align_enable[2], align0[2], align_b[2], align_h[2];
  int tiles_per_bh;     // key tiles per (b, h)
  int num_tiles;        // batch * heads * tiles_per_bh
  int steps;            // query tiles per (b, h)
  float scale, scale_log2e;
};

template <int TAIL>
struct BwdStreamTraits {
  static_assert(TAIL == 0 || TAIL == 16, "shared memory holds the rings only up to head_dim 80");
  static constexpr int kDPad = 64 + TAIL;
  // A tile of 128 rows x kDPad head-dim columns lies in shared memory as kAtoms blocks of 16 columns (32-byte
  // rows, 32-byte swizzle): one block is one k-step of a product over the head dim, and the blocks side by side
  // are ONE operand of kDPad columns for a product over the rows (a single instruction per k-step; with the head
  // dim split 64 + 16 every k-step took two, and each re-read the 4 KB A operand from shared memory).
  static constexpr int kAtoms = kDPad / 16;
  static constexpr int kAtomBytes = 128 * 32;
  static constexpr int kTileBytes = kAtoms * kAtomBytes;
  static constexpr int kQStages = 3, kDoStages = 2, kDsBufs = 2;
  static constexpr int kDsBytes = 128 * 128 * 2;   // dS^T: two atoms of 64 query columns, 128-byte rows
  static constexpr int kRowBytes = 2 * 512;        // per Q slot: -lse log2 e [128], -delta[128]
  static_assert(kTileBytes <= kDsBytes, "the dK / dV staging tiles alias the dS buffers");
  static constexpr int kOffKV = 0;
  static constexpr int kOffQ = kOffKV + 2 * kTileBytes;
  static constexpr int kOffDo = kOffQ + kQStages * kTileBytes;
  static constexpr int kOffDs = kOffDo + kDoStages * kTileBytes;
  static constexpr int kOffRows = kOffDs + kDsBufs * kDsBytes;
  static constexpr int kOffBars = kOffRows + kQStages * kRowBytes;
  static constexpr int kBarKFull = 0, kBarVFull = 1, kBarQFull = 2 /* +slot */, kBarStepDone = 5 /* +slot */,
                       kBarDoFull = 8 /* +slot */, kBarPvDone = 10 /* +slot */, kBarSFull = 12, kBarPFull = 13,
                       kBarDFull = 14, kBarGFull = 15, kBarQpEmpty = 16, kBarQpFull = 17, kBarSEmpty = 18,
                       kBarTileDone = 19, kBarAccEmpty = 20, kBarKVStaged = 21, kBarStageFree = 22, kNumBars = 23;
  static constexpr int kSmemBytes = 1024 + kOffBars + kNumBars * 8 + 16;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  static_assert(kOffDs % 1024 == 0 && kOffQ % 1024 == 0 && kOffDo % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  // the dQ partial of a step is written over the dP columns of the same step (dP is in registers by then)
  static constexpr uint32_t kColS = 0, kColP = 128, kColD = 192, kColQp = kColD, kColDK = 320, kColDV = 320 + kDPad;
  static_assert(kColDV + kDPad <= 512, "tensor memory");
  static constexpr uint32_t kTmemCols = 512;
};

// four fp32 atomic adds with one instruction (16-byte aligned address), no return value
__device__ __forceinline__ void red_add_v4(float* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(addr), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)),
                 "f"(__uint_as_float(d))
               : "memory");
}

// ---- MMA issue helpers for tiles of 16-column blocks (executed by the MMA warp, the instruction by its leader) ----

// acc[128 x 128] (+)= A[128 x DPAD] * B[128 x DPAD]^T: both operands K-major, one block per k-step.
template <typename TR>
__device__ __forceinline__ void issue_qk_blocks(bool leader, uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile,
                                                uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < TR::kAtoms; ++kk) {
    const uint64_t ad = make_smem_desc(a_tile + kk * TR::kAtomBytes, 16, 256, kSwizzle32);
    const uint64_t bd = make_smem_desc(b_tile + kk * TR::kAtomBytes, 16, 256, kSwizzle32);
    mma_ss(d_tmem, ad, bd, idesc, kk > 0 ? 1u : 0u, leader);
  }
}

// B operand of a product over a tile's rows: k-step kk = rows 16 kk .. + 15 (512 bytes), the blocks (16 columns of
// N each) 4 KB apart, groups of 8 rows 256 bytes apart.
template <typename TR>
__device__ __forceinline__ uint64_t rows_b_desc(uint32_t tile, int kk) {
  return make_smem_desc(tile + kk * 512, TR::kAtomBytes, 256, kSwizzle32);
}

// acc[128 x DPAD] (+)= A[128 x 128] * B[128 x DPAD]: the 16-bit A operand in 64 columns of tensor memory.
template <typename TR>
__device__ __forceinline__ void issue_pv_blocks(bool leader, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_tile,
                                                uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    mma_ts(d_tmem, a_tmem + kk * 8, rows_b_desc<TR>(b_tile, kk), idesc,
           (accumulate || kk > 0) ? 1u : 0u, leader);
}

// acc[128 x DPAD] (+)= A[128 x 128] * B[128 x DPAD], A 16-bit in SHARED memory as two atoms of 64 columns
// (128-byte rows, 128-byte swizzle, 16 KB apart).  kTransA = false: A rows are the stored rows (K-major read).
// kTransA = true: A is the transpose of what is stored (MN-major read).
template <typename TR, bool kTransA>
__device__ __forceinline__ void issue_ds_blocks(bool leader, uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile,
                                                uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t ad = kTransA ? make_smem_desc(a_tile + kk * 2048, 16384, 1024, kSwizzle128)
                                : make_smem_desc(a_tile + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, kSwizzle128);
    mma_ss(d_tmem, ad, rows_b_desc<TR>(b_tile, kk), idesc, (accumulate || kk > 0) ? 1u : 0u, leader);
  }
}

// TMA load / store of a whole tile, block by block (columns beyond the head dim are filled with zeros on the way
// in and clipped on the way out)
// (shift = 8: the tile starts 8 columns before the head; those columns come back as zeros and head-dim column d
// lies at tile column d + 8)
template <typename TR>
__device__ __forceinline__ void load_tile_blocks(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row0, int h,
                                                 int b, int shift) {
#pragma unroll
  for (int a = 0; a < TR::kAtoms; ++a) tma_load_4d(dst + a * TR::kAtomBytes, map, bar, 16 * a - shift, row0, h, b);
}

// 8 when the rows of head (b, h) of tensor group grp start in the middle of a 32-byte sector and may be shifted
__device__ __forceinline__ int stream_shift(const BwdStreamParams& p, int grp, int b, int h) {
  if (!p.align_enable[grp]) return 0;
  return (((p.align0[grp] + b * p.align_b[grp] + h * p.align_h[grp]) & 31) == 16) ? 8 : 0;
}
template <typename TR>
__device__ __forceinline__ void store_tile_blocks(const CUtensorMap* map, uint32_t src, int row0, int h, int b) {
#pragma unroll
  for (int a = 0; a < TR::kAtoms; ++a) tma_store_4d(map, src + a * TR::kAtomBytes, 16 * a, row0, h, b);
}

// ---- -delta = -rowsum(dO * O) and -lse * log2(e), fp32, written as (B, H, L) ----
// A block takes `lrows` consecutive positions l of one batch element, all heads: one thread per 16-byte chunk of a
// row (consecutive threads read consecutive chunks), the chunk sums of a row added up in a fixed order by one
// thread, which then writes with l running fastest (32 consecutive positions of a head are 128 contiguous bytes).
template <typename T>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout,
                                                        const float* __restrict__ lse, float* __restrict__ ndelta,
                                                        float* __restrict__ nlse2, int batch, int seqlen, int heads,
                                                        int head_dim, int lrows, int64_t o_sb, int64_t o_sl,
                                                        int64_t o_sh, int64_t do_sb, int64_t do_sl, int64_t do_sh) {
  extern __shared__ float dl_part[];  // [lrows * heads][chunks]
  const int chunks = head_dim / 8;
  const int rows = lrows * heads;
  const int groups_per_b = seqlen / lrows;
  for (int grp = blockIdx.x; grp < batch * groups_per_b; grp += gridDim.x) {
    const int b = grp / groups_per_b;
    const int l0 = (grp % groups_per_b) * lrows;
    for (int item = threadIdx.x; item < rows * chunks; item += blockDim.x) {
      const int r = item / chunks, c = item % chunks;
      const int l = l0 + r / heads, h = r % heads;
      const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o + b * o_sb + l * o_sl + h * o_sh) + c);
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dout + b * do_sb + l * do_sl + h * do_sh) + c);
      const uint32_t ou[4] = {ov.x, ov.y, ov.z, ov.w}, du[4] = {dv.x, dv.y, dv.z, dv.w};
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = unpack2<T>(ou[i]), g = unpack2<T>(du[i]);
        acc = fmaf(a.x, g.x, acc);
        acc = fmaf(a.y, g.y, acc);
      }
      dl_part[item] = acc;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows; idx += blockDim.x) {
      const int h = idx / lrows, li = idx % lrows;
      const float* part = dl_part + (li * heads + h) * chunks;
      float acc = 0.f;
      for (int c = 0; c < chunks; ++c) acc += part[c];
      const int64_t at = (static_cast<int64_t>(b) * heads + h) * seqlen + l0 + li;
      ndelta[at] = -acc;
      nlse2[at] = -lse[at] * 1.4426950408889634f;
    }
    __syncthreads();
  }
}

// ---- dq = scale * accumulator, rounded to T: one block per (b, h, query tile) ----
// The tile is read as it lies ([column / 4][row][4] floats, coalesced, four loads in flight per thread) into
// shared memory; every thread then writes 8 consecutive columns of one row (16 bytes), threads of a row next to
// each other.
template <typename T>
__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, int heads,
                                                             int head_dim, int tiles_per_bh, int64_t sb, int64_t sl,
                                                             int64_t sh, float scale) {
  extern __shared__ float4 cv_tile[];  // [head_dim / 4][128]
  const int groups = head_dim / 4;
  const int64_t tile = blockIdx.x;
  const float4* src = reinterpret_cast<const float4*>(acc) + tile * (static_cast<int64_t>(groups) * 128);
  const int n = groups * 128;
  for (int i0 = threadIdx.x; i0 < n; i0 += 4 * 256) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * 256 < n) v[u] = __ldcs(src + i0 + u * 256);  // read once: streaming
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * 256 < n) cv_tile[i0 + u * 256] = v[u];
  }
  __syncthreads();
  const int i_tile = static_cast<int>(tile % tiles_per_bh);
  const int64_t bh = tile / tiles_per_bh;
  const int h = static_cast<int>(bh % heads), b = static_cast<int>(bh / heads);
  const int chunks = head_dim / 8;
  for (int i = threadIdx.x; i < 128 * chunks; i += blockDim.x) {
    const int row = i / chunks, ch = i % chunks;
    const float4 x = cv_tile[(2 * ch) * 128 + row], y = cv_tile[(2 * ch + 1) * 128 + row];
    uint4 out;
    out.x = Pack2<T>::pack(x.x * scale, x.y * scale);
    out.y = Pack2<T>::pack(x.z * scale, x.w * scale);
    out.z = Pack2<T>::pack(y.x * scale, y.y * scale);
    out.w = Pack2<T>::pack(y.z * scale, y.w * scale);
    T* dst = dq + b * sb + (static_cast<int64_t>(i_tile) * 128 + row) * sl + h * sh + ch * 8;
    *reinterpret_cast<uint4*>(dst) = out;
  }
}

constexpr int kRoleStreamStore = 500;

// Diagnostic builds only (-DDMF_STREAM_DIAG=mask): leave parts of a step out to see what the rest costs.  The
// results are then wrong, only the timing is of interest.  1: elementwise math, 2: the atomics, 4: S, 8: dP,
// 16: dV, 32: dK, 64: the dQ partial (products skipped, their commits kept).
#ifdef DMF_STREAM_DIAG
constexpr int kStreamDiag = DMF_STREAM_DIAG;
#else
constexpr int kStreamDiag = 0;
#endif

// In-kernel timeline for diagnostic builds (-DDMF_TRACE), in the list the two-tile kernel's trace uses: the first
// thread of each role in CTA 0.
#ifdef DMF_TRACE
#define DMF_STRACE_EVENT(role, id)                                                                      \
  do {                                                                                                   \
    if (blockIdx.x == 0 && lane == 0 && trace_n < kTraceEvents)                                          \
      g_bwd_fused_trace[0][role][trace_n++] = (static_cast<unsigned long long>(clock64()) << 8) | (id); \
  } while (0)
#else
#define DMF_STRACE_EVENT(role, id) do { } while (0)
#endif

// ---- the kernel ---------------------------------------------------------------
// Steps are counted through all key tiles of this CTA (g); step g uses Q slot g % 3, dO slot g % 2, dS buffer
// g % 2.  Every barrier that completes once per step is waited with the parity of its own completion count.
template <typename T, int TAIL>
__global__ void __launch_bounds__(kBwdStreamThreads, 1)
attn_bwd_stream_kernel(const __grid_constant__ BwdStreamParams p) {
  using TR = BwdStreamTraits<TAIL>;
  constexpr int DPAD = TR::kDPad;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_kv = s_base + TR::kOffKV, s_q = s_base + TR::kOffQ, s_do = s_base + TR::kOffDo;
  const uint32_t s_ds = s_base + TR::kOffDs, s_rows = s_base + TR::kOffRows;
  const float* rows = reinterpret_cast<const float*>(smem + TR::kOffRows);  // [slot][-lse log2 e: 128 | -delta: 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::kOffBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + TR::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) -> uint32_t { return bar0 + 8u * static_cast<uint32_t>(i); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int J = p.steps;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < TR::kNumBars; ++i) {
      uint32_t count = 1;  // TMA transaction, tcgen05.commit, or the drain warps' issuing thread
      if (i == TR::kBarPFull || i == TR::kBarGFull || i == TR::kBarSEmpty) count = 8;  // one arrival per elementwise warp
      if (i == TR::kBarQpEmpty || i == TR::kBarAccEmpty || i == TR::kBarKVStaged)
        count = 4;                                              // one arrival per drain warp
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
      prefetch_tensor_map(&p.q);
      prefetch_tensor_map(&p.dout);
      prefetch_tensor_map(&p.k);
      prefetch_tensor_map(&p.v);
      uint32_t tcnt = 0, g = 0;
      bool ok = true;
      DMF_TRACE_DECL
      auto wait = [&](int b_, uint32_t parity) -> bool {
        return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleProducer + b_);
      };
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt) {
        const int bh = tile / p.tiles_per_bh;
        const int k0 = (tile % p.tiles_per_bh) * 128;
        const int b = bh / p.heads, h = bh % p.heads;
        const int64_t row0 = (static_cast<int64_t>(b) * p.heads + h) * p.seqlen_q;
        const int sqk = stream_shift(p, 0, b, h), svo = stream_shift(p, 1, b, h);
        for (int i = 0; ok && i < J; ++i, ++g) {
          const int q0 = i * 128;
          {  // Q_i with its two rows: the slot was freed by the last product of step g - 3
            const uint32_t sl = g % 3u;
            ok = wait(TR::kBarStepDone + sl, ((g / 3u) & 1u) ^ 1u);
            if (!ok) break;
            const uint32_t dst = s_q + sl * TR::kTileBytes, fb = bar(TR::kBarQFull + sl);
            mbar_arrive_expect_tx(fb, TR::kTileBytes + TR::kRowBytes);
            load_tile_blocks<TR>(dst, &p.q, fb, q0, h, b, sqk);
            bulk_load_1d(s_rows + sl * TR::kRowBytes, p.nlse2 + row0 + q0, 512, fb);
            bulk_load_1d(s_rows + sl * TR::kRowBytes + 512, p.ndelta + row0 + q0, 512, fb);
            DMF_STRACE_EVENT(0, 1);
          }
          {  // dO_i: the slot was freed by dV += P^T dO of step g - 2
            const uint32_t sl = g & 1u;
            ok = wait(TR::kBarPvDone + sl, ((g >> 1) & 1u) ^ 1u);
            if (!ok) break;
            const uint32_t dst = s_do + sl * TR::kTileBytes, fb = bar(TR::kBarDoFull + sl);
            mbar_arrive_expect_tx(fb, TR::kTileBytes);
            load_tile_blocks<TR>(dst, &p.dout, fb, q0, h, b, svo);
            DMF_STRACE_EVENT(0, 2);
          }
          if (i == 0) {  // K_j, then V_j: free when every product of the previous key tile is complete (the first
                         // Q and dO tiles of this key tile are already on their way by then)
            if (tcnt > 0) ok = wait(TR::kBarTileDone, (tcnt - 1u) & 1u);
            if (!ok) break;
            const uint32_t fk = bar(TR::kBarKFull), fv = bar(TR::kBarVFull);
            mbar_arrive_expect_tx(fk, TR::kTileBytes);
            load_tile_blocks<TR>(s_kv, &p.k, fk, k0, h, b, sqk);
            mbar_arrive_expect_tx(fv, TR::kTileBytes);
            load_tile_blocks<TR>(s_kv + TR::kTileBytes, &p.v, fv, k0, h, b, svo);
            DMF_STRACE_EVENT(0, 3);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ================================
    // Products issued by this thread execute in the order of issue: accumulating products follow one another
    // without a wait.
    const bool leader = elect_one();
    auto commit = [&](int b_) { tc_commit(bar(b_), leader); };
    constexpr uint32_t idesc_qk = make_idesc(kBf16, false, false, 128, 128);
    constexpr uint32_t idesc_pv = make_idesc(kBf16, false, true, 128, DPAD);
    constexpr uint32_t idesc_tr = make_idesc(kBf16, true, true, 128, DPAD);   // A read transposed
    const uint32_t t_s = tmem + TR::kColS, t_p = tmem + TR::kColP, t_d = tmem + TR::kColD, t_qp = tmem + TR::kColQp;
    const uint32_t t_dk = tmem + TR::kColDK, t_dv = tmem + TR::kColDV;
    const uint32_t k_tile = s_kv, v_tile = s_kv + TR::kTileBytes;
    uint32_t tcnt = 0, g0 = 0;
    bool ok = true;
    DMF_TRACE_DECL
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleMma + b_);
    };
    auto q_tile = [&](uint32_t g) -> uint32_t { return s_q + (g % 3u) * TR::kTileBytes; };
    auto do_tile = [&](uint32_t g) -> uint32_t { return s_do + (g & 1u) * TR::kTileBytes; };
    // S_g = K Q_g^T: the Q tile is there, and the elementwise warps have S_{g-1} in registers
    auto issue_s = [&](uint32_t g) -> bool {
      bool r = wait(TR::kBarQFull + g % 3u, (g / 3u) & 1u);
      if (r && g > 0) r = wait(TR::kBarSEmpty, (g - 1u) & 1u);
      if (!r) return false;
      tc_fence_after_sync();
      if (!(kStreamDiag & 4)) issue_qk_blocks<TR>(leader, t_s, k_tile, q_tile(g), idesc_qk);
      commit(TR::kBarSFull);
      return true;
    };
    // dP_g = V dO_g^T: the dO tile is there, and the drain warps have the dQ partial of step g - 1 (which lies in
    // the same columns, and was issued after dP_{g-1} had been read) in registers
    auto issue_dp = [&](uint32_t g) -> bool {
      bool r = wait(TR::kBarDoFull + (g & 1u), (g >> 1) & 1u);
      if (r && g > 0) r = wait(TR::kBarQpEmpty, (g - 1u) & 1u);
      if (!r) return false;
      tc_fence_after_sync();
      if (!(kStreamDiag & 8)) issue_qk_blocks<TR>(leader, t_d, v_tile, do_tile(g), idesc_qk);
      commit(TR::kBarDFull);
      return true;
    };
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt, g0 += static_cast<uint32_t>(J)) {
      // ---- S_0, dP_0, S_1 ----
      ok = wait(TR::kBarKFull, tcnt & 1u) && issue_s(g0);
      if (ok) ok = wait(TR::kBarVFull, tcnt & 1u) && issue_dp(g0);
      if (ok && J > 1) ok = issue_s(g0 + 1u);
      if (!ok) break;
      for (int k = 0; k < J; ++k) {
        const uint32_t g = g0 + static_cast<uint32_t>(k);
        const uint32_t ds_buf = s_ds + (g & 1u) * TR::kDsBytes;
        ok = wait(TR::kBarPFull, g & 1u);
        if (ok && k == 0 && tcnt > 0) ok = wait(TR::kBarAccEmpty, (tcnt - 1u) & 1u);  // the previous dK, dV have been read
        if (!ok) break;
        tc_fence_after_sync();
        DMF_STRACE_EVENT(1, 10);
        if (!(kStreamDiag & 16)) issue_pv_blocks<TR>(leader, t_dv, t_p, do_tile(g), idesc_pv, k > 0);  // dV += P^T dO
        commit(TR::kBarPvDone + (g & 1u));                    // dO slot free, P may be overwritten
        ok = wait(TR::kBarGFull, g & 1u);                     // dS_k is in shared memory, dP_k has been read
        if (!ok) break;
        tc_fence_after_sync();
        DMF_STRACE_EVENT(1, 14);
        if (!(kStreamDiag & 64)) issue_ds_blocks<TR, true>(leader, t_qp, ds_buf, k_tile, idesc_tr, false);        // dQ partial = dS K
        commit(TR::kBarQpFull);
        if (!(kStreamDiag & 32)) issue_ds_blocks<TR, false>(leader, t_dk, ds_buf, q_tile(g), idesc_pv, k > 0);    // dK += dS^T Q
        commit(TR::kBarStepDone + g % 3u);                    // Q slot free, dS buffer dead
        DMF_STRACE_EVENT(1, 11);
        if (k + 1 < J) {
          ok = issue_dp(g + 1u);
          if (!ok) break;
          DMF_STRACE_EVENT(1, 12);
        }
        if (k + 2 < J) {
          ok = issue_s(g + 2u);
          if (!ok) break;
          DMF_STRACE_EVENT(1, 13);
        }
      }
      if (!ok) break;
      commit(TR::kBarTileDone);
    }
  } else if (warp < 10) {
    // ========================= elementwise warps ============================
    // warp (quarter, half): key rows 32 quarter .. + 31 (its tensor-memory lanes), query columns 64 half .. + 63
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem + lane_base + TR::kColS + half * 64;   // S columns of this warp
    const uint32_t t_p = tmem + lane_base + TR::kColP + half * 32;   // its P columns (two queries per column)
    const uint32_t t_d = tmem + lane_base + TR::kColD + half * 64;
    const float sl2 = p.scale_log2e;
    const uint64_t sl2_2 = pack_f2(sl2, sl2);
    uint32_t tcnt = 0, g0 = 0;
    bool ok = true;
    DMF_TRACE_DECL
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleSoftmax + b_));
    };
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt, g0 += static_cast<uint32_t>(J)) {
      for (int k = 0; k < J; ++k) {
        const uint32_t g = g0 + static_cast<uint32_t>(k);
        const float* nrow = rows + (g % 3u) * 256 + half * 64;        // -lse log2 e of this warp's 64 queries
        const float* drow = rows + (g % 3u) * 256 + 128 + half * 64;  // -delta of the same
        uint8_t* ds_rows = smem + TR::kOffDs + (g & 1u) * TR::kDsBytes + half * 16384 + row * 128;
        ok = wait(TR::kBarQFull + g % 3u, (g / 3u) & 1u);             // (the two rows came with the Q tile)
        if (ok) ok = wait(TR::kBarSFull, g & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        if (warp == 2) DMF_STRACE_EVENT(2, 30);
        // ---- P^T = exp2(S^T c - lse log2 e), 16-bit ----
        uint32_t pk[32];
        {
          uint32_t r[2][32];
          tmem_ld_x32(t_s, r[0]);
          tmem_ld_x32(t_s + 32, r[1]);
          tmem_wait_ld();
          tc_fence_before_sync();
          mbar_arrive_warp(bar(TR::kBarSEmpty));  // S is in registers: the next S may be written
          if (warp == 2) DMF_STRACE_EVENT(2, 31);
#pragma unroll
          for (int c = 0; c < ((kStreamDiag & 1) ? 0 : 2); ++c) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 nv = *reinterpret_cast<const float4*>(nrow + c * 32 + i);
              float x0, x1, x2, x3;
              unpack_f2(fma2(pack_u2(r[c][i], r[c][i + 1]), sl2_2, pack_f2(nv.x, nv.y)), x0, x1);
              unpack_f2(fma2(pack_u2(r[c][i + 2], r[c][i + 3]), sl2_2, pack_f2(nv.z, nv.w)), x2, x3);
              pk[c * 16 + i / 2] = Pack2<T>::pack(fast_exp2(x0), fast_exp2(x1));
              pk[c * 16 + i / 2 + 1] = Pack2<T>::pack(fast_exp2(x2), fast_exp2(x3));
            }
          }
        }
        if (warp == 2) DMF_STRACE_EVENT(2, 32);
        if (g > 0) {  // dV += P^T dO of the step before has read the P columns
          ok = wait(TR::kBarPvDone + ((g - 1u) & 1u), ((g - 1u) >> 1) & 1u);
          if (!ok) break;
          tc_fence_after_sync();
        }
        tmem_st_x32(t_p, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(bar(TR::kBarPFull));
        if (warp == 2) DMF_STRACE_EVENT(2, 34);
        // ---- dS^T = P^T * (dP^T + (-delta)), 16-bit, into the step's shared-memory buffer ----
        ok = wait(TR::kBarDFull, g & 1u);
        // the buffer: the products of step g - 2 are done with it; in the first two steps of a key tile, the
        // stores of the previous tile's dK / dV, which were staged in the two buffers
        if (ok && k >= 2) ok = wait(TR::kBarStepDone + (g - 2u) % 3u, ((g - 2u) / 3u) & 1u);
        if (ok && k < 2 && tcnt > 0) ok = wait(TR::kBarStageFree, (tcnt - 1u) & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        if (warp == 2) DMF_STRACE_EVENT(2, 35);
        uint32_t d[2][32];
        tmem_ld_x32(t_d, d[0]);
        tmem_ld_x32(t_d + 32, d[1]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < ((kStreamDiag & 1) ? 0 : 2); ++c) {
          uint32_t out[16];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float4 nd = *reinterpret_cast<const float4*>(drow + c * 32 + 2 * i);
            const float2 pa = unpack2<T>(pk[c * 16 + i]), pb = unpack2<T>(pk[c * 16 + i + 1]);
            float g0_, g1_, g2_, g3_;
            unpack_f2(mul2(pack_f2(pa.x, pa.y), add2(pack_u2(d[c][2 * i], d[c][2 * i + 1]), pack_f2(nd.x, nd.y))), g0_, g1_);
            unpack_f2(mul2(pack_f2(pb.x, pb.y), add2(pack_u2(d[c][2 * i + 2], d[c][2 * i + 3]), pack_f2(nd.z, nd.w))), g2_, g3_);
            out[i] = Pack2<T>::pack(g0_, g1_);
            out[i + 1] = Pack2<T>::pack(g2_, g3_);
          }
          // query columns 64 half + 32 c .. + 31 of this key row: atom `half`, 16-byte chunks 4 c .. 4 c + 3
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            *reinterpret_cast<uint4*>(ds_rows + (((c * 4 + kk) ^ (row & 7)) << 4)) =
                make_uint4(out[4 * kk], out[4 * kk + 1], out[4 * kk + 2], out[4 * kk + 3]);
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive_warp(bar(TR::kBarGFull));  // dS^T is in shared memory, dP has been read
        if (warp == 2) DMF_STRACE_EVENT(2, 36);
      }
    }
  } else {
    // ============================== drain warps =============================
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;   // query row of a dQ partial; key row of dK / dV
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_qp = tmem + lane_base + TR::kColQp, t_dk = tmem + lane_base + TR::kColDK;
    const bool issuer = (warp == 10) && (lane == 0);  // issues the TMA stores
    const int groups = p.head_dim >> 2;               // real column groups of four (padding columns are dropped)
    uint32_t tcnt = 0, g0 = 0;
    bool ok = true;
    DMF_TRACE_DECL
    auto wait = [&](int b_, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar(b_), parity, abort_flag, p.status_word, kRoleStreamStore + b_));
    };
    auto chunk_off = [&](int cc) -> uint32_t {  // 16-byte chunk of head-dim column cc of this thread's row in a tile
      return static_cast<uint32_t>((cc >> 4) * TR::kAtomBytes + row * 32 + ((((cc >> 3) & 1) ^ ((row >> 2) & 1)) << 4));
    };
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++tcnt, g0 += static_cast<uint32_t>(J)) {
      const int bh = tile / p.tiles_per_bh;
      const int k0 = (tile % p.tiles_per_bh) * 128;
      const int b = bh / p.heads, h = bh % p.heads;
      // where the head's tiles were loaded 8 columns early, accumulator column c is head-dim column c - 8: the dQ
      // partial and dK follow q and k, dV follows v and dout
      const int sqk = stream_shift(p, 0, b, h), svo = stream_shift(p, 1, b, h);
      const int gs = sqk >> 2;  // column groups of four to skip in the dQ partial
      for (int k = 0; k < J; ++k) {
        const uint32_t g = g0 + static_cast<uint32_t>(k);
        // the dQ partial -> registers, so that its columns can take the next dP at once
        ok = wait(TR::kBarQpFull, g & 1u);
        if (!ok) break;
        tc_fence_after_sync();
        if (warp == 10) DMF_STRACE_EVENT(3, 53);
        uint32_t a[DPAD / 16][16];
#pragma unroll
        for (int c = 0; c < DPAD / 16; ++c) tmem_ld_x16(t_qp + c * 16, a[c]);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive_warp(bar(TR::kBarQpEmpty));
        // registers -> the fp32 accumulator tile of query tile k: [column / 4][row][4], a warp's 32 rows of one
        // column group are 512 contiguous bytes
        float* acc = p.dq_acc + (static_cast<int64_t>(bh) * J + k) * (static_cast<int64_t>(p.head_dim) * 128) + row * 4;
#pragma unroll
        for (int c = 0; c < DPAD / 16; ++c) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            if (c * 4 + q4 >= gs && c * 4 + q4 - gs < groups && !(kStreamDiag & 2))
              red_add_v4(acc + (c * 4 + q4 - gs) * 512, a[c][4 * q4], a[c][4 * q4 + 1], a[c][4 * q4 + 2], a[c][4 * q4 + 3]);
        }
        if (warp == 10) DMF_STRACE_EVENT(3, 51);
      }
      // ---- end of the key tile: dK (scaled) staged in dS buffer 0, dV in dS buffer 1, then stored ----
      if (ok) ok = wait(TR::kBarTileDone, tcnt & 1u);  // every product of the tile is complete: the dS buffers are dead
      if (!ok) break;
      tc_fence_after_sync();
      uint8_t* dk_stage = smem + TR::kOffDs;
      uint8_t* dv_stage = smem + TR::kOffDs + TR::kDsBytes;
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
        for (int hh = 0; hh < 2; ++hh) {  // the staged tiles are NOT shifted (a store must not start left of column 0)
          const int ck = c * 16 + hh * 8 - sqk, cv = c * 16 + hh * 8 - svo;
          if (ck >= 0)
            *reinterpret_cast<uint4*>(dk_stage + chunk_off(ck)) = make_uint4(p0[4 * hh], p0[4 * hh + 1], p0[4 * hh + 2], p0[4 * hh + 3]);
          if (cv >= 0)
            *reinterpret_cast<uint4*>(dv_stage + chunk_off(cv)) = make_uint4(p1[4 * hh], p1[4 * hh + 1], p1[4 * hh + 2], p1[4 * hh + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive_warp(bar(TR::kBarAccEmpty));  // the next key tile may overwrite dK, dV
      fence_proxy_async_smem();
      mbar_arrive_warp(bar(TR::kBarKVStaged));
      if (warp == 10) {
        ok = wait(TR::kBarKVStaged, tcnt & 1u);   // all 128 rows of both tiles are staged
        if (ok && issuer) {
          store_tile_blocks<TR>(&p.dk, s_ds, k0, h, b);
          store_tile_blocks<TR>(&p.dv, s_ds + TR::kDsBytes, k0, h, b);
          tma_store_commit();
          tma_store_wait_read();                  // both staging tiles have been read
          mbar_arrive(bar(TR::kBarStageFree));
        }
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    if (issuer) tma_store_wait_all();             // the stores of this thread are complete
  }

  // ============================== teardown ==================================
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem, TR::kTmemCols);
}

}  // namespace dmf
