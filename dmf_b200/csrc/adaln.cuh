// adaLN-Zero elementwise ops of the DiT block with their tangents, and their primal backwards:
//
//   y   = LayerNorm(x) (1 + scale) + shift           (models/layers.py:28-29 modulate, :196-197, :219)
//   out = x + gate * h                               (models/layers.py:196-197)
//
// One warp owns one row of C channels: lane i holds the 4-channel vectors i, i + 32, ... (every load
// of the warp is 512 contiguous bytes of fp32, 256 of bf16) and keeps the whole row in registers, so
// each tensor is read once and written once and the row statistics are plain warp shuffles.  The
// LayerNorm kernels and the backward kernels are compiled per NV = C / 128 vectors per lane.
// Arithmetic is fp32; the variance is the two-pass one (mean first, then centred squares).
//
// Backward kernels: the sums over l (dshift, dscale, dgate) are kept per warp (in shared memory for the
// LayerNorm backward, in registers for the gate backward) over the rows of one (batch, row-range) block,
// added across the block's 8 warps, and written as one partial row per block; a second small kernel adds the partials of a batch in a
// fixed order (no atomics: bit-reproducible).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace dmf {

// two bf16 in a 32-bit word <-> two floats
__device__ __forceinline__ float2 ada_unpack_bf16x2(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
__device__ __forceinline__ uint32_t ada_pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct AdaParams {
  const void *x, *tx;          // wide rows
  const void *h, *th;          // narrow rows
  const void *dy;              // narrow rows (LayerNorm backward) / wide rows dout (gate backward)
  const void *shift, *scale, *tshift, *tscale, *gate, *tgate;  // (B, C)
  void *y, *ty;                // narrow rows (LayerNorm) / wide rows out, tout (gate)
  void *dx;                    // wide rows dx (LayerNorm backward) / narrow rows dh (gate backward)
  float* partial;              // (B, splits, nq, C)
  int64_t x_sb, x_sl, tx_sb, tx_sl, h_sb, h_sl, th_sb, th_sl, dy_sb, dy_sl;
  int64_t y_sb, y_sl, ty_sb, ty_sl, dx_sb, dx_sl;
  int64_t shift_sb, scale_sb, tshift_sb, tscale_sb, gate_sb, tgate_sb;
  int batch, seqlen, channels;
  int mod_f32;                 // shift / scale / gate are fp32 (else bf16)
  int rows_per_block, splits;  // backward: rows of one block, blocks per batch
  float eps;
};

constexpr int kAdaThreads = 256;
constexpr int kAdaWarps = kAdaThreads / 32;

__device__ __forceinline__ float ada_warp_sum(float v) {
#pragma unroll
  for (int d = 16; d >= 1; d /= 2) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// 4 consecutive channels <-> 4 floats
__device__ __forceinline__ void ada_load4(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void ada_load4(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = ada_unpack_bf16x2(v.x), b = ada_unpack_bf16x2(v.y);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void ada_store4(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void ada_store4(__nv_bfloat16* p, const float (&f)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(ada_pack_bf16x2(f[0], f[1]), ada_pack_bf16x2(f[2], f[3]));
}
// a (B, C) modulation tensor, fp32 or bf16 (the same for the whole launch)
__device__ __forceinline__ void ada_mod4(const void* base, int f32, int64_t off, float (&f)[4]) {
  if (f32) ada_load4(reinterpret_cast<const float*>(base) + off, f);
  else ada_load4(reinterpret_cast<const __nv_bfloat16*>(base) + off, f);
}

// ---- y = LayerNorm(x) (1 + scale) + shift, with tangent ----
// grid (splits, batch); block (s, b) owns rows [s * rows_per_block, (s + 1) * rows_per_block) of batch b, so that the
// batch's modulation rows are staged once per block in shared memory as fp32 (1 + scale, shift, tscale, tshift).
// Reading them from global memory inside the per-vector loop put nine dependent L2 round trips into every row
// (2.7 TB/s with 16 warps per SM).
template <typename TW, typename TN, int NV, bool kDual>
__global__ void __launch_bounds__(kAdaThreads) ln_modulate_fwd_kernel(const AdaParams p) {
  constexpr int C = NV * 128;
  constexpr float kInvC = 1.f / static_cast<float>(C);
  __shared__ __align__(16) float s_mod[(kDual ? 4 : 2) * C];  // [1 + scale | shift | tscale | tshift]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.y;
  const int l0 = blockIdx.x * p.rows_per_block;
  const int l1 = min(p.seqlen, l0 + p.rows_per_block);
  const bool tmod = kDual && p.tshift != nullptr;
  for (int c = 4 * threadIdx.x; c < C; c += 4 * kAdaThreads) {
    float v[4];
    ada_mod4(p.scale, p.mod_f32, b * p.scale_sb + c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) s_mod[c + i] = 1.f + v[i];
    ada_mod4(p.shift, p.mod_f32, b * p.shift_sb + c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) s_mod[C + c + i] = v[i];
    if constexpr (kDual) {
      float z[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
      if (tmod) {
        ada_mod4(p.tscale, p.mod_f32, b * p.tscale_sb + c, z);
        ada_mod4(p.tshift, p.mod_f32, b * p.tshift_sb + c, w);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s_mod[2 * C + c + i] = z[i];
        s_mod[3 * C + c + i] = w[i];
      }
    }
  }
  __syncthreads();
  for (int l = l0 + warp; l < l1; l += kAdaWarps) {
    const TW* xp = reinterpret_cast<const TW*>(p.x) + b * p.x_sb + l * p.x_sl;
    const TW* txp = reinterpret_cast<const TW*>(p.tx) + b * p.tx_sb + l * p.tx_sl;
    float x[NV][4], tx[NV][4];
#pragma unroll
    for (int k = 0; k < NV; ++k) ada_load4(xp + 4 * (lane + 32 * k), x[k]);
    if constexpr (kDual) {
#pragma unroll
      for (int k = 0; k < NV; ++k) ada_load4(txp + 4 * (lane + 32 * k), tx[k]);
    }
    float s = 0.f, ts = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s += x[k][i];
        if constexpr (kDual) ts += tx[k][i];
      }
    const float mean = ada_warp_sum(s) * kInvC;
    float tmean = 0.f;
    if constexpr (kDual) tmean = ada_warp_sum(ts) * kInvC;
    float v = 0.f, d = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[k][i] -= mean;
        v = fmaf(x[k][i], x[k][i], v);
        if constexpr (kDual) {
          tx[k][i] -= tmean;
          d = fmaf(x[k][i], tx[k][i], d);
        }
      }
    const float r = rsqrtf(ada_warp_sum(v) * kInvC + p.eps);
    float coef = 0.f;  // mean(n * centred tx)
    if constexpr (kDual) coef = r * ada_warp_sum(d) * kInvC;
    TN* yp = reinterpret_cast<TN*>(p.y) + b * p.y_sb + l * p.y_sl;
    TN* typ = reinterpret_cast<TN*>(p.ty) + b * p.ty_sb + l * p.ty_sl;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = 4 * (lane + 32 * k);
      const float4 sc = *reinterpret_cast<const float4*>(s_mod + c);       // 1 + scale
      const float4 sh = *reinterpret_cast<const float4*>(s_mod + C + c);
      const float sc_[4] = {sc.x, sc.y, sc.z, sc.w}, sh_[4] = {sh.x, sh.y, sh.z, sh.w};
      float y[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[k][i] *= r;  // n
        y[i] = fmaf(x[k][i], sc_[i], sh_[i]);
      }
      ada_store4(yp + c, y);
      if constexpr (kDual) {
        const float4 tc = *reinterpret_cast<const float4*>(s_mod + 2 * C + c);
        const float4 th = *reinterpret_cast<const float4*>(s_mod + 3 * C + c);
        const float tc_[4] = {tc.x, tc.y, tc.z, tc.w}, th_[4] = {th.x, th.y, th.z, th.w};
        float ty[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          ty[i] = fmaf(r * fmaf(-x[k][i], coef, tx[k][i]), sc_[i], fmaf(x[k][i], tc_[i], th_[i]));
        ada_store4(typ + c, ty);
      }
    }
  }
}

// Adds the per-warp column sums acc[NV][4] of a block's 8 warps and writes them as row `q` of the
// block's partial (nq rows of C floats).  All threads of the block must call it.
template <int NV>
__device__ __forceinline__ void ada_block_column_sum(float (*red)[NV * 128], const float (&acc)[NV][4], float* partial_row) {
  constexpr int C = NV * 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // the previous use of red is over
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp][4 * (lane + 32 * k) + i] = acc[k][i];
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += kAdaThreads) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kAdaWarps; ++w) s += red[w][c];
    partial_row[c] = s;
  }
}

// ---- backward of y = LayerNorm(x) (1 + scale) + shift ----
// grid (splits, batch); block (s, b) owns rows [s * rows_per_block, (s + 1) * rows_per_block) of batch b.
// The column sums of dshift / dscale are kept per warp in shared memory, not in registers: 72 registers less per
// thread, two blocks per SM instead of one (4330 -> 5560 GB/s at 64 x 1024 rows of 1152 channels).
// Dynamic shared memory: (1 + 16) * C floats.
template <typename TW, typename TN, int NV>
__global__ void __launch_bounds__(kAdaThreads, 2) ln_modulate_bwd_kernel(const AdaParams p) {
  constexpr int C = NV * 128;
  constexpr float kInvC = 1.f / static_cast<float>(C);
  extern __shared__ __align__(16) float ada_dyn[];
  float* s_sc = ada_dyn;            // 1 + scale of this batch
  float* s_acc = ada_dyn + C;       // [warp][shift | scale][C]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.y;
  const int l0 = blockIdx.x * p.rows_per_block;
  const int l1 = min(p.seqlen, l0 + p.rows_per_block);
  for (int c = 4 * threadIdx.x; c < C; c += 4 * kAdaThreads) {
    float v[4];
    ada_mod4(p.scale, p.mod_f32, b * p.scale_sb + c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) s_sc[c + i] = 1.f + v[i];
  }
  float* my_shift = s_acc + (warp * 2) * C;
  float* my_scale = my_shift + C;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    *reinterpret_cast<float4*>(my_shift + 4 * (lane + 32 * k)) = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(my_scale + 4 * (lane + 32 * k)) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  for (int l = l0 + warp; l < l1; l += kAdaWarps) {
    const TW* xp = reinterpret_cast<const TW*>(p.x) + b * p.x_sb + l * p.x_sl;
    const TN* gp = reinterpret_cast<const TN*>(p.dy) + b * p.dy_sb + l * p.dy_sl;
    float x[NV][4], g[NV][4];
#pragma unroll
    for (int k = 0; k < NV; ++k) ada_load4(xp + 4 * (lane + 32 * k), x[k]);
#pragma unroll
    for (int k = 0; k < NV; ++k) ada_load4(gp + 4 * (lane + 32 * k), g[k]);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int i = 0; i < 4; ++i) s += x[k][i];
    const float mean = ada_warp_sum(s) * kInvC;
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[k][i] -= mean;
        v = fmaf(x[k][i], x[k][i], v);
      }
    const float r = rsqrtf(ada_warp_sum(v) * kInvC + p.eps);
    float sg = 0.f, sgn = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = 4 * (lane + 32 * k);
      const float4 sv = *reinterpret_cast<const float4*>(s_sc + c);
      const float sc[4] = {sv.x, sv.y, sv.z, sv.w};
      float4 a0 = *reinterpret_cast<float4*>(my_shift + c), a1 = *reinterpret_cast<float4*>(my_scale + c);
      float* a0_ = reinterpret_cast<float*>(&a0);
      float* a1_ = reinterpret_cast<float*>(&a1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[k][i] *= r;  // n
        a0_[i] += g[k][i];
        a1_[i] = fmaf(g[k][i], x[k][i], a1_[i]);
        g[k][i] *= sc[i];  // the gradient of n
        sg += g[k][i];
        sgn = fmaf(g[k][i], x[k][i], sgn);
      }
      *reinterpret_cast<float4*>(my_shift + c) = a0;
      *reinterpret_cast<float4*>(my_scale + c) = a1;
    }
    const float mg = ada_warp_sum(sg) * kInvC, mgn = ada_warp_sum(sgn) * kInvC;
    TW* dxp = reinterpret_cast<TW*>(p.dx) + b * p.dx_sb + l * p.dx_sl;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float dx[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dx[i] = r * (g[k][i] - mg - x[k][i] * mgn);
      ada_store4(dxp + 4 * (lane + 32 * k), dx);
    }
  }
  __syncthreads();
  float* prow = p.partial + ((b * p.splits + blockIdx.x) * 2) * C;
  for (int c = threadIdx.x; c < 2 * C; c += kAdaThreads) {  // c < C: dshift, else dscale
    const int q = c >= C, cc = c - q * C;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kAdaWarps; ++w) t += s_acc[(w * 2 + q) * C + cc];
    prow[c] = t;
  }
}

// out[q][b][c] = sum over s of partial[b][s][q][c], s in order.  grid (ceil(C / 256), batch, nq).
__global__ void __launch_bounds__(kAdaThreads) ada_partial_reduce_kernel(const float* partial, float* out0, float* out1,
                                                                         int splits, int channels, int nq) {
  const int c = blockIdx.x * kAdaThreads + threadIdx.x;
  if (c >= channels) return;
  const int64_t b = blockIdx.y;
  const int q = blockIdx.z;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += partial[((b * splits + k) * nq + q) * channels + c];
  (q == 0 ? out0 : out1)[b * channels + c] = s;
}

// ---- out = x + gate * h, with tangent; any C that is a multiple of 4 ----
template <typename TW, typename TN, bool kDual>
__global__ void __launch_bounds__(kAdaThreads) gate_residual_fwd_kernel(const AdaParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t rows = static_cast<int64_t>(p.batch) * p.seqlen;
  const int nvec = p.channels / 4;
  const bool tmod = kDual && p.tgate != nullptr;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kAdaWarps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kAdaWarps) {
    const int64_t b = row / p.seqlen, l = row - b * p.seqlen;
    const TW* xp = reinterpret_cast<const TW*>(p.x) + b * p.x_sb + l * p.x_sl;
    const TW* txp = reinterpret_cast<const TW*>(p.tx) + b * p.tx_sb + l * p.tx_sl;
    const TN* hp = reinterpret_cast<const TN*>(p.h) + b * p.h_sb + l * p.h_sl;
    const TN* thp = reinterpret_cast<const TN*>(p.th) + b * p.th_sb + l * p.th_sl;
    TW* op = reinterpret_cast<TW*>(p.y) + b * p.y_sb + l * p.y_sl;
    TW* top = reinterpret_cast<TW*>(p.ty) + b * p.ty_sb + l * p.ty_sl;
#pragma unroll 3
    for (int vi = lane; vi < nvec; vi += 32) {
      const int c = 4 * vi;
      float x[4], h[4], gt[4], o[4];
      ada_load4(xp + c, x);
      ada_load4(hp + c, h);
      ada_mod4(p.gate, p.mod_f32, b * p.gate_sb + c, gt);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = fmaf(gt[i], h[i], x[i]);
      ada_store4(op + c, o);
      if constexpr (kDual) {
        float tx[4], th[4], to[4];
        ada_load4(txp + c, tx);
        ada_load4(thp + c, th);
#pragma unroll
        for (int i = 0; i < 4; ++i) to[i] = fmaf(gt[i], th[i], tx[i]);
        if (tmod) {
          float tg[4];
          ada_mod4(p.tgate, p.mod_f32, b * p.tgate_sb + c, tg);
#pragma unroll
          for (int i = 0; i < 4; ++i) to[i] = fmaf(tg[i], h[i], to[i]);
        }
        ada_store4(top + c, to);
      }
    }
  }
}

// ---- backward of out = x + gate * h: dh = gate * dout, dgate = sum_l dout * h ----
template <typename TW, typename TN, int NV>
__global__ void __launch_bounds__(kAdaThreads) gate_residual_bwd_kernel(const AdaParams p) {
  constexpr int C = NV * 128;
  __shared__ float red[kAdaWarps][C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.y;
  const int l0 = blockIdx.x * p.rows_per_block;
  const int l1 = min(p.seqlen, l0 + p.rows_per_block);
  float gate[NV][4], acc[NV][4];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    ada_mod4(p.gate, p.mod_f32, b * p.gate_sb + 4 * (lane + 32 * k), gate[k]);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[k][i] = 0.f;
  }
  for (int l = l0 + warp; l < l1; l += kAdaWarps) {
    const TW* gp = reinterpret_cast<const TW*>(p.dy) + b * p.dy_sb + l * p.dy_sl;
    const TN* hp = reinterpret_cast<const TN*>(p.h) + b * p.h_sb + l * p.h_sl;
    TN* dhp = reinterpret_cast<TN*>(p.dx) + b * p.dx_sb + l * p.dx_sl;
    float g[NV][4], h[NV][4];
#pragma unroll
    for (int k = 0; k < NV; ++k) ada_load4(gp + 4 * (lane + 32 * k), g[k]);
#pragma unroll
    for (int k = 0; k < NV; ++k) ada_load4(hp + 4 * (lane + 32 * k), h[k]);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float dh[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[k][i] = fmaf(g[k][i], h[k][i], acc[k][i]);
        dh[i] = gate[k][i] * g[k][i];
      }
      ada_store4(dhp + 4 * (lane + 32 * k), dh);
    }
  }
  ada_block_column_sum<NV>(red, acc, p.partial + (b * p.splits + blockIdx.x) * C);
}

}  // namespace dmf
