// Per-head RMS normalisation of q / k with its tangent, and its primal backward.
//
//   r  = rsqrt(mean_d(x^2) + eps)            y  = x * r * w
//   tr = -r^3 * mean_d(x * tx)               ty = (tx * r + x * tr) * w
//   backward of y (the tangent output carries no gradient, like the attention's):
//   g = dy * w      dx = r * g - x * r^3 * mean_d(x * g)      dw_d = sum_rows dy_d * x_d * r
//
// These are the q_norm / k_norm of the reference's Attention block (models/layers.py:33-42, 148),
// which PyTorch's forward-mode AD runs as a dozen elementwise kernels over (B, L, H, D) tensors.
// Here each row is read once and written once: the kernels are bound by HBM bandwidth.
//
// Layout: tensors are (B, L, H, D) with element strides for B, L, H and stride 1 for D (the
// strided views of a packed qkv projection work in place); a row is one (b, l, h).  A row of
// head_dim = 8 C elements is handled by C neighbouring lanes, one 16-byte chunk (8 elements) per
// lane, 32 / C whole rows per warp (3 rows on 27 lanes at head_dim 72); the row reductions are
// shuffles inside the C lanes.  The kernels are compiled per C: with generic 16-lane rows 7 of 16
// lanes idle at head_dim 72 and the kernel is bound by instruction issue at half the HBM bandwidth.
// Arithmetic is fp32 with one rounding to the 16-bit output type (the reference rounds after every
// step).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace dmf {

struct RmsParams {
  const void* x;
  const void* tx;     // nullptr: no tangent
  const void* dy;     // backward only
  const float* w;     // (D) fp32
  void* y;
  void* ty;
  void* dx;           // backward only
  float* dw_partial;  // backward only: (gridDim.x, D) fp32
  int64_t x_sb, x_sl, x_sh;
  int64_t tx_sb, tx_sl, tx_sh;
  int64_t dy_sb, dy_sl, dy_sh;
  int64_t y_sb, y_sl, y_sh;
  int64_t ty_sb, ty_sl, ty_sh;
  int64_t dx_sb, dx_sl, dx_sh;
  int batch, seqlen, heads, head_dim;
  int64_t rows;
  float eps;
};

constexpr int kRmsThreads = 256;
constexpr int kRmsWarps = kRmsThreads / 32;
// Rows each thread keeps in flight (all their loads are issued before the first use): enough
// 16-byte loads per thread to cover the HBM latency at the occupancy the registers allow.
#ifndef DMF_RMS_UNROLL_DUAL
#define DMF_RMS_UNROLL_DUAL 2
#endif
#ifndef DMF_RMS_UNROLL_PLAIN
#define DMF_RMS_UNROLL_PLAIN 4
#endif
#ifndef DMF_RMS_UNROLL_BWD
#define DMF_RMS_UNROLL_BWD 2
#endif
__host__ __device__ constexpr int rms_unroll_fwd(bool dual) { return dual ? DMF_RMS_UNROLL_DUAL : DMF_RMS_UNROLL_PLAIN; }
constexpr int kRmsUnrollBwd = DMF_RMS_UNROLL_BWD;
// A row of C 16-byte chunks takes C neighbouring lanes; a warp holds 32 / C whole rows.
__host__ __device__ constexpr int rms_rows_per_warp(int chunks) { return 32 / chunks; }
__host__ __device__ constexpr int rms_rows_per_block(int chunks, int unroll) {
  return rms_rows_per_warp(chunks) * kRmsWarps * unroll;
}

// Sum over the C lanes of a row, returned to all of them.  `idx` is the lane's place in its row.
// Lanes outside a row's group may feed garbage into lanes whose partial sums are never read.
template <int C>
__device__ __forceinline__ float rms_group_sum(float v, int idx, int lane) {
  constexpr int P = C >= 16 ? 16 : C >= 8 ? 8 : C >= 4 ? 4 : C >= 2 ? 2 : 1;  // largest power of two <= C
  if constexpr (P == C) {
#pragma unroll
    for (int d = P / 2; d >= 1; d /= 2) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
  } else {
    const float t = __shfl_down_sync(0xffffffffu, v, P);
    if (idx < C - P) v += t;  // fold the lanes beyond the power of two onto the first ones
#pragma unroll
    for (int d = P / 2; d >= 1; d /= 2) v += __shfl_down_sync(0xffffffffu, v, d);
    return __shfl_sync(0xffffffffu, v, lane - idx);
  }
}

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {  // read-once data: no L1 allocation
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <typename T>
__device__ __forceinline__ void rms_unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = unpack2<T>(u[i]);
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}

template <typename T>
__device__ __forceinline__ void rms_store8(T* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(Pack2<T>::pack(f[0], f[1]), Pack2<T>::pack(f[2], f[3]),
                                            Pack2<T>::pack(f[4], f[5]), Pack2<T>::pack(f[6], f[7]));
}

// the weight as the reference uses it: cast to the tensor's 16-bit type first
template <typename T>
__device__ __forceinline__ float rms_round(float v) {
  const float2 a = unpack2<T>(Pack2<T>::pack(v, 0.f));
  return a.x;
}

// A row number as (b, l, h), stepped without divisions: the two divisions per row of a plain
// decomposition cost more issue slots than the arithmetic of the row itself.
struct RmsPos {
  uint32_t b, l, h;
  __device__ __forceinline__ RmsPos(int64_t row, uint32_t seqlen, uint32_t heads) {
    const uint32_t lh = seqlen * heads, r = static_cast<uint32_t>(row);
    b = r / lh;
    const uint32_t rem = r - b * lh;
    l = rem / heads;
    h = rem - l * heads;
  }
  // add a step (given as a position with l < seqlen, h < heads)
  __device__ __forceinline__ void advance(const RmsPos& d, uint32_t seqlen, uint32_t heads) {
    h += d.h;
    if (h >= heads) { h -= heads; ++l; }
    l += d.l;
    if (l >= seqlen) { l -= seqlen; ++b; }
    b += d.b;
  }
  // Off = int32_t where the host found every element offset of the launch below 2^31 (one 32-bit multiply-add per
  // term instead of a 64-bit one: the kernels are bound by instruction issue), else int64_t
  template <typename Off>
  __device__ __forceinline__ Off at(int64_t sb, int64_t sl, int64_t sh) const {
    return static_cast<Off>(b) * static_cast<Off>(sb) + static_cast<Off>(l) * static_cast<Off>(sl) +
           static_cast<Off>(h) * static_cast<Off>(sh);
  }
};

// head_dim = 8 * C.  Grid-stride over slices of rms_rows_per_block(C) rows.
template <typename T, int C, bool kDual, typename Off>
__global__ void __launch_bounds__(kRmsThreads) rmsnorm_fwd_kernel(const RmsParams p) {
  constexpr int R = rms_rows_per_warp(C);
  constexpr int kSlice = R * kRmsWarps;  // rows of one unroll step of the block
  constexpr int kRmsUnroll = rms_unroll_fwd(kDual);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / C, idx = lane - grp * C;
  const int col = idx * 8;
  const bool active = grp < R;
  float w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = rms_round<T>(p.w[col + i]);
  const float inv_d = 1.f / static_cast<float>(8 * C);
  const uint32_t seqlen = p.seqlen, heads = p.heads;
  const int64_t rows = p.rows;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * (kSlice * kRmsUnroll);
  // the loop bound is the warp's first row: the same for all its lanes (the shuffles name all 32)
  int64_t wrow = static_cast<int64_t>(blockIdx.x) * (kSlice * kRmsUnroll) + warp * R;
  RmsPos pos(wrow + grp, seqlen, heads);
  const RmsPos step_slice(kSlice, seqlen, heads);
  const RmsPos step_rest(stride - kSlice * kRmsUnroll, seqlen, heads);
  for (; wrow < rows; wrow += stride) {
    uint4 xr[kRmsUnroll], tr_[kRmsUnroll];
    Off oy[kRmsUnroll], oty[kRmsUnroll];
    bool on[kRmsUnroll];
#pragma unroll
    for (int u = 0; u < kRmsUnroll; ++u) {
      on[u] = active && (wrow + u * kSlice + grp) < rows;
      xr[u] = make_uint4(0u, 0u, 0u, 0u);
      tr_[u] = make_uint4(0u, 0u, 0u, 0u);
      oy[u] = 0;
      oty[u] = 0;
      if (on[u]) {
        xr[u] = ld_nc_v4(reinterpret_cast<const T*>(p.x) + pos.at<Off>(p.x_sb, p.x_sl, p.x_sh) + col);
        if constexpr (kDual) tr_[u] = ld_nc_v4(reinterpret_cast<const T*>(p.tx) + pos.at<Off>(p.tx_sb, p.tx_sl, p.tx_sh) + col);
        oy[u] = pos.at<Off>(p.y_sb, p.y_sl, p.y_sh) + col;
        if constexpr (kDual) oty[u] = pos.at<Off>(p.ty_sb, p.ty_sl, p.ty_sh) + col;
      }
      pos.advance(step_slice, seqlen, heads);
    }
    pos.advance(step_rest, seqlen, heads);
#pragma unroll
    for (int u = 0; u < kRmsUnroll; ++u) {
      // (fp32 pairs - two elements per instruction - were tried here: slower at the same register count)
      float x[8], tx[8];
      rms_unpack8<T>(xr[u], x);
      if constexpr (kDual) rms_unpack8<T>(tr_[u], tx);
      float ss = 0.f, dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss = fmaf(x[i], x[i], ss);
        if constexpr (kDual) dot = fmaf(x[i], tx[i], dot);
      }
      ss = rms_group_sum<C>(ss, idx, lane);
      const float r = rsqrtf(ss * inv_d + p.eps);
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = x[i] * r * w[i];
      if (on[u]) rms_store8(reinterpret_cast<T*>(p.y) + oy[u], y);
      if constexpr (kDual) {
        dot = rms_group_sum<C>(dot, idx, lane);
        const float tr = -r * r * r * dot * inv_d;
        float ty[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) ty[i] = fmaf(tx[i], r, x[i] * tr) * w[i];
        if (on[u]) rms_store8(reinterpret_cast<T*>(p.ty) + oty[u], ty);
      }
    }
  }
}

template <typename T, int C, typename Off>
__global__ void __launch_bounds__(kRmsThreads) rmsnorm_bwd_kernel(const RmsParams p) {
  constexpr int R = rms_rows_per_warp(C);
  constexpr int kSlice = R * kRmsWarps;
  constexpr int kRmsUnroll = kRmsUnrollBwd;
  __shared__ float red[kSlice][8 * C + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / C, idx = lane - grp * C;
  const int col = idx * 8;
  const bool active = grp < R;
  float w[8], dw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = rms_round<T>(p.w[col + i]);
    dw[i] = 0.f;
  }
  const float inv_d = 1.f / static_cast<float>(8 * C);
  const uint32_t seqlen = p.seqlen, heads = p.heads;
  const int64_t rows = p.rows;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * (kSlice * kRmsUnroll);
  int64_t wrow = static_cast<int64_t>(blockIdx.x) * (kSlice * kRmsUnroll) + warp * R;
  RmsPos pos(wrow + grp, seqlen, heads);
  const RmsPos step_slice(kSlice, seqlen, heads);
  const RmsPos step_rest(stride - kSlice * kRmsUnroll, seqlen, heads);
  for (; wrow < rows; wrow += stride) {
    uint4 xr[kRmsUnroll], gr[kRmsUnroll];
    Off od[kRmsUnroll];
    bool on[kRmsUnroll];
#pragma unroll
    for (int u = 0; u < kRmsUnroll; ++u) {
      on[u] = active && (wrow + u * kSlice + grp) < rows;
      xr[u] = make_uint4(0u, 0u, 0u, 0u);
      gr[u] = make_uint4(0u, 0u, 0u, 0u);
      od[u] = 0;
      if (on[u]) {
        xr[u] = ld_nc_v4(reinterpret_cast<const T*>(p.x) + pos.at<Off>(p.x_sb, p.x_sl, p.x_sh) + col);
        gr[u] = ld_nc_v4(reinterpret_cast<const T*>(p.dy) + pos.at<Off>(p.dy_sb, p.dy_sl, p.dy_sh) + col);
        od[u] = pos.at<Off>(p.dx_sb, p.dx_sl, p.dx_sh) + col;
      }
      pos.advance(step_slice, seqlen, heads);
    }
    pos.advance(step_rest, seqlen, heads);
#pragma unroll
    for (int u = 0; u < kRmsUnroll; ++u) {
      float x[8], dy[8];
      rms_unpack8<T>(xr[u], x);
      rms_unpack8<T>(gr[u], dy);
      float ss = 0.f, xg = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dy[i] *= w[i];  // g = dy * w
        ss = fmaf(x[i], x[i], ss);
        xg = fmaf(x[i], dy[i], xg);
      }
      ss = rms_group_sum<C>(ss, idx, lane);
      xg = rms_group_sum<C>(xg, idx, lane);
      const float r = rsqrtf(ss * inv_d + p.eps);
      const float c = r * r * r * xg * inv_d;
      float dx[8], raw[8];
      rms_unpack8<T>(gr[u], raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dx[i] = fmaf(r, dy[i], -x[i] * c);
        dw[i] = fmaf(raw[i], x[i] * r, dw[i]);  // rows that are off hold zeros
      }
      if (on[u]) rms_store8(reinterpret_cast<T*>(p.dx) + od[u], dx);
    }
  }
  // this block's share of dw: sum over the rows its warps hold side by side
  if (active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[warp * R + grp][col + i] = dw[i];
  }
  __syncthreads();
  if (threadIdx.x < 8 * C) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kSlice; ++k) s += red[k][threadIdx.x];
    p.dw_partial[static_cast<int64_t>(blockIdx.x) * (8 * C) + threadIdx.x] = s;
  }
}

// dw[d] = sum over the blocks' partial sums, in a fixed order (bit-reproducible).  One block of
// 32 x 32 threads per 32 columns: thread (g, c) sums the partials g, g + 32, ... of column c, then
// the 32 sums of a column are added in order.
__global__ void __launch_bounds__(1024) rmsnorm_dw_reduce_kernel(const float* partial, float* dw, int blocks, int head_dim) {
  __shared__ float red[32][33];
  const int c = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + c;
  float s = 0.f;
  if (d < head_dim)
    for (int k = g; k < blocks; k += 32) s += partial[static_cast<int64_t>(k) * head_dim + d];
  red[g][c] = s;
  __syncthreads();
  if (g == 0 && d < head_dim) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += red[k][c];
    dw[d] = t;
  }
}

}  // namespace dmf
