// C ABI of the adaLN-Zero elementwise ops (include/dmf_adaln.h): validation and launches.
#include <cuda_runtime.h>

#include <cstring>
#include <type_traits>

#include "adaln.cuh"
#include "dmf_adaln.h"
#include "dmf_attn.h"

namespace {

using namespace dmf;

int sm_count_of_current_device(int* sm_count) {
  static int cached_dev = -1, cached_sms = 0, cached_ok = 0;  // one device per process in practice
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return DMF_ATTN_ERR_DEVICE;
  if (dev != cached_dev) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return DMF_ATTN_ERR_DEVICE;
    cached_dev = dev;
    cached_sms = sms;
    cached_ok = (major == 10);
  }
  if (!cached_ok) return DMF_ATTN_ERR_DEVICE;
  *sm_count = cached_sms;
  return DMF_ATTN_OK;
}

int check_dtypes(int wide, int narrow, int mod) {
  const bool ok = (wide == DMF_ADALN_F32 && (narrow == DMF_ADALN_F32 || narrow == DMF_ADALN_BF16)) ||
                  (wide == DMF_ADALN_BF16 && narrow == DMF_ADALN_BF16);
  if (!ok) return DMF_ATTN_ERR_DTYPE;
  if (mod != DMF_ADALN_F32 && mod != DMF_ADALN_BF16) return DMF_ATTN_ERR_DTYPE;
  return DMF_ATTN_OK;
}

int check_rows(const dmf_rows& t, int /*dtype*/) {
  if (t.ptr == nullptr) return DMF_ATTN_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  if (t.stride_b < 0 || t.stride_l < 0) return DMF_ATTN_ERR_STRIDE;
  if ((t.stride_b % 4) != 0 || (t.stride_l % 4) != 0) return DMF_ATTN_ERR_STRIDE;  // rows are read as 4-element vectors
  return DMF_ATTN_OK;
}

int check_mod(const dmf_mod& t, int /*dtype*/) {
  if (t.ptr == nullptr) return DMF_ATTN_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  if (t.stride_b < 0 || (t.stride_b % 4) != 0) return DMF_ATTN_ERR_STRIDE;
  return DMF_ATTN_OK;
}

bool width_compiled(int channels) { return channels == 384 || channels == 768 || channels == 1024 || channels == 1152; }

int check_shape(int batch, int seqlen, int channels, bool need_compiled_width) {
  if (batch < 1 || seqlen < 1 || channels < 4) return DMF_ATTN_ERR_SHAPE;
  if (batch > 65535) return DMF_ATTN_ERR_SHAPE;  // batch is a grid y dimension in the backward kernels
  if (need_compiled_width ? !width_compiled(channels) : (channels % 4) != 0) return DMF_ATTN_ERR_SHAPE;
  return DMF_ATTN_OK;
}

int row_grid(int64_t rows, int sm_count) {
  const int64_t want = (rows + kAdaWarps - 1) / kAdaWarps;
  const int64_t cap = static_cast<int64_t>(sm_count) * 8;
  return static_cast<int>(want < cap ? want : cap);
}

// Rows of one block: 32 where that still gives every SM a few blocks, fewer for small problems (a training
// micro-batch of 32 x 256 tokens has 8192 rows).  A function of the shape only, so that the workspace size is too.
int rows_per_block(int batch, int seqlen) {
  constexpr int64_t kWantBlocks = 4 * 148;
  for (int rpb = 32; rpb > 8; rpb /= 2)
    if (static_cast<int64_t>(batch) * ((seqlen + rpb - 1) / rpb) >= kWantBlocks) return rpb;
  return 8;
}

int bwd_splits(int batch, int seqlen) {
  const int rpb = rows_per_block(batch, seqlen);
  return (seqlen + rpb - 1) / rpb;
}

size_t bwd_workspace_bytes(int batch, int seqlen, int channels) {
  if (batch < 1 || seqlen < 1 || channels < 1) return 0;
  return static_cast<size_t>(batch) * bwd_splits(batch, seqlen) * 2 * channels * sizeof(float);
}

// (wide, narrow) -> types; NV -> the compiled widths
template <typename F>
int with_types(int wide, int narrow, F&& f) {
  if (wide == DMF_ADALN_F32 && narrow == DMF_ADALN_F32) return f(float{}, float{});
  if (wide == DMF_ADALN_F32 && narrow == DMF_ADALN_BF16) return f(float{}, __nv_bfloat16{});
  return f(__nv_bfloat16{}, __nv_bfloat16{});
}

template <typename F>
int with_width(int channels, F&& f) {
  switch (channels) {
    case 384: return f(std::integral_constant<int, 3>{});
    case 768: return f(std::integral_constant<int, 6>{});
    case 1024: return f(std::integral_constant<int, 8>{});
    case 1152: return f(std::integral_constant<int, 9>{});
    default: return DMF_ATTN_ERR_SHAPE;
  }
}

int launched() { return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH; }

int run_ln_modulate_fwd(const dmf_ln_modulate_args* a) {
  if (a == nullptr) return DMF_ATTN_ERR_NULL;
  int st;
  if ((st = check_dtypes(a->wide_dtype, a->narrow_dtype, a->mod_dtype)) != DMF_ATTN_OK) return st;
  if ((st = check_shape(a->batch, a->seqlen, a->channels, true)) != DMF_ATTN_OK) return st;
  const bool dual = a->tx.ptr != nullptr;
  const bool tmod = dual && (a->tshift.ptr != nullptr || a->tscale.ptr != nullptr);
  if ((st = check_rows(a->x, a->wide_dtype)) != DMF_ATTN_OK || (st = check_rows(a->y, a->narrow_dtype)) != DMF_ATTN_OK ||
      (st = check_mod(a->shift, a->mod_dtype)) != DMF_ATTN_OK || (st = check_mod(a->scale, a->mod_dtype)) != DMF_ATTN_OK)
    return st;
  if (dual && ((st = check_rows(a->tx, a->wide_dtype)) != DMF_ATTN_OK || (st = check_rows(a->ty, a->narrow_dtype)) != DMF_ATTN_OK))
    return st;
  if (tmod && ((st = check_mod(a->tshift, a->mod_dtype)) != DMF_ATTN_OK || (st = check_mod(a->tscale, a->mod_dtype)) != DMF_ATTN_OK))
    return st;  // the two tangents come together
  int sms = 0;
  if ((st = sm_count_of_current_device(&sms)) != DMF_ATTN_OK) return st;
  AdaParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = a->x.ptr; p.x_sb = a->x.stride_b; p.x_sl = a->x.stride_l;
  p.y = a->y.ptr; p.y_sb = a->y.stride_b; p.y_sl = a->y.stride_l;
  p.shift = a->shift.ptr; p.shift_sb = a->shift.stride_b;
  p.scale = a->scale.ptr; p.scale_sb = a->scale.stride_b;
  if (dual) {
    p.tx = a->tx.ptr; p.tx_sb = a->tx.stride_b; p.tx_sl = a->tx.stride_l;
    p.ty = a->ty.ptr; p.ty_sb = a->ty.stride_b; p.ty_sl = a->ty.stride_l;
  }
  if (tmod) {
    p.tshift = a->tshift.ptr; p.tshift_sb = a->tshift.stride_b;
    p.tscale = a->tscale.ptr; p.tscale_sb = a->tscale.stride_b;
  }
  p.batch = a->batch; p.seqlen = a->seqlen; p.channels = a->channels;
  p.mod_f32 = a->mod_dtype == DMF_ADALN_F32;
  p.eps = a->eps;
  p.rows_per_block = rows_per_block(a->batch, a->seqlen);
  p.splits = bwd_splits(a->batch, a->seqlen);
  const dim3 grid(p.splits, a->batch);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  return with_types(a->wide_dtype, a->narrow_dtype, [&](auto tw, auto tn) {
    using TW = decltype(tw);
    using TN = decltype(tn);
    return with_width(a->channels, [&](auto nv) {
      constexpr int NV = decltype(nv)::value;
      if (dual) ln_modulate_fwd_kernel<TW, TN, NV, true><<<grid, kAdaThreads, 0, stream>>>(p);
      else ln_modulate_fwd_kernel<TW, TN, NV, false><<<grid, kAdaThreads, 0, stream>>>(p);
      return launched();
    });
  });
}

int run_ln_modulate_bwd(const dmf_ln_modulate_bwd_args* a) {
  if (a == nullptr || a->dshift == nullptr || a->dscale == nullptr) return DMF_ATTN_ERR_NULL;
  int st;
  if ((st = check_dtypes(a->wide_dtype, a->narrow_dtype, a->mod_dtype)) != DMF_ATTN_OK) return st;
  if ((st = check_shape(a->batch, a->seqlen, a->channels, true)) != DMF_ATTN_OK) return st;
  if ((st = check_rows(a->dy, a->narrow_dtype)) != DMF_ATTN_OK || (st = check_rows(a->x, a->wide_dtype)) != DMF_ATTN_OK ||
      (st = check_rows(a->dx, a->wide_dtype)) != DMF_ATTN_OK || (st = check_mod(a->scale, a->mod_dtype)) != DMF_ATTN_OK)
    return st;
  if (a->workspace == nullptr || a->workspace_bytes < bwd_workspace_bytes(a->batch, a->seqlen, a->channels))
    return DMF_ATTN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  int sms = 0;
  if ((st = sm_count_of_current_device(&sms)) != DMF_ATTN_OK) return st;
  AdaParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = a->x.ptr; p.x_sb = a->x.stride_b; p.x_sl = a->x.stride_l;
  p.dy = a->dy.ptr; p.dy_sb = a->dy.stride_b; p.dy_sl = a->dy.stride_l;
  p.dx = a->dx.ptr; p.dx_sb = a->dx.stride_b; p.dx_sl = a->dx.stride_l;
  p.scale = a->scale.ptr; p.scale_sb = a->scale.stride_b;
  p.partial = static_cast<float*>(a->workspace);
  p.batch = a->batch; p.seqlen = a->seqlen; p.channels = a->channels;
  p.mod_f32 = a->mod_dtype == DMF_ADALN_F32;
  p.rows_per_block = rows_per_block(a->batch, a->seqlen);
  p.splits = bwd_splits(a->batch, a->seqlen);
  p.eps = a->eps;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const dim3 grid(p.splits, a->batch);
  st = with_types(a->wide_dtype, a->narrow_dtype, [&](auto tw, auto tn) {
    using TW = decltype(tw);
    using TN = decltype(tn);
    return with_width(a->channels, [&](auto nv) {
      constexpr int NV = decltype(nv)::value;
      constexpr int kSmem = (1 + 2 * kAdaWarps) * NV * 128 * static_cast<int>(sizeof(float));
      static bool configured = false;  // per instantiation
      if (!configured) {
        if (cudaFuncSetAttribute(ln_modulate_bwd_kernel<TW, TN, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmem) != cudaSuccess)
          return static_cast<int>(DMF_ATTN_ERR_LAUNCH);
        configured = true;
      }
      ln_modulate_bwd_kernel<TW, TN, NV><<<grid, kAdaThreads, kSmem, stream>>>(p);
      return launched();
    });
  });
  if (st != DMF_ATTN_OK) return st;
  const dim3 rgrid((a->channels + kAdaThreads - 1) / kAdaThreads, a->batch, 2);
  ada_partial_reduce_kernel<<<rgrid, kAdaThreads, 0, stream>>>(p.partial, a->dshift, a->dscale, p.splits, a->channels, 2);
  return launched();
}

int run_gate_residual_fwd(const dmf_gate_residual_args* a) {
  if (a == nullptr) return DMF_ATTN_ERR_NULL;
  int st;
  if ((st = check_dtypes(a->wide_dtype, a->narrow_dtype, a->mod_dtype)) != DMF_ATTN_OK) return st;
  if ((st = check_shape(a->batch, a->seqlen, a->channels, false)) != DMF_ATTN_OK) return st;
  const bool dual = a->tx.ptr != nullptr;
  if ((st = check_rows(a->x, a->wide_dtype)) != DMF_ATTN_OK || (st = check_rows(a->h, a->narrow_dtype)) != DMF_ATTN_OK ||
      (st = check_rows(a->out, a->wide_dtype)) != DMF_ATTN_OK || (st = check_mod(a->gate, a->mod_dtype)) != DMF_ATTN_OK)
    return st;
  if (dual && ((st = check_rows(a->tx, a->wide_dtype)) != DMF_ATTN_OK || (st = check_rows(a->th, a->narrow_dtype)) != DMF_ATTN_OK ||
               (st = check_rows(a->tout, a->wide_dtype)) != DMF_ATTN_OK))
    return st;
  const bool tmod = dual && a->tgate.ptr != nullptr;
  if (tmod && (st = check_mod(a->tgate, a->mod_dtype)) != DMF_ATTN_OK) return st;
  int sms = 0;
  if ((st = sm_count_of_current_device(&sms)) != DMF_ATTN_OK) return st;
  AdaParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = a->x.ptr; p.x_sb = a->x.stride_b; p.x_sl = a->x.stride_l;
  p.h = a->h.ptr; p.h_sb = a->h.stride_b; p.h_sl = a->h.stride_l;
  p.y = a->out.ptr; p.y_sb = a->out.stride_b; p.y_sl = a->out.stride_l;
  p.gate = a->gate.ptr; p.gate_sb = a->gate.stride_b;
  if (dual) {
    p.tx = a->tx.ptr; p.tx_sb = a->tx.stride_b; p.tx_sl = a->tx.stride_l;
    p.th = a->th.ptr; p.th_sb = a->th.stride_b; p.th_sl = a->th.stride_l;
    p.ty = a->tout.ptr; p.ty_sb = a->tout.stride_b; p.ty_sl = a->tout.stride_l;
  }
  if (tmod) { p.tgate = a->tgate.ptr; p.tgate_sb = a->tgate.stride_b; }
  p.batch = a->batch; p.seqlen = a->seqlen; p.channels = a->channels;
  p.mod_f32 = a->mod_dtype == DMF_ADALN_F32;
  const int grid = row_grid(static_cast<int64_t>(a->batch) * a->seqlen, sms);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  return with_types(a->wide_dtype, a->narrow_dtype, [&](auto tw, auto tn) {
    using TW = decltype(tw);
    using TN = decltype(tn);
    if (dual) gate_residual_fwd_kernel<TW, TN, true><<<grid, kAdaThreads, 0, stream>>>(p);
    else gate_residual_fwd_kernel<TW, TN, false><<<grid, kAdaThreads, 0, stream>>>(p);
    return launched();
  });
}

int run_gate_residual_bwd(const dmf_gate_residual_bwd_args* a) {
  if (a == nullptr || a->dgate == nullptr) return DMF_ATTN_ERR_NULL;
  int st;
  if ((st = check_dtypes(a->wide_dtype, a->narrow_dtype, a->mod_dtype)) != DMF_ATTN_OK) return st;
  if ((st = check_shape(a->batch, a->seqlen, a->channels, true)) != DMF_ATTN_OK) return st;
  if ((st = check_rows(a->dout, a->wide_dtype)) != DMF_ATTN_OK || (st = check_rows(a->h, a->narrow_dtype)) != DMF_ATTN_OK ||
      (st = check_rows(a->dh, a->narrow_dtype)) != DMF_ATTN_OK || (st = check_mod(a->gate, a->mod_dtype)) != DMF_ATTN_OK)
    return st;
  if (a->workspace == nullptr || a->workspace_bytes < bwd_workspace_bytes(a->batch, a->seqlen, a->channels))
    return DMF_ATTN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  int sms = 0;
  if ((st = sm_count_of_current_device(&sms)) != DMF_ATTN_OK) return st;
  AdaParams p;
  std::memset(&p, 0, sizeof(p));
  p.dy = a->dout.ptr; p.dy_sb = a->dout.stride_b; p.dy_sl = a->dout.stride_l;
  p.h = a->h.ptr; p.h_sb = a->h.stride_b; p.h_sl = a->h.stride_l;
  p.dx = a->dh.ptr; p.dx_sb = a->dh.stride_b; p.dx_sl = a->dh.stride_l;
  p.gate = a->gate.ptr; p.gate_sb = a->gate.stride_b;
  p.partial = static_cast<float*>(a->workspace);
  p.batch = a->batch; p.seqlen = a->seqlen; p.channels = a->channels;
  p.mod_f32 = a->mod_dtype == DMF_ADALN_F32;
  p.rows_per_block = rows_per_block(a->batch, a->seqlen);
  p.splits = bwd_splits(a->batch, a->seqlen);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const dim3 grid(p.splits, a->batch);
  st = with_types(a->wide_dtype, a->narrow_dtype, [&](auto tw, auto tn) {
    using TW = decltype(tw);
    using TN = decltype(tn);
    return with_width(a->channels, [&](auto nv) {
      gate_residual_bwd_kernel<TW, TN, decltype(nv)::value><<<grid, kAdaThreads, 0, stream>>>(p);
      return launched();
    });
  });
  if (st != DMF_ATTN_OK) return st;
  const dim3 rgrid((a->channels + kAdaThreads - 1) / kAdaThreads, a->batch, 1);
  ada_partial_reduce_kernel<<<rgrid, kAdaThreads, 0, stream>>>(p.partial, a->dgate, a->dgate, p.splits, a->channels, 1);
  return launched();
}

}  // namespace

#define DMF_API __attribute__((visibility("default")))

extern "C" {

DMF_API int dmf_ln_modulate_fwd(const dmf_ln_modulate_args* args) { return run_ln_modulate_fwd(args); }
DMF_API size_t dmf_adaln_bwd_workspace_bytes(int32_t batch, int32_t seqlen, int32_t channels) {
  return bwd_workspace_bytes(batch, seqlen, channels);
}
DMF_API int dmf_ln_modulate_bwd(const dmf_ln_modulate_bwd_args* args) { return run_ln_modulate_bwd(args); }
DMF_API int dmf_gate_residual_fwd(const dmf_gate_residual_args* args) { return run_gate_residual_fwd(args); }
DMF_API int dmf_gate_residual_bwd(const dmf_gate_residual_bwd_args* args) { return run_gate_residual_bwd(args); }

}  // extern "C"
