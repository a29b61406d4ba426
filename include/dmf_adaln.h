/*
 * dmf_adaln.h - C ABI of the adaLN-Zero elementwise ops around the attention, with tangents.
 *
 * These are the memory-bound ops of the reference's DiTBlock / FinalLayer (models/layers.py:28-29
 * `modulate`, :195-201 `DiTBlock.forward`, :217-221 `FinalLayer.forward`):
 *
 *     y   = LayerNorm(x) * (1 + scale) + shift          (LayerNorm without affine, eps inside the sqrt)
 *     out = x + gate * h
 *
 * which PyTorch's forward-mode AD (torch.func.jvp, loss.py:149-166) runs as about twenty
 * elementwise / reduction kernels each.  Here one kernel computes the primal and the tangent
 *
 *     ty   = tLN * (1 + scale) + LN * tscale + tshift,  tLN = r (tx - mean(tx) - n mean(n tx)),
 *            n = (x - mean x) r,  r = rsqrt(var x + eps)
 *     tout = tx + tgate * h + gate * th
 *
 * and one kernel (plus a small fixed-order reduction) the primal backward; the tangent outputs
 * carry no gradient, as for the attention (the reference's losses detach what is computed from
 * the tangent, loss.py:171-173).
 *
 * Tensors: x, tx, y, ty, h, th, out, tout, dy, dx, dout, dh are (B, L, C) with element strides for
 * B and L and stride 1 for C; shift, scale, gate and their tangents / gradients are (B, C) with an
 * element stride for B (the chunks of the adaLN projection work in place).  C must be one of
 * 384, 768, 1024, 1152 (the reference's model widths) for the LayerNorm ops and the backward of
 * the gate op, and a multiple of 4 for the forward of the gate op.  Base pointers must be 16-byte
 * aligned and all strides multiples of 4 elements (rows are read as 4-element vectors).
 *
 * dtypes (enum dmf_adaln_dtype) are given per tensor class: "wide" for the residual stream
 * (x, tx, dx, out, tout, dout), "narrow" for what feeds or leaves a matmul (y, ty, dy, h, th, dh),
 * "mod" for shift / scale / gate and their tangents.  Supported (wide, narrow): (F32, F32),
 * (F32, BF16), (BF16, BF16); mod: F32 or BF16.  Gradients of shift / scale / gate are fp32.
 * Arithmetic is fp32 with one rounding of each result.
 *
 * Return values: the DMF_ATTN_* status codes of dmf_attn.h.  No call allocates or synchronises.
 */
#ifndef DMF_ADALN_H_
#define DMF_ADALN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum dmf_adaln_dtype {
  DMF_ADALN_BF16 = 0,
  DMF_ADALN_F32 = 2
};

/* a (B, L, C) tensor: element strides, channel stride 1 */
typedef struct dmf_rows {
  void* ptr;
  int64_t stride_b;
  int64_t stride_l;
} dmf_rows;

/* a (B, C) tensor: element stride of B, channel stride 1 */
typedef struct dmf_mod {
  void* ptr;
  int64_t stride_b;
} dmf_mod;

/*
 * y = LayerNorm(x) (1 + scale) + shift and, if tx.ptr is not NULL, its tangent ty.
 * tshift / tscale may have a NULL ptr (zero tangent) while tx is given.
 * Replaces modulate(norm(x), shift, scale): models/layers.py:196-197, 219.
 */
typedef struct dmf_ln_modulate_args {
  int32_t batch, seqlen, channels;
  int32_t wide_dtype, narrow_dtype, mod_dtype;
  float eps;                    /* the reference uses 1e-6 */
  int32_t reserved;
  dmf_rows x, tx;               /* wide, read only */
  dmf_mod shift, scale;         /* mod, read only */
  dmf_mod tshift, tscale;       /* mod, read only, optional */
  dmf_rows y, ty;               /* narrow, out */
  void* stream;                 /* cudaStream_t */
} dmf_ln_modulate_args;

int dmf_ln_modulate_fwd(const dmf_ln_modulate_args* args);

/*
 * Backward of y: with g = dy (1 + scale),
 *   dx = r (g - mean g - n mean(g n)),  dshift = sum_l dy,  dscale = sum_l dy n.
 * dshift, dscale: (B, C) fp32 contiguous, overwritten.  workspace: device memory of at least
 * dmf_adaln_bwd_workspace_bytes(batch, seqlen, channels) bytes (per-block partial sums, reduced in a
 * fixed order: bit-reproducible); its contents on entry do not matter.
 */
typedef struct dmf_ln_modulate_bwd_args {
  int32_t batch, seqlen, channels;
  int32_t wide_dtype, narrow_dtype, mod_dtype;
  float eps;
  int32_t reserved;
  dmf_rows dy;                  /* narrow, read only */
  dmf_rows x;                   /* wide, read only */
  dmf_mod scale;                /* mod, read only */
  dmf_rows dx;                  /* wide, out */
  float* dshift;                /* out (B, C) */
  float* dscale;                /* out (B, C) */
  void* workspace;
  size_t workspace_bytes;
  void* stream;
} dmf_ln_modulate_bwd_args;

size_t dmf_adaln_bwd_workspace_bytes(int32_t batch, int32_t seqlen, int32_t channels);
int dmf_ln_modulate_bwd(const dmf_ln_modulate_bwd_args* args);

/*
 * out = x + gate * h and, if tx.ptr is not NULL, tout = tx + tgate * h + gate * th
 * (tgate may have a NULL ptr: zero tangent).  Replaces x + gate * branch(x):
 * models/layers.py:196-197.
 */
typedef struct dmf_gate_residual_args {
  int32_t batch, seqlen, channels;
  int32_t wide_dtype, narrow_dtype, mod_dtype;
  dmf_rows x, tx;               /* wide, read only */
  dmf_rows h, th;               /* narrow, read only */
  dmf_mod gate, tgate;          /* mod, read only */
  dmf_rows out, tout;           /* wide, out */
  void* stream;
} dmf_gate_residual_args;

int dmf_gate_residual_fwd(const dmf_gate_residual_args* args);

/*
 * Backward of out: dx = dout (the caller passes the gradient through, no kernel),
 * dh = gate * dout, dgate = sum_l dout * h.  dgate: (B, C) fp32 contiguous, overwritten.
 * workspace as for dmf_ln_modulate_bwd.
 */
typedef struct dmf_gate_residual_bwd_args {
  int32_t batch, seqlen, channels;
  int32_t wide_dtype, narrow_dtype, mod_dtype;
  dmf_rows dout;                /* wide, read only */
  dmf_rows h;                   /* narrow, read only */
  dmf_mod gate;                 /* mod, read only */
  dmf_rows dh;                  /* narrow, out */
  float* dgate;                 /* out (B, C) */
  void* workspace;
  size_t workspace_bytes;
  void* stream;
} dmf_gate_residual_bwd_args;

int dmf_gate_residual_bwd(const dmf_gate_residual_bwd_args* args);

#ifdef __cplusplus
}
#endif

#endif /* DMF_ADALN_H_ */
