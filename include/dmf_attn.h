/*
 * dmf_attn.h - C ABI of the B200 (sm_100a) attention kernels behind
 * Decoupled MeanFlow's flash_attn_func.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, never
 * allocates or frees device memory, never keeps a pointer after it returns and
 * launches asynchronously on the CUDA stream it is given.  All tensors use the
 * reference layout (B, L, H, D) with an arbitrary element stride for B, L and H
 * and stride 1 for D, so the strided q/k/v views of a packed qkv projection are
 * consumed without a copy.
 *
 * Return value: 0 (DMF_ATTN_OK) or one of the DMF_ATTN_ERR_* codes below; the
 * text for a code comes from dmf_attn_status_string().  There is no CPU path:
 * on a machine without an sm_100 device the compute entry points return
 * DMF_ATTN_ERR_DEVICE.
 */
#ifndef DMF_ATTN_H_
#define DMF_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DMF_ATTN_ABI_VERSION 1

enum dmf_attn_dtype {
  DMF_ATTN_BF16 = 0,
  DMF_ATTN_FP16 = 1
};

enum dmf_attn_status {
  DMF_ATTN_OK = 0,
  DMF_ATTN_ERR_NULL = 1,        /* a required pointer is NULL                                  */
  DMF_ATTN_ERR_DTYPE = 2,       /* dtype is not bf16 / fp16                                    */
  DMF_ATTN_ERR_HEAD_DIM = 3,    /* head_dim not in {64, 72, 80, 88, 96, 104, ..., 128}         */
  DMF_ATTN_ERR_SEQLEN = 4,      /* seqlen_q or seqlen_kv is not a positive multiple of 128     */
  DMF_ATTN_ERR_SHAPE = 5,       /* batch or heads < 1, or a size overflows                     */
  DMF_ATTN_ERR_STRIDE = 6,      /* a stride (in bytes) is not a multiple of 16                 */
  DMF_ATTN_ERR_ALIGN = 7,       /* a base pointer is not 16-byte aligned                       */
  DMF_ATTN_ERR_DEVICE = 8,      /* no CUDA device, or the device is not compute capability 10.x */
  DMF_ATTN_ERR_TENSOR_MAP = 9,  /* the driver rejected a TMA tensor map                        */
  DMF_ATTN_ERR_LAUNCH = 10,     /* the kernel launch failed (see cudaGetLastError)             */
  DMF_ATTN_ERR_WORKSPACE = 11,  /* workspace missing or too small                              */
  DMF_ATTN_ERR_TIMEOUT = 12,    /* a device-side wait ran out (reported by dmf_attn_check_status_word) */
  DMF_ATTN_ERR_TOO_LARGE = 13   /* problem exceeds the built-in scratch of dmf_attn_bwd_static         */
};

/* One (B, L, H, D) tensor: base pointer and element strides; the D stride is 1. */
typedef struct dmf_attn_tensor {
  void* ptr;
  int64_t stride_b;
  int64_t stride_l;
  int64_t stride_h;
} dmf_attn_tensor;

/*
 * Arguments of the forward kernels.
 *
 * status_word (optional, may be NULL): one int32 in device memory, zeroed by
 * the caller.  Every device-side wait has an upper limit; a kernel whose wait
 * runs out writes a non-zero code there, releases what it holds and returns
 * normally, so the CUDA context stays usable.  Read it back with
 * dmf_attn_check_status_word().
 */
typedef struct dmf_attn_fwd_args {
  int32_t batch;
  int32_t seqlen_q;
  int32_t seqlen_kv;
  int32_t heads;
  int32_t head_dim;
  int32_t dtype;            /* enum dmf_attn_dtype                                   */
  float softmax_scale;      /* applied to Q K^T; the reference default is D^-0.5     */
  int32_t reserved;
  dmf_attn_tensor q, k, v;  /* primals, read only                                    */
  dmf_attn_tensor tq, tk, tv; /* tangents, read only (ignored by dmf_attn_fwd)       */
  dmf_attn_tensor o;        /* out: softmax(s Q K^T) V                               */
  dmf_attn_tensor to;       /* out: tangent of o (ignored by dmf_attn_fwd)           */
  float* lse;               /* out: (B, H, Lq) contiguous fp32, natural-log LSE of s Q K^T */
  int32_t* status_word;     /* optional device int32, see above                      */
  void* stream;             /* cudaStream_t                                          */
} dmf_attn_fwd_args;

/*
 * Arguments of the primal backward.  grads of lse and of the tangent output are
 * not inputs: the reference drops them (stop-gradient on the tangent).
 * workspace: device memory, 16-byte aligned, of at least 8 * batch * heads *
 * seqlen_q bytes (two fp32 rows per query); its contents on entry do not matter.
 * dmf_attn_bwd_workspace_bytes() reports what the fastest kernel for the problem
 * wants: for sequences of more than two tiles at head_dim <= 80 that is room for
 * an fp32 dQ accumulator (4 * batch * heads * seqlen_q * head_dim bytes) behind
 * the two rows, with the workspace 256-byte aligned.  That kernel visits every
 * 128 x 128 block of scores once and sums a query tile's dQ over the key tiles
 * with fp32 atomics, so the last bits of dq depend on the order the blocks
 * finished in (dk and dv do not; the FlashAttention backward the reference
 * calls behaves the same way with deterministic=False).  With a workspace
 * smaller than reported, or DMF_ATTN_BWD_STREAM=0 in the environment, the call
 * runs the two-launch kernels, whose results are reproducible bit for bit.
 */
typedef struct dmf_attn_bwd_args {
  int32_t batch;
  int32_t seqlen_q;
  int32_t seqlen_kv;
  int32_t heads;
  int32_t head_dim;
  int32_t dtype;
  float softmax_scale;
  int32_t reserved;
  dmf_attn_tensor dout;     /* grad of o, read only                                  */
  dmf_attn_tensor q, k, v;  /* saved primals                                         */
  dmf_attn_tensor o;        /* saved output                                          */
  const float* lse;         /* saved (B, H, Lq) fp32 LSE                             */
  dmf_attn_tensor dq, dk, dv; /* out                                                 */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status_word;
  void* stream;
} dmf_attn_bwd_args;

/* ABI version of the loaded library (DMF_ATTN_ABI_VERSION it was built with). */
int dmf_attn_abi_version(void);

/* Static, NUL-terminated description of a status code. */
const char* dmf_attn_status_string(int status);

/*
 * Fused forward + tangent ("dual" forward): o, to and lse from q, k, v and
 * their tangents in one online-softmax pass.
 * Replaces the Triton launches _attn_fwd_dual / _attn_fwd_dual_split made by
 * FlashAttnFunc.forward (models/flash_attention_2_jvp.py:186-230,
 * models/flash_attention_3_jvp.py:171-215; kernels models/triton_utils.py:258-500).
 */
int dmf_attn_fwd_dual(const dmf_attn_fwd_args* args);

/*
 * Plain forward: o and lse from q, k, v (no dropout, non-causal, no window).
 * Replaces flash_attn_2_cuda.fwd (models/flash_attention_2_jvp.py:47-61) and
 * torch.ops.flash_attn_3.fwd (models/flash_attention_3_jvp.py:72-107) as called
 * from the non-dual branch of FlashAttnFunc.forward
 * (models/flash_attention_2_jvp.py:231-243).
 */
int dmf_attn_fwd(const dmf_attn_fwd_args* args);

/*
 * Primal backward: dq, dk, dv from dout, q, k, v, o, lse.
 * Replaces flash_attn_2_cuda.bwd (models/flash_attention_2_jvp.py:119-139) and
 * torch.ops.flash_attn_3.bwd (models/flash_attention_3_jvp.py:136-159) as called
 * from FlashAttnFunc.backward (models/flash_attention_2_jvp.py:260-276).
 */
int dmf_attn_bwd(const dmf_attn_bwd_args* args);

/* Bytes of workspace the fastest kernel of dmf_attn_bwd wants for this problem size (0 on bad sizes);
 * see dmf_attn_bwd_args for the minimum a call is valid with. */
size_t dmf_attn_bwd_workspace_bytes(int32_t batch, int32_t seqlen_q, int32_t seqlen_kv,
                                    int32_t heads, int32_t head_dim);

/*
 * Primal backward for callers that have no way to hand over scratch memory.
 * (No counterpart in the reference: its backward lets the FlashAttention
 * library allocate whatever it needs through torch.)
 *
 * Some hosts of this library cannot allocate device memory at the point where
 * they need a backward pass: a plugin that is given input and output buffers by
 * a framework whose allocator it cannot reach, a service running inside a fixed
 * memory reservation, a step that must not call cudaMalloc because that call
 * synchronises the whole device.  For them this entry point does exactly what
 * dmf_attn_bwd does with its minimal workspace (two floats per query row; the
 * kernels whose results are reproducible bit for bit), but takes that scratch
 * from a fixed array that lives inside the library image instead of
 * args->workspace, which is ignored together with args->workspace_bytes.  It
 * calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limit: batch * heads * seqlen_q <= DMF_ATTN_STATIC_MAX_ROWS (1,048,576 rows,
 * i.e. 8 MiB of device memory, held by every GPU that loads the library until
 * the process exits).  Larger problems return DMF_ATTN_ERR_TOO_LARGE and launch
 * nothing.
 *
 * The first call on each device looks the array's device address up (with that
 * device current) and caches it; make that first call outside any stream
 * capture.  All calls on a device share the one array: its contents are
 * overwritten by every call (nothing in it needs clearing - the first pass
 * writes every slot the second pass reads), so two calls whose kernels may
 * overlap on the GPU (different streams, no dependency) race with each other
 * and must be ordered by the caller.
 */
#define DMF_ATTN_STATIC_MAX_ROWS (1 << 20)
int dmf_attn_bwd_static(const dmf_attn_bwd_args* args);

/*
 * Copy a status word back (synchronises the stream) and translate it:
 * DMF_ATTN_OK if it is zero, DMF_ATTN_ERR_TIMEOUT otherwise; *raw (optional)
 * receives the word itself (which wait gave up).
 */
int dmf_attn_check_status_word(const int32_t* status_word, void* stream, int32_t* raw);

/*
 * Checking hooks.  None of them has a counterpart in the reference; they exist so that the library's
 * own tests can reach behaviour that a normal call cannot show.
 *
 * dmf_attn_fwd_dual_f32out: dmf_attn_fwd_dual with args->o and args->to as FLOAT tensors (strides in
 * floats, 16-byte aligned rows): the accumulators are normalised and stored before the rounding to
 * the 16-bit output type.  This is how the "fp32-accumulated output" tolerance of the path is
 * checked (max|a-b| / max|b| <= 1e-3 against an fp64 evaluation that rounds its operands where the
 * kernel does).  bf16 inputs, head_dim <= 80, an even number of 128-row query tiles; anything else
 * is DMF_ATTN_ERR_HEAD_DIM.  Slow per-row stores: not a production path.
 *
 * dmf_attn_selftest_wait_limit: runs one small kernel in which a thread waits on a barrier that is
 * never signalled, with a wait limit of limit_cycles SM cycles (1e3 .. 5e7) instead of the
 * library's ~2 s.  The wait must give up, write 901 to *status_word, and the kernel must return
 * normally with the context intact.  result: four int32 in device memory, {first wait succeeded
 * (expect 0), a second thread's longer wait succeeded (expect 0: it sees the abort flag), a wait
 * on a signalled barrier succeeded (expect 1), cycles the first thread waited}.
 *
 * dmf_attn_kernel_name: the kernel template instance the launcher picks for a problem, as text
 * (op: 0 = fused forward + tangent, 1 = plain forward, 2 = backward).
 */
int dmf_attn_fwd_dual_f32out(const dmf_attn_fwd_args* args);
int dmf_attn_selftest_wait_limit(int64_t limit_cycles, int32_t* status_word, int32_t* result, void* stream);
int dmf_attn_kernel_name(int32_t op, int32_t seqlen_q, int32_t seqlen_kv, int32_t head_dim, int32_t dtype,
                         char* buf, size_t len);

/*
 * Argument validation only (no device work): the status the compute entry
 * points would return for these arguments before touching the GPU.
 */
int dmf_attn_validate_fwd(const dmf_attn_fwd_args* args, int dual);
int dmf_attn_validate_bwd(const dmf_attn_bwd_args* args);

/*
 * Per-head RMS normalisation of q or k, with its tangent, and its primal backward.
 *
 * Replaces RMSNorm.forward of the reference's attention block (models/layers.py:33-42, applied to
 * q and k at layers.py:148) and what PyTorch's forward-mode AD makes of it under torch.func.jvp:
 *   r = rsqrt(mean_d(x^2) + eps)    y = x r w    ty = (tx r - x r^3 mean_d(x tx)) w
 * x, tx, y, ty: (B, L, H, D) tensors in the layout rules above (tx.ptr == NULL: no tangent, ty is
 * not written); weight: D floats in device memory (the module's parameter; it is rounded to the
 * tensors' 16-bit type before use, as the reference casts it).  head_dim: a multiple of 8, at most
 * 128; seqlen: any positive value.  Arithmetic is fp32 with one rounding of the result.
 */
typedef struct dmf_rmsnorm_args {
  int32_t batch;
  int32_t seqlen;
  int32_t heads;
  int32_t head_dim;
  int32_t dtype;          /* enum dmf_attn_dtype */
  float eps;              /* the reference uses 1e-6 */
  dmf_attn_tensor x, tx;  /* read only */
  dmf_attn_tensor y, ty;  /* out */
  const float* weight;    /* (D) */
  void* stream;           /* cudaStream_t */
} dmf_rmsnorm_args;

int dmf_rmsnorm_fwd(const dmf_rmsnorm_args* args);

/*
 * Backward of y with respect to x and weight (the tangent output carries no gradient, like the
 * attention's): dx = r g - x r^3 mean_d(x g) with g = dy w, dweight_d = sum over rows of dy_d x_d r.
 * dweight: D floats, overwritten.  workspace: device memory of at least
 * dmf_rmsnorm_bwd_workspace_bytes(head_dim) bytes (per-block partial sums of dweight, reduced in a
 * fixed order: the result is bit-reproducible); its contents on entry do not matter.
 */
typedef struct dmf_rmsnorm_bwd_args {
  int32_t batch;
  int32_t seqlen;
  int32_t heads;
  int32_t head_dim;
  int32_t dtype;
  float eps;
  dmf_attn_tensor dy, x;  /* read only */
  dmf_attn_tensor dx;     /* out */
  const float* weight;    /* (D) */
  float* dweight;         /* out, (D) */
  void* workspace;
  size_t workspace_bytes;
  void* stream;
} dmf_rmsnorm_bwd_args;

size_t dmf_rmsnorm_bwd_workspace_bytes(int32_t head_dim);
int dmf_rmsnorm_bwd(const dmf_rmsnorm_bwd_args* args);

#ifdef __cplusplus
}
#endif

#endif /* DMF_ATTN_H_ */
