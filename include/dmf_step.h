/*
 * dmf_step.h - C ABI of the fused end of an optimisation step of Decoupled MeanFlow fine-tuning on B200:
 * gradient clipping, AdamW and the EMA of the weights in ONE pass over flat fp32 buffers.
 *
 * Replaces, for a model whose trainable parameters, gradients, AdamW moments and EMA copy each live in one
 * contiguous fp32 buffer, the sequence train_dmf.py:331-338 runs after backward:
 *   accelerator.clip_grad_norm_(model.parameters(), max_grad_norm)        (train_dmf.py:332-333)
 *   optimizer.step()          torch.optim.AdamW(..., fused=True)          (train_dmf.py:221-228, 334)
 *   optimizer.zero_grad()                                                  (train_dmf.py:335)
 *   update_ema(ema, model, decay)      ema = ema * decay + p * (1 - decay) (train_dmf.py:54-99, 338)
 * As separate library kernels these read and write the buffers about 16 times (43 GB for DMFT-XL/2, 675 M parameters);
 * fused, every buffer is read once and written once (27 GB).  HBM-bound streaming: algorithmic bytes 40 per element.
 *
 * Same conventions as dmf_attn.h: extern "C", plain pointers, no allocation, asynchronous on the given stream,
 * status codes of enum dmf_attn_status.
 */
#ifndef DMF_STEP_H_
#define DMF_STEP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dmf_step_tail_args {
  int64_t count;          /* elements of every buffer                                                       */
  float* grad;            /* in: the gradient (already averaged over micro-batches and ranks); out: zeros    */
  float* param;           /* in / out                                                                        */
  float* exp_avg;         /* in / out: AdamW first moment                                                    */
  float* exp_avg_sq;      /* in / out: AdamW second moment                                                   */
  float* ema;             /* in / out: EMA of param; NULL: no EMA                                            */
  const float* grad_norm; /* device scalar: 2-norm of grad, as clip_grad_norm_ computes it; NULL: no clipping */
  float max_grad_norm;    /* gradients are scaled by min(1, max_grad_norm / (*grad_norm + 1e-6))             */
  float lr;
  float beta1, beta2;
  float eps;
  float weight_decay;     /* decoupled: param *= 1 - lr * weight_decay                                       */
  float step_size;        /* lr / (1 - beta1^t), t = number of this step (from 1), computed by the caller    */
  float bias_correction2_sqrt; /* sqrt(1 - beta2^t)                                                          */
  float ema_decay;
  int32_t reserved;
  void* stream;           /* cudaStream_t */
} dmf_step_tail_args;

/*
 * g = grad * clip;  m = m + (1 - beta1) (g - m);  v = beta2 v + (1 - beta2) g g;
 * param = param (1 - lr wd) - step_size m / (sqrt(v) / bias_correction2_sqrt + eps);
 * ema = ema decay + param (1 - decay);  grad = 0.
 * The arithmetic of torch's fused AdamW kernel, in fp32.  All pointers 16-byte aligned.
 */
int dmf_step_tail(const dmf_step_tail_args* args);

#ifdef __cplusplus
}
#endif

#endif /* DMF_STEP_H_ */
