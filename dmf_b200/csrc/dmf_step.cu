// Host side and kernel of include/dmf_step.h: clip + AdamW + EMA + zero-grad in one pass over flat fp32 buffers.
#include "dmf_step.h"

#include <cuda_runtime.h>

#include <cstdint>

#include "dmf_attn.h"  // status codes

namespace {

struct StepParams {
  float* __restrict__ grad;
  float* __restrict__ param;
  float* __restrict__ exp_avg;
  float* __restrict__ exp_avg_sq;
  float* __restrict__ ema;
  const float* __restrict__ grad_norm;
  int64_t count;
  float max_grad_norm, lr, beta1, beta2, eps, weight_decay, step_size, bias_correction2_sqrt, ema_decay;
};

__device__ __forceinline__ void step_one(float& g, float& p, float& m, float& v, float& e, float clip, bool has_ema,
                                         const StepParams& a) {
  g *= clip;
  if (a.weight_decay != 0.f) p -= a.lr * a.weight_decay * p;
  m = m + (1.f - a.beta1) * (g - m);
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v) / a.bias_correction2_sqrt + a.eps;
  p -= a.step_size * m / denom;
  if (has_ema) e = e * a.ema_decay + p * (1.f - a.ema_decay);
}

// One thread handles one float4 of each buffer per iteration; all loads of an iteration are issued before the first
// use.  kEma = false: no EMA buffer.  Grid-stride; the last (count % 4) elements are handled by thread 0 of block 0.
template <bool kEma>
__global__ void __launch_bounds__(256) step_tail_kernel(const StepParams a) {
  const float clip = a.grad_norm != nullptr ? fminf(1.f, a.max_grad_norm / (*a.grad_norm + 1e-6f)) : 1.f;
  const int64_t n4 = a.count >> 2;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float4* g4 = reinterpret_cast<float4*>(a.grad);
  float4* p4 = reinterpret_cast<float4*>(a.param);
  float4* m4 = reinterpret_cast<float4*>(a.exp_avg);
  float4* v4 = reinterpret_cast<float4*>(a.exp_avg_sq);
  float4* e4 = reinterpret_cast<float4*>(a.ema);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 g = __ldcs(g4 + i), p = __ldcs(p4 + i), m = __ldcs(m4 + i), v = __ldcs(v4 + i);
    float4 e = kEma ? __ldcs(e4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    step_one(g.x, p.x, m.x, v.x, e.x, clip, kEma, a);
    step_one(g.y, p.y, m.y, v.y, e.y, clip, kEma, a);
    step_one(g.z, p.z, m.z, v.z, e.z, clip, kEma, a);
    step_one(g.w, p.w, m.w, v.w, e.w, clip, kEma, a);
    __stcs(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
    p4[i] = p;  // the weights are read again right away by the next forward pass: keep them cacheable
    __stcs(m4 + i, m);
    __stcs(v4 + i, v);
    if (kEma) __stcs(e4 + i, e);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int64_t i = n4 << 2; i < a.count; ++i) {
      float g = a.grad[i], p = a.param[i], m = a.exp_avg[i], v = a.exp_avg_sq[i], e = kEma ? a.ema[i] : 0.f;
      step_one(g, p, m, v, e, clip, kEma, a);
      a.grad[i] = 0.f;
      a.param[i] = p;
      a.exp_avg[i] = m;
      a.exp_avg_sq[i] = v;
      if (kEma) a.ema[i] = e;
    }
  }
}

int run_step_tail(const dmf_step_tail_args* a) {
  if (a == nullptr || a->grad == nullptr || a->param == nullptr || a->exp_avg == nullptr || a->exp_avg_sq == nullptr)
    return DMF_ATTN_ERR_NULL;
  if (a->count < 1) return DMF_ATTN_ERR_SHAPE;
  const void* ptrs[] = {a->grad, a->param, a->exp_avg, a->exp_avg_sq, a->ema};
  for (const void* ptr : ptrs)
    if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  if (!(a->bias_correction2_sqrt > 0.f) || !(a->step_size == a->step_size)) return DMF_ATTN_ERR_SHAPE;
  int dev = -1, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_DEVICE;
  }
  StepParams p;
  p.grad = a->grad; p.param = a->param; p.exp_avg = a->exp_avg; p.exp_avg_sq = a->exp_avg_sq; p.ema = a->ema;
  p.grad_norm = a->grad_norm;
  p.count = a->count;
  p.max_grad_norm = a->max_grad_norm; p.lr = a->lr; p.beta1 = a->beta1; p.beta2 = a->beta2; p.eps = a->eps;
  p.weight_decay = a->weight_decay; p.step_size = a->step_size; p.bias_correction2_sqrt = a->bias_correction2_sqrt;
  p.ema_decay = a->ema_decay;
  const int64_t n4 = a->count >> 2;
  int64_t blocks = (n4 + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sms) * 8;  // 8 blocks of 256 threads per SM, grid-stride
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (a->ema != nullptr) step_tail_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(p);
  else step_tail_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int dmf_step_tail(const dmf_step_tail_args* args) {
  return run_step_tail(args);
}
