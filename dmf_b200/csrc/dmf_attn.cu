// Host side of the C ABI declared in include/dmf_attn.h: argument validation,
// TMA tensor-map construction and kernel launches.  No torch types, no device
// allocation, no global mutable state besides per-device cached attributes.
#include "dmf_attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "attn_bwd.cuh"
#include "attn_bwd_fused.cuh"
#include "attn_bwd_split.cuh"
#include "attn_bwd_stream.cuh"
#include "attn_fwd.cuh"
#include "attn_fwd_pair.cuh"
#include "rmsnorm.cuh"

namespace {

using namespace dmf;

// ---- driver entry point for tensor-map encoding (no link-time libcuda dependency) ----

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (fn != nullptr) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || sym == nullptr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  cached.store(fn, std::memory_order_release);
  return fn;
}

// ---- per-device attributes ----

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  std::atomic<int> ready{0};
  int sm_count = 0;
  int cc_major = 0;
};
DeviceInfo g_devices[kMaxDevices];

int device_info(int* sm_count) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_DEVICE;
  }
  DeviceInfo& d = g_devices[dev];
  if (d.ready.load(std::memory_order_acquire) == 0) {
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      return DMF_ATTN_ERR_DEVICE;
    }
    d.sm_count = sms;
    d.cc_major = major;
    d.ready.store(1, std::memory_order_release);
  }
  if (d.cc_major != 10) return DMF_ATTN_ERR_DEVICE;
  *sm_count = d.sm_count;
  return DMF_ATTN_OK;
}

// ---- validation ----

inline int tail_of(int d) {
  if (d == 64) return 0;
  if (d > 64 && d <= 80) return 16;
  if (d > 80 && d <= 96) return 32;
  if (d > 96 && d <= 128) return 64;
  return -1;
}

inline int check_tensor(const dmf_attn_tensor& t, int elem_bytes) {
  if (t.ptr == nullptr) return DMF_ATTN_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  const int64_t s[3] = {t.stride_b, t.stride_l, t.stride_h};
  for (int i = 0; i < 3; ++i) {
    if (s[i] < 0) return DMF_ATTN_ERR_STRIDE;
    if ((s[i] * elem_bytes) % 16 != 0) return DMF_ATTN_ERR_STRIDE;
  }
  return DMF_ATTN_OK;
}

inline int check_dims(int batch, int lq, int lkv, int heads, int d, int dtype) {
  if (dtype != DMF_ATTN_BF16 && dtype != DMF_ATTN_FP16) return DMF_ATTN_ERR_DTYPE;
  if (d < 64 || d > 128 || (d % 8) != 0) return DMF_ATTN_ERR_HEAD_DIM;
  if (batch < 1 || heads < 1) return DMF_ATTN_ERR_SHAPE;
  if (lq < kBlockQ || lkv < kBlockKV || (lq % kBlockQ) != 0 || (lkv % kBlockKV) != 0) return DMF_ATTN_ERR_SEQLEN;
  if (static_cast<int64_t>(batch) * heads * (lq / kBlockQ) > 0x7fffffffll) return DMF_ATTN_ERR_SHAPE;
  return DMF_ATTN_OK;
}

int validate_fwd(const dmf_attn_fwd_args* a, bool dual, int out_elem_bytes = 2) {
  if (a == nullptr) return DMF_ATTN_ERR_NULL;
  int st = check_dims(a->batch, a->seqlen_q, a->seqlen_kv, a->heads, a->head_dim, a->dtype);
  if (st != DMF_ATTN_OK) return st;
  if (a->lse == nullptr) return DMF_ATTN_ERR_NULL;
  if (!std::isfinite(a->softmax_scale)) return DMF_ATTN_ERR_SHAPE;
  const dmf_attn_tensor* prim[] = {&a->q, &a->k, &a->v};
  for (const dmf_attn_tensor* t : prim)
    if ((st = check_tensor(*t, 2)) != DMF_ATTN_OK) return st;
  if ((st = check_tensor(a->o, out_elem_bytes)) != DMF_ATTN_OK) return st;
  if (dual) {
    const dmf_attn_tensor* tang[] = {&a->tq, &a->tk, &a->tv};
    for (const dmf_attn_tensor* t : tang)
      if ((st = check_tensor(*t, 2)) != DMF_ATTN_OK) return st;
    if ((st = check_tensor(a->to, out_elem_bytes)) != DMF_ATTN_OK) return st;
  }
  return DMF_ATTN_OK;
}

// ---- tensor maps ----

// Map of a (B, L, H, D) tensor seen as dims (D, L, H, B); box = box_d columns x box_l rows of one (b, h).
int make_map(CUtensorMap* map, const dmf_attn_tensor& t, int dtype, int batch, int seqlen, int heads, int d,
             int box_d, int box_l, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return DMF_ATTN_ERR_DEVICE;
  const cuuint64_t es = 2;
  const cuuint64_t row_bytes = ((static_cast<cuuint64_t>(d) * es + 15) / 16) * 16;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(seqlen),
                        static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // a dimension of extent 1 may carry any stride in the caller's tensor; give the map a legal one
  cuuint64_t strides[3] = {
      seqlen > 1 ? static_cast<cuuint64_t>(t.stride_l) * es : row_bytes,
      heads > 1 ? static_cast<cuuint64_t>(t.stride_h) * es : row_bytes,
      batch > 1 ? static_cast<cuuint64_t>(t.stride_b) * es : row_bytes,
  };
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || (strides[i] % 16) != 0) return DMF_ATTN_ERR_STRIDE;
  cuuint32_t box[4] = {static_cast<cuuint32_t>(box_d), static_cast<cuuint32_t>(box_l), 1, 1};
  cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt =
      dtype == DMF_ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = encode(map, dt, 4, t.ptr, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DMF_ATTN_OK : DMF_ATTN_ERR_TENSOR_MAP;
}

inline CUtensorMapSwizzle tail_swizzle(int tail) {
  return tail == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (tail == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

int make_map_pair(CUtensorMap* main_map, CUtensorMap* tail_map, const dmf_attn_tensor& t, int dtype, int batch,
                  int seqlen, int heads, int d, int tail, int box_l) {
  int st = make_map(main_map, t, dtype, batch, seqlen, heads, d, 64, box_l, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != DMF_ATTN_OK) return st;
  if (tail > 0) return make_map(tail_map, t, dtype, batch, seqlen, heads, d, tail, box_l, tail_swizzle(tail));
  std::memset(tail_map, 0, sizeof(CUtensorMap));
  return DMF_ATTN_OK;
}

// ---- forward launch ----

template <typename T, int TAIL, bool kDual>
int launch_fwd_inst(const FwdParams& p, int grid, cudaStream_t stream) {
  using TR = FwdTraits<TAIL, kDual>;
  auto kernel = attn_fwd_kernel<T, TAIL, kDual>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  kernel<<<grid, kFwdThreads, TR::kSmemBytes, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

template <typename T, bool kDual>
int launch_fwd_tail(const FwdParams& p, int tail, int grid, cudaStream_t stream) {
  switch (tail) {
    case 0: return launch_fwd_inst<T, 0, kDual>(p, grid, stream);
    case 16: return launch_fwd_inst<T, 16, kDual>(p, grid, stream);
    case 32: return launch_fwd_inst<T, 32, kDual>(p, grid, stream);
    case 64: return launch_fwd_inst<T, 64, kDual>(p, grid, stream);
    default: return DMF_ATTN_ERR_HEAD_DIM;
  }
}

// ---- forward launch, CTA-pair variant (dual pass, head_dim <= 96, even number of query tiles) ----

template <typename T, int TAIL, bool kDual, bool kShort, bool kF32Out = false>
int launch_pair_inst(const FwdParams& p, int clusters, cudaStream_t stream) {
  using TR = PairTraits<TAIL, kShort>;
  auto kernel = attn_fwd_pair_kernel<T, TAIL, kDual, kShort, kF32Out>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = TR::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (std::getenv("DMF_ATTN_DEBUG") != nullptr) {
    int n = -1;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
    std::fprintf(stderr, "[dmf_attn] pair kernel: %d clusters requested, max active clusters %d (%s)\n", clusters, n,
                 cudaGetErrorString(e));
  }
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  return DMF_ATTN_OK;
}

template <typename T, bool kDual>
int launch_pair_tail(const FwdParams& p, int tail, int clusters, cudaStream_t stream) {
  switch (tail) {
    case 0: return launch_pair_inst<T, 0, kDual, false>(p, clusters, stream);
    case 16:  // the only head_dim whose shared-memory split depends on the length of the key sequence
      return p.seqlen_kv <= kShortMaxBlocks * kBlockKV ? launch_pair_inst<T, 16, kDual, true>(p, clusters, stream)
                                                       : launch_pair_inst<T, 16, kDual, false>(p, clusters, stream);
    case 32: return launch_pair_inst<T, 32, kDual, false>(p, clusters, stream);
    default: return DMF_ATTN_ERR_HEAD_DIM;
  }
}

// The fp32-output checking mode: bf16, dual pass, head_dim 64 and 65..80 only (what its test covers).
int launch_pair_f32out(const FwdParams& p, int tail, int clusters, cudaStream_t stream) {
  const bool is_short = p.seqlen_kv <= kShortMaxBlocks * kBlockKV;
  switch (tail) {
    case 0: return launch_pair_inst<__nv_bfloat16, 0, true, false, true>(p, clusters, stream);
    case 16:
      return is_short ? launch_pair_inst<__nv_bfloat16, 16, true, true, true>(p, clusters, stream)
                      : launch_pair_inst<__nv_bfloat16, 16, true, false, true>(p, clusters, stream);
    default: return DMF_ATTN_ERR_HEAD_DIM;
  }
}

// DMF_ATTN_PAIR=0 in the environment keeps the single-CTA kernel (for comparisons).
bool pair_kernel_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("DMF_ATTN_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  return enabled;
}

// Which kernel template the launcher picks for a problem; one rule for the launch and for dmf_attn_kernel_name.
bool fwd_uses_pair(int tail, int seqlen_q) {
  return tail >= 0 && tail <= 32 && ((seqlen_q / kBlockQ) % 2 == 0) && pair_kernel_enabled();
}

int run_fwd(const dmf_attn_fwd_args* a, bool dual, bool f32out = false) {
  int st = validate_fwd(a, dual, f32out ? 4 : 2);
  if (st != DMF_ATTN_OK) return st;
  int sm_count = 0;
  if ((st = device_info(&sm_count)) != DMF_ATTN_OK) return st;

  const int tail = tail_of(a->head_dim);
  FwdParams p;
  std::memset(&p, 0, sizeof(p));
  const int B = a->batch, H = a->heads, D = a->head_dim, Lq = a->seqlen_q, Lk = a->seqlen_kv, dt = a->dtype;
  if ((st = make_map_pair(&p.q_main, &p.q_tail, a->q, dt, B, Lq, H, D, tail, kBlockQ)) != DMF_ATTN_OK) return st;
  // CTA-pair kernel: dual pass, P in its own tensor-memory columns (head_dim <= 96), tiles pair up
  const bool pair = fwd_uses_pair(tail, Lq);
  if (f32out && !(pair && dual && dt == DMF_ATTN_BF16 && tail <= 16)) return DMF_ATTN_ERR_HEAD_DIM;
  const int k_box_rows = pair ? kBlockKV / 2 : kBlockKV;  // a CTA of a pair loads half of the key rows
  if ((st = make_map_pair(&p.k_main, &p.k_tail, a->k, dt, B, Lk, H, D, tail, k_box_rows)) != DMF_ATTN_OK) return st;
  if ((st = make_map(&p.v_map, a->v, dt, B, Lk, H, D, 32, kBlockKV, CU_TENSOR_MAP_SWIZZLE_64B)) != DMF_ATTN_OK) return st;
  if (dual) {
    if ((st = make_map_pair(&p.tq_main, &p.tq_tail, a->tq, dt, B, Lq, H, D, tail, kBlockQ)) != DMF_ATTN_OK) return st;
    if ((st = make_map_pair(&p.tk_main, &p.tk_tail, a->tk, dt, B, Lk, H, D, tail, k_box_rows)) != DMF_ATTN_OK) return st;
    if ((st = make_map(&p.tv_map, a->tv, dt, B, Lk, H, D, 32, kBlockKV, CU_TENSOR_MAP_SWIZZLE_64B)) != DMF_ATTN_OK) return st;
  }
  p.o = a->o.ptr;
  p.o_sb = a->o.stride_b; p.o_sl = a->o.stride_l; p.o_sh = a->o.stride_h;
  if (dual) {
    p.to = a->to.ptr;
    p.to_sb = a->to.stride_b; p.to_sl = a->to.stride_l; p.to_sh = a->to.stride_h;
  }
  p.lse = a->lse;
  p.status_word = a->status_word;
  p.batch = B; p.heads = H; p.seqlen_q = Lq; p.seqlen_kv = Lk; p.head_dim = D;
  p.num_q_tiles = Lq / kBlockQ;
  p.num_tiles = B * H * p.num_q_tiles;
  p.scale = a->softmax_scale;
  p.scale_log2e = a->softmax_scale * 1.4426950408889634f;
  if (D == 72) {
    // head rows of 144 bytes straddle 32-byte sectors on every other head: let the kernel start its
    // boxes 8 columns early there.  All tensors of a group must agree on the alignment pattern.
    auto pattern = [](const dmf_attn_tensor& t, int* out) -> bool {
      if ((t.stride_l * 2) % 32 != 0) return false;  // alignment must not change along the sequence
      out[0] = static_cast<int>(reinterpret_cast<uintptr_t>(t.ptr) & 31);
      out[1] = static_cast<int>((t.stride_b * 2) & 31);
      out[2] = static_cast<int>((t.stride_h * 2) & 31);
      return true;
    };
    const dmf_attn_tensor* g0[4] = {&a->q, &a->k, &a->tq, &a->tk};
    const dmf_attn_tensor* g1[2] = {&a->v, &a->tv};
    const dmf_attn_tensor* const* groups[2] = {g0, g1};
    const int counts[2] = {dual ? 4 : 2, dual ? 2 : 1};
    for (int g = 0; g < 2; ++g) {
      int ref[3] = {0, 0, 0};
      bool ok = pattern(*groups[g][0], ref);
      for (int i = 1; ok && i < counts[g]; ++i) {
        int cur[3];
        ok = pattern(*groups[g][i], cur) && cur[0] == ref[0] && cur[1] == ref[1] && cur[2] == ref[2];
      }
      p.align_enable[g] = ok ? 1 : 0;
      p.align0[g] = ref[0]; p.align_b[g] = ref[1]; p.align_h[g] = ref[2];
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if ((pair || !dual) && !f32out) {  // kernels that write their outputs with TMA stores
    if ((st = make_map_pair(&p.o_main, &p.o_tail, a->o, dt, B, Lq, H, D, tail, kBlockQ)) != DMF_ATTN_OK) return st;
  }
  if (pair) {
    if (dual && !f32out &&
        (st = make_map_pair(&p.to_main, &p.to_tail, a->to, dt, B, Lq, H, D, tail, kBlockQ)) != DMF_ATTN_OK)
      return st;
    p.align_enable[1] = 0;  // the pair kernel's V column order has no room for the 8-column shift
    p.num_tiles /= 2;       // tile pairs
    const int max_clusters = sm_count / 2;
    const int clusters = p.num_tiles < max_clusters ? p.num_tiles : max_clusters;
    if (f32out) return launch_pair_f32out(p, tail, clusters, stream);
    if (dual)
      return dt == DMF_ATTN_BF16 ? launch_pair_tail<__nv_bfloat16, true>(p, tail, clusters, stream)
                                 : launch_pair_tail<__half, true>(p, tail, clusters, stream);
    return dt == DMF_ATTN_BF16 ? launch_pair_tail<__nv_bfloat16, false>(p, tail, clusters, stream)
                               : launch_pair_tail<__half, false>(p, tail, clusters, stream);
  }
  const int grid = p.num_tiles < sm_count ? p.num_tiles : sm_count;
  if (dt == DMF_ATTN_BF16)
    return dual ? launch_fwd_tail<__nv_bfloat16, true>(p, tail, grid, stream)
                : launch_fwd_tail<__nv_bfloat16, false>(p, tail, grid, stream);
  return dual ? launch_fwd_tail<__half, true>(p, tail, grid, stream)
              : launch_fwd_tail<__half, false>(p, tail, grid, stream);
}

// ---- backward ----

// The part of the workspace every backward kernel needs: -lse*log2(e) and delta = rowsum(dO*O), one float per
// query row each.  A call is valid with this much.
size_t bwd_workspace_min_bytes(int batch, int lq, int heads) {
  return 2 * sizeof(float) * static_cast<size_t>(batch) * heads * lq;
}

// Offset of the fp32 dQ accumulator of the one-pass long-sequence kernel behind the two rows.
size_t bwd_stream_acc_offset(int batch, int lq, int heads) {
  return (bwd_workspace_min_bytes(batch, lq, heads) + 255) & ~static_cast<size_t>(255);
}

bool bwd_uses_fused(int tail, int seqlen_q, int seqlen_kv);
bool bwd_stream_applies(int tail, int seqlen_q, int seqlen_kv);

// What dmf_attn_bwd_workspace_bytes reports: where the one-pass long-sequence kernel applies, room for its dQ
// accumulator too (with less, dmf_attn_bwd runs the two-launch kernels).
size_t bwd_workspace_bytes(int batch, int lq, int lkv, int heads, int d) {
  if (check_dims(batch, lq, lkv, heads, d, DMF_ATTN_BF16) != DMF_ATTN_OK) return 0;
  if (bwd_stream_applies(tail_of(d), lq, lkv))
    return bwd_stream_acc_offset(batch, lq, heads) + sizeof(float) * static_cast<size_t>(batch) * heads * lq * d;
  return bwd_workspace_min_bytes(batch, lq, heads);
}

int validate_bwd(const dmf_attn_bwd_args* a) {
  if (a == nullptr) return DMF_ATTN_ERR_NULL;
  int st = check_dims(a->batch, a->seqlen_q, a->seqlen_kv, a->heads, a->head_dim, a->dtype);
  if (st != DMF_ATTN_OK) return st;
  if (a->lse == nullptr) return DMF_ATTN_ERR_NULL;
  if (!std::isfinite(a->softmax_scale)) return DMF_ATTN_ERR_SHAPE;
  const dmf_attn_tensor* ts[] = {&a->dout, &a->q, &a->k, &a->v, &a->o, &a->dq, &a->dk, &a->dv};
  for (const dmf_attn_tensor* t : ts)
    if ((st = check_tensor(*t, 2)) != DMF_ATTN_OK) return st;
  const size_t need = bwd_workspace_min_bytes(a->batch, a->seqlen_q, a->heads);
  if (a->workspace == nullptr || a->workspace_bytes < need) return DMF_ATTN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  return DMF_ATTN_OK;
}

template <typename T, int TAIL, int kMode>
int launch_bwd_inst(const BwdParams& p, int grid, cudaStream_t stream) {
  using TR = BwdTraits<TAIL>;
  auto kernel = attn_bwd_kernel<T, TAIL, kMode>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  kernel<<<grid, kBwdThreads, TR::kSmemBytes, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

// head_dim <= 96: the role-split kernel (P warps / D warps, three ring stages)
template <typename T, int TAIL, int kMode>
int launch_bwd_split_inst(const BwdParams& p, int grid, cudaStream_t stream) {
  using TR = BwdSplitTraits<TAIL>;
  auto kernel = attn_bwd_split_kernel<T, TAIL, kMode>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  kernel<<<grid, kBwdSplitThreads, TR::kSmemBytes, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

// DMF_ATTN_BWD_SPLIT=0 in the environment keeps the single-warpgroup kernel (for comparisons).
bool bwd_split_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("DMF_ATTN_BWD_SPLIT");
    return e == nullptr || e[0] != '0';
  }();
  return enabled;
}

template <typename T, int kMode>
int launch_bwd_tail(const BwdParams& p, int tail, int grid, cudaStream_t stream) {
  if (tail <= 32 && bwd_split_enabled()) {
    switch (tail) {
      case 0: return launch_bwd_split_inst<T, 0, kMode>(p, grid, stream);
      case 16: return launch_bwd_split_inst<T, 16, kMode>(p, grid, stream);
      case 32: return launch_bwd_split_inst<T, 32, kMode>(p, grid, stream);
      default: return DMF_ATTN_ERR_HEAD_DIM;
    }
  }
  switch (tail) {
    case 0: return launch_bwd_inst<T, 0, kMode>(p, grid, stream);
    case 16: return launch_bwd_inst<T, 16, kMode>(p, grid, stream);
    case 32: return launch_bwd_inst<T, 32, kMode>(p, grid, stream);
    case 64: return launch_bwd_inst<T, 64, kMode>(p, grid, stream);
    default: return DMF_ATTN_ERR_HEAD_DIM;
  }
}

// ---- backward in one pass (two-tile sequences, head_dim <= 80) ----

// DMF_ATTN_BWD_FUSED=0 in the environment takes this kernel out (for comparisons): two-tile sequences then go the
// way of longer ones.
bool bwd_fused_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("DMF_ATTN_BWD_FUSED");
    return e == nullptr || e[0] != '0';
  }();
  return enabled;
}

bool bwd_uses_fused(int tail, int seqlen_q, int seqlen_kv) {
  return tail >= 0 && tail <= 16 && seqlen_q == kBwdFusedSeqlen && seqlen_kv == kBwdFusedSeqlen && bwd_fused_enabled();
}

template <typename T, int TAIL>
int launch_bwd_fused_inst(const BwdFusedParams& p, int clusters, cudaStream_t stream) {
  using TR = BwdFusedTraits<TAIL>;
  auto kernel = attn_bwd_fused_kernel<T, TAIL>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kBwdFusedThreads, 1, 1);
  cfg.dynamicSmemBytes = TR::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  return DMF_ATTN_OK;
}

int run_bwd_fused(const dmf_attn_bwd_args* a, int tail, int sm_count) {
  const int B = a->batch, H = a->heads, D = a->head_dim, L = a->seqlen_q, dt = a->dtype;
  BwdFusedParams p;
  std::memset(&p, 0, sizeof(p));
  int st;
  if ((st = make_map_pair(&p.q_main, &p.q_tail, a->q, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.do_main, &p.do_tail, a->dout, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.k_main, &p.k_tail, a->k, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.v_main, &p.v_tail, a->v, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.o_main, &p.o_tail, a->o, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.dq_main, &p.dq_tail, a->dq, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.dk_main, &p.dk_tail, a->dk, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.dv_main, &p.dv_tail, a->dv, dt, B, L, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  p.lse = a->lse;
  p.status_word = a->status_word;
  p.batch = B; p.heads = H; p.head_dim = D;
  p.num_heads_total = B * H;
  p.scale = a->softmax_scale;
  p.scale_log2e = a->softmax_scale * 1.4426950408889634f;
  const int max_clusters = sm_count / 2;
  const int clusters = p.num_heads_total < max_clusters ? p.num_heads_total : max_clusters;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (dt == DMF_ATTN_BF16)
    return tail == 0 ? launch_bwd_fused_inst<__nv_bfloat16, 0>(p, clusters, stream)
                     : launch_bwd_fused_inst<__nv_bfloat16, 16>(p, clusters, stream);
  return tail == 0 ? launch_bwd_fused_inst<__half, 0>(p, clusters, stream)
                   : launch_bwd_fused_inst<__half, 16>(p, clusters, stream);
}

// ---- backward in one pass, long sequences (head_dim <= 80): key tiles resident, dQ summed with atomics ----

// DMF_ATTN_BWD_STREAM=0 in the environment keeps the two-launch backward (for comparisons, and for callers that
// need a dQ that is reproducible bit for bit).
bool bwd_stream_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("DMF_ATTN_BWD_STREAM");
    return e == nullptr || e[0] != '0';
  }();
  return enabled;
}

bool bwd_stream_applies(int tail, int seqlen_q, int seqlen_kv) {
  return tail >= 0 && tail <= 16 && !bwd_uses_fused(tail, seqlen_q, seqlen_kv) && bwd_stream_enabled();
}

template <typename T, int TAIL>
int launch_bwd_stream_inst(const BwdStreamParams& p, const dmf_attn_bwd_args* a, int sm_count, cudaStream_t stream) {
  using TR = BwdStreamTraits<TAIL>;
  auto kernel = attn_bwd_stream_kernel<T, TAIL>;
  auto convert = bwd_dq_convert_kernel<T>;
  const int convert_smem = (p.head_dim / 4) * 128 * 16;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::kSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(convert, cudaFuncAttributeMaxDynamicSharedMemorySize, convert_smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  // rows of the pre-kernel's block: 32 positions of all heads, fewer when that does not fit 48 KB of shared memory
  int lrows = 32;
  while (lrows > 1 && static_cast<size_t>(lrows) * p.heads * (p.head_dim / 8) * sizeof(float) > 48 * 1024) lrows /= 2;
  const size_t delta_smem = static_cast<size_t>(lrows) * p.heads * (p.head_dim / 8) * sizeof(float);
  if (delta_smem > 48 * 1024) return DMF_ATTN_ERR_SHAPE;
  const int64_t want = static_cast<int64_t>(p.batch) * (p.seqlen_q / lrows);
  const int delta_grid = static_cast<int>(want < 16 * sm_count ? want : 16 * sm_count);
  bwd_delta_kernel<T><<<delta_grid, 256, delta_smem, stream>>>(
      static_cast<const T*>(a->o.ptr), static_cast<const T*>(a->dout.ptr), a->lse, const_cast<float*>(p.ndelta),
      const_cast<float*>(p.nlse2), p.batch, p.seqlen_q, p.heads, p.head_dim, lrows, a->o.stride_b, a->o.stride_l,
      a->o.stride_h, a->dout.stride_b, a->dout.stride_l, a->dout.stride_h);
  const int grid = p.num_tiles < sm_count ? p.num_tiles : sm_count;
  kernel<<<grid, kBwdStreamThreads, TR::kSmemBytes, stream>>>(p);
  convert<<<p.batch * p.heads * p.steps, 256, convert_smem, stream>>>(
      p.dq_acc, static_cast<T*>(a->dq.ptr), p.heads, p.head_dim, p.steps, a->dq.stride_b, a->dq.stride_l,
      a->dq.stride_h, p.scale);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

int run_bwd_stream(const dmf_attn_bwd_args* a, int tail, int sm_count) {
  const int B = a->batch, H = a->heads, D = a->head_dim, Lq = a->seqlen_q, Lk = a->seqlen_kv, dt = a->dtype;
  BwdStreamParams p;
  std::memset(&p, 0, sizeof(p));
  int st;
  const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_32B;  // tiles as blocks of 16 columns
  if ((st = make_map(&p.q, a->q, dt, B, Lq, H, D, 16, 128, sw)) != DMF_ATTN_OK) return st;
  if ((st = make_map(&p.dout, a->dout, dt, B, Lq, H, D, 16, 128, sw)) != DMF_ATTN_OK) return st;
  if ((st = make_map(&p.k, a->k, dt, B, Lk, H, D, 16, 128, sw)) != DMF_ATTN_OK) return st;
  if ((st = make_map(&p.v, a->v, dt, B, Lk, H, D, 16, 128, sw)) != DMF_ATTN_OK) return st;
  if ((st = make_map(&p.dk, a->dk, dt, B, Lk, H, D, 16, 128, sw)) != DMF_ATTN_OK) return st;
  if ((st = make_map(&p.dv, a->dv, dt, B, Lk, H, D, 16, 128, sw)) != DMF_ATTN_OK) return st;
  float* ws = static_cast<float*>(a->workspace);
  p.nlse2 = ws;
  p.ndelta = ws + static_cast<size_t>(B) * H * Lq;
  p.dq_acc = reinterpret_cast<float*>(static_cast<char*>(a->workspace) + bwd_stream_acc_offset(B, Lq, H));
  p.status_word = a->status_word;
  p.batch = B; p.heads = H; p.head_dim = D; p.seqlen_q = Lq; p.seqlen_kv = Lk;
  p.tiles_per_bh = Lk / 128;
  p.num_tiles = B * H * p.tiles_per_bh;
  p.steps = Lq / 128;
  p.scale = a->softmax_scale;
  p.scale_log2e = a->softmax_scale * 1.4426950408889634f;
  if (D == 72) {
    // head rows of 144 bytes straddle 32-byte sectors on every other head: let the kernel start its boxes 8 columns
    // early there (the tile has 80 columns).  Both tensors of a group must agree on the alignment pattern.
    auto pattern = [](const dmf_attn_tensor& t, int* out) -> bool {
      if ((t.stride_l * 2) % 32 != 0) return false;  // alignment must not change along the sequence
      out[0] = static_cast<int>(reinterpret_cast<uintptr_t>(t.ptr) & 31);
      out[1] = static_cast<int>((t.stride_b * 2) & 31);
      out[2] = static_cast<int>((t.stride_h * 2) & 31);
      return true;
    };
    const dmf_attn_tensor* pairs[2][2] = {{&a->q, &a->k}, {&a->v, &a->dout}};
    for (int g = 0; g < 2; ++g) {
      int ref[3] = {0, 0, 0}, cur[3] = {0, 0, 0};
      const bool same = pattern(*pairs[g][0], ref) && pattern(*pairs[g][1], cur) && cur[0] == ref[0] &&
                        cur[1] == ref[1] && cur[2] == ref[2];
      p.align_enable[g] = same ? 1 : 0;
      p.align0[g] = ref[0]; p.align_b[g] = ref[1]; p.align_h[g] = ref[2];
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  if (cudaMemsetAsync(p.dq_acc, 0, sizeof(float) * static_cast<size_t>(B) * H * Lq * D, stream) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_LAUNCH;
  }
  if (dt == DMF_ATTN_BF16)
    return tail == 0 ? launch_bwd_stream_inst<__nv_bfloat16, 0>(p, a, sm_count, stream)
                     : launch_bwd_stream_inst<__nv_bfloat16, 16>(p, a, sm_count, stream);
  return tail == 0 ? launch_bwd_stream_inst<__half, 0>(p, a, sm_count, stream)
                   : launch_bwd_stream_inst<__half, 16>(p, a, sm_count, stream);
}

void bwd_kernel_name(const char* t, int tail, int seqlen_q, int seqlen_kv, char* buf, size_t len) {
  if (bwd_uses_fused(tail, seqlen_q, seqlen_kv)) {
    std::snprintf(buf, len, "attn_bwd_fused_kernel<%s, TAIL=%d> (one pass, cluster of two CTAs per head)", t, tail);
    return;
  }
  if (bwd_stream_applies(tail, seqlen_q, seqlen_kv)) {
    std::snprintf(buf, len,
                  "bwd_delta_kernel<%s> + attn_bwd_stream_kernel<%s, TAIL=%d> (one pass, dQ by atomics) + "
                  "bwd_dq_convert_kernel<%s>",
                  t, t, tail, t);
    return;
  }
  const char* name = (tail <= 32 && bwd_split_enabled()) ? "attn_bwd_split_kernel" : "attn_bwd_kernel";
  std::snprintf(buf, len, "%s<%s, TAIL=%d, dQ> + %s<%s, TAIL=%d, dK/dV>", name, t, tail, name, t, tail);
}

int run_bwd(const dmf_attn_bwd_args* a) {
  int st = validate_bwd(a);
  if (st != DMF_ATTN_OK) return st;
  int sm_count = 0;
  if ((st = device_info(&sm_count)) != DMF_ATTN_OK) return st;
  const int tail = tail_of(a->head_dim);
  const int B = a->batch, H = a->heads, D = a->head_dim, Lq = a->seqlen_q, Lk = a->seqlen_kv, dt = a->dtype;
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  // two-tile sequences: the one-pass kernel (it needs no workspace; lse rows are fetched with 16-byte bulk copies)
  if (bwd_uses_fused(tail, Lq, Lk) && (reinterpret_cast<uintptr_t>(a->lse) & 15u) == 0)
    return run_bwd_fused(a, tail, sm_count);
  // long sequences at head_dim <= 80, when the workspace has room for the fp32 dQ accumulator: one pass
  if (bwd_stream_applies(tail, Lq, Lk) && a->workspace_bytes >= bwd_workspace_bytes(B, Lq, Lk, H, D) &&
      (reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0)
    return run_bwd_stream(a, tail, sm_count);

  BwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.o = a->o.ptr; p.o_sb = a->o.stride_b; p.o_sl = a->o.stride_l; p.o_sh = a->o.stride_h;
  p.dout = a->dout.ptr; p.do_sb = a->dout.stride_b; p.do_sl = a->dout.stride_l; p.do_sh = a->dout.stride_h;
  p.lse = a->lse;
  p.ws_neg_lse2 = static_cast<float*>(a->workspace);
  p.ws_delta = p.ws_neg_lse2 + static_cast<size_t>(B) * H * Lq;
  p.status_word = a->status_word;
  p.batch = B; p.heads = H; p.seqlen_q = Lq; p.seqlen_kv = Lk; p.head_dim = D;
  p.scale = a->softmax_scale;
  p.scale_log2e = a->softmax_scale * 1.4426950408889634f;

  // pass 1: dQ (query tiles resident, K/V streamed); also fills the workspace
  if ((st = make_map_pair(&p.r0_main, &p.r0_tail, a->q, dt, B, Lq, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.r1_main, &p.r1_tail, a->dout, dt, B, Lq, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.x0_main, &p.x0_tail, a->k, dt, B, Lk, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  if ((st = make_map_pair(&p.x1_main, &p.x1_tail, a->v, dt, B, Lk, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  p.out0 = a->dq.ptr; p.out0_sb = a->dq.stride_b; p.out0_sl = a->dq.stride_l; p.out0_sh = a->dq.stride_h;
  if (tail <= 32) {  // the role-split kernel loads o and stores its outputs through TMA
    if ((st = make_map_pair(&p.o_main, &p.o_tail, a->o, dt, B, Lq, H, D, tail, 128)) != DMF_ATTN_OK) return st;
    if ((st = make_map_pair(&p.out0_main, &p.out0_tail, a->dq, dt, B, Lq, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  }
  p.tiles_per_bh = Lq / 128;
  p.num_tiles = B * H * p.tiles_per_bh;
  p.inner_blocks = Lk / 128;
  int grid = p.num_tiles < sm_count ? p.num_tiles : sm_count;
  st = dt == DMF_ATTN_BF16 ? launch_bwd_tail<__nv_bfloat16, kModeDQ>(p, tail, grid, stream)
                           : launch_bwd_tail<__half, kModeDQ>(p, tail, grid, stream);
  if (st != DMF_ATTN_OK) return st;

  // pass 2: dK, dV (key tiles resident, Q/dO and the workspace rows streamed)
  BwdParams p2 = p;
  p2.r0_main = p.x0_main; p2.r0_tail = p.x0_tail; p2.r1_main = p.x1_main; p2.r1_tail = p.x1_tail;
  p2.x0_main = p.r0_main; p2.x0_tail = p.r0_tail; p2.x1_main = p.r1_main; p2.x1_tail = p.r1_tail;
  p2.out0 = a->dk.ptr; p2.out0_sb = a->dk.stride_b; p2.out0_sl = a->dk.stride_l; p2.out0_sh = a->dk.stride_h;
  p2.out1 = a->dv.ptr; p2.out1_sb = a->dv.stride_b; p2.out1_sl = a->dv.stride_l; p2.out1_sh = a->dv.stride_h;
  if (tail <= 32) {
    if ((st = make_map_pair(&p2.out0_main, &p2.out0_tail, a->dk, dt, B, Lk, H, D, tail, 128)) != DMF_ATTN_OK) return st;
    if ((st = make_map_pair(&p2.out1_main, &p2.out1_tail, a->dv, dt, B, Lk, H, D, tail, 128)) != DMF_ATTN_OK) return st;
  }
  p2.tiles_per_bh = Lk / 128;
  p2.num_tiles = B * H * p2.tiles_per_bh;
  p2.inner_blocks = Lq / 128;
  grid = p2.num_tiles < sm_count ? p2.num_tiles : sm_count;
  return dt == DMF_ATTN_BF16 ? launch_bwd_tail<__nv_bfloat16, kModeDKV>(p2, tail, grid, stream)
                             : launch_bwd_tail<__half, kModeDKV>(p2, tail, grid, stream);
}

// ---- backward without a caller-provided workspace ----

// Scratch of dmf_attn_bwd_static: -lse*log2(e) and delta for up to DMF_ATTN_STATIC_MAX_ROWS query
// rows.  In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_bwd_static_scratch[2 * DMF_ATTN_STATIC_MAX_ROWS];

struct StaticScratch {
  std::atomic<float*> ptr{nullptr};
};
StaticScratch g_static_scratch[kMaxDevices];

// Device address of the scratch array on the current device (looked up once per device).
int static_scratch_ptr(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_DEVICE;
  }
  StaticScratch& s = g_static_scratch[dev];
  float* ptr = s.ptr.load(std::memory_order_acquire);
  if (ptr == nullptr) {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_bwd_static_scratch) != cudaSuccess || addr == nullptr) {
      (void)cudaGetLastError();
      return DMF_ATTN_ERR_DEVICE;
    }
    ptr = static_cast<float*>(addr);  // first callers that race all look up, and store, the same address
    s.ptr.store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return DMF_ATTN_OK;
}

int run_bwd_static(const dmf_attn_bwd_args* a) {
  if (a == nullptr) return DMF_ATTN_ERR_NULL;
  int st = check_dims(a->batch, a->seqlen_q, a->seqlen_kv, a->heads, a->head_dim, a->dtype);
  if (st != DMF_ATTN_OK) return st;
  const int64_t rows = static_cast<int64_t>(a->batch) * a->heads * a->seqlen_q;
  if (rows > DMF_ATTN_STATIC_MAX_ROWS) return DMF_ATTN_ERR_TOO_LARGE;
  dmf_attn_bwd_args local = *a;
  local.workspace = reinterpret_cast<void*>(static_cast<uintptr_t>(256));  // placeholder for validation only
  local.workspace_bytes = sizeof(g_bwd_static_scratch);
  if ((st = validate_bwd(&local)) != DMF_ATTN_OK) return st;
  int sm_count = 0;
  if ((st = device_info(&sm_count)) != DMF_ATTN_OK) return st;
  float* scratch = nullptr;
  if ((st = static_scratch_ptr(&scratch)) != DMF_ATTN_OK) return st;
  local.workspace = scratch;
  // only the two rows per query: the call then never takes the one-pass long-sequence kernel, whose fp32 dQ
  // accumulator does not fit the scratch array for most shapes, and stays reproducible bit for bit
  local.workspace_bytes = bwd_workspace_min_bytes(a->batch, a->seqlen_q, a->heads);
  return run_bwd(&local);
}

// ---- self-test of the bounded wait ----

constexpr int kRoleSelftest = 900;

// One CTA, two waiting threads.  Thread 0 waits on a barrier that nobody ever arrives on: its wait must run
// out after `limit_cycles`, record kRoleSelftest + 1 in the status word and raise the CTA's abort flag.
// Thread 32 waits on a second such barrier with a limit 64 times as long: it must come back early, because
// it sees the abort flag.  Thread 64 arrives on a third barrier and then waits on it: that wait succeeds.
// result[0..2]: what the three waits returned; result[3]: cycles thread 0 waited.  The kernel holds no
// tensor memory and no copy in flight, and returns normally.
__global__ void selftest_wait_limit_kernel(long long limit_cycles, int32_t* status_word, int32_t* result) {
  __shared__ __align__(8) uint64_t bars[3];
  __shared__ int abort_flag_mem;
  volatile int* abort_flag = &abort_flag_mem;
  if (threadIdx.x == 0) {
    abort_flag_mem = 0;
    for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&bars[i]), 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = mbar_try_wait(smem_u32(&bars[0]), 0) ||
                    mbar_wait_slow(smem_u32(&bars[0]), 0, abort_flag, status_word, kRoleSelftest + 1, limit_cycles);
    const long long dt = clock64() - t0;
    result[0] = ok ? 1 : 0;
    result[3] = dt > 0x7fffffffll ? 0x7fffffff : static_cast<int32_t>(dt);
  } else if (threadIdx.x == 32) {
    const bool ok = mbar_try_wait(smem_u32(&bars[1]), 0) ||
                    mbar_wait_slow(smem_u32(&bars[1]), 0, abort_flag, status_word, kRoleSelftest + 2, 64 * limit_cycles);
    result[1] = ok ? 1 : 0;
  } else if (threadIdx.x == 64) {
    mbar_arrive(smem_u32(&bars[2]));
    const bool ok = mbar_try_wait(smem_u32(&bars[2]), 0) ||
                    mbar_wait_slow(smem_u32(&bars[2]), 0, abort_flag, status_word, kRoleSelftest + 3, limit_cycles);
    result[2] = ok ? 1 : 0;
  }
}

int run_selftest_wait_limit(int64_t limit_cycles, int32_t* status_word, int32_t* result, void* stream) {
  if (status_word == nullptr || result == nullptr) return DMF_ATTN_ERR_NULL;
  // between a few microseconds and the library's own limit: this call must end by itself, quickly
  if (limit_cycles < 1000 || limit_cycles > 50000000) return DMF_ATTN_ERR_SHAPE;
  int sm_count = 0;
  int st = device_info(&sm_count);
  if (st != DMF_ATTN_OK) return st;
  selftest_wait_limit_kernel<<<1, 96, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, status_word, result);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

// ---- name of the kernel a call would launch ----

int kernel_name(int op, int seqlen_q, int seqlen_kv, int head_dim, int dtype, char* buf, size_t len) {
  if (buf == nullptr || len == 0) return DMF_ATTN_ERR_NULL;
  if (dtype != DMF_ATTN_BF16 && dtype != DMF_ATTN_FP16) return DMF_ATTN_ERR_DTYPE;
  const int tail = tail_of(head_dim);
  if (tail < 0) return DMF_ATTN_ERR_HEAD_DIM;
  if (seqlen_q < kBlockQ || seqlen_kv < kBlockKV || seqlen_q % kBlockQ || seqlen_kv % kBlockKV) return DMF_ATTN_ERR_SEQLEN;
  const char* t = dtype == DMF_ATTN_BF16 ? "bf16" : "fp16";
  if (op == 0 || op == 1) {
    const char* kind = op == 0 ? "dual" : "plain";
    if (fwd_uses_pair(tail, seqlen_q)) {
      const bool is_short = tail == 16 && seqlen_kv <= kShortMaxBlocks * kBlockKV;
      std::snprintf(buf, len, "attn_fwd_pair_kernel<%s, TAIL=%d, %s%s> (cta_group::2 cluster pair)", t, tail, kind,
                    is_short ? ", short" : "");
    } else {
      std::snprintf(buf, len, "attn_fwd_kernel<%s, TAIL=%d, %s>", t, tail, kind);
    }
    return DMF_ATTN_OK;
  }
  if (op == 2) {
    bwd_kernel_name(t, tail, seqlen_q, seqlen_kv, buf, len);
    return DMF_ATTN_OK;
  }
  return DMF_ATTN_ERR_SHAPE;
}

// ---- per-head RMS norm (q / k) with tangent, and its backward ----

constexpr int kRmsMaxBlocks = 2048;  // upper bound of the grid, fixes the size of the backward's workspace

int rms_check(int batch, int seqlen, int heads, int d, int dtype) {
  if (dtype != DMF_ATTN_BF16 && dtype != DMF_ATTN_FP16) return DMF_ATTN_ERR_DTYPE;
  if (d < 8 || d > 128 || (d % 8) != 0) return DMF_ATTN_ERR_HEAD_DIM;
  if (batch < 1 || heads < 1 || seqlen < 1) return DMF_ATTN_ERR_SHAPE;
  if (static_cast<int64_t>(batch) * seqlen * heads >= (int64_t{1} << 31)) return DMF_ATTN_ERR_SHAPE;
  return DMF_ATTN_OK;
}

int rms_grid(int64_t rows, int head_dim, int unroll, int sm_count) {
  const int64_t block_rows = rms_rows_per_block(head_dim / 8, unroll);
  const int64_t want = (rows + block_rows - 1) / block_rows;
  int64_t cap = static_cast<int64_t>(sm_count) * 8;  // 8 blocks of 256 threads per SM
  if (cap > kRmsMaxBlocks) cap = kRmsMaxBlocks;
  return static_cast<int>(want < cap ? want : cap);
}

// the kernels are compiled per number of 16-byte chunks in a row (head_dim / 8 = 1..16)
template <typename T, typename Off, int C = 16>
void rms_launch_fwd(int chunks, bool dual, int grid, cudaStream_t stream, const RmsParams& p) {
  if (chunks == C) {
    if (dual) rmsnorm_fwd_kernel<T, C, true, Off><<<grid, kRmsThreads, 0, stream>>>(p);
    else rmsnorm_fwd_kernel<T, C, false, Off><<<grid, kRmsThreads, 0, stream>>>(p);
  } else if constexpr (C > 1) {
    rms_launch_fwd<T, Off, C - 1>(chunks, dual, grid, stream, p);
  }
}

template <typename T, typename Off, int C = 16>
void rms_launch_bwd(int chunks, int grid, cudaStream_t stream, const RmsParams& p) {
  if (chunks == C) rmsnorm_bwd_kernel<T, C, Off><<<grid, kRmsThreads, 0, stream>>>(p);
  else if constexpr (C > 1) rms_launch_bwd<T, Off, C - 1>(chunks, grid, stream, p);
}

// every element offset of the tensor fits 31 bits: the kernels can index it with 32-bit arithmetic
bool rms_small(const dmf_attn_tensor& t, int batch, int seqlen, int heads, int d) {
  if (t.ptr == nullptr) return true;
  const __int128 last = static_cast<__int128>(batch - 1) * t.stride_b + static_cast<__int128>(seqlen - 1) * t.stride_l +
                        static_cast<__int128>(heads - 1) * t.stride_h + d;
  return last < (static_cast<__int128>(1) << 31) && t.stride_b < (int64_t{1} << 31) && t.stride_l < (int64_t{1} << 31) &&
         t.stride_h < (int64_t{1} << 31);
}

int run_rmsnorm_fwd(const dmf_rmsnorm_args* a) {
  if (a == nullptr || a->weight == nullptr) return DMF_ATTN_ERR_NULL;
  int st = rms_check(a->batch, a->seqlen, a->heads, a->head_dim, a->dtype);
  if (st != DMF_ATTN_OK) return st;
  const bool dual = a->tx.ptr != nullptr;
  if ((st = check_tensor(a->x, 2)) != DMF_ATTN_OK || (st = check_tensor(a->y, 2)) != DMF_ATTN_OK) return st;
  if (dual && ((st = check_tensor(a->tx, 2)) != DMF_ATTN_OK || (st = check_tensor(a->ty, 2)) != DMF_ATTN_OK)) return st;
  int sm_count = 0;
  if ((st = device_info(&sm_count)) != DMF_ATTN_OK) return st;
  RmsParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = a->x.ptr; p.x_sb = a->x.stride_b; p.x_sl = a->x.stride_l; p.x_sh = a->x.stride_h;
  p.y = a->y.ptr; p.y_sb = a->y.stride_b; p.y_sl = a->y.stride_l; p.y_sh = a->y.stride_h;
  if (dual) {
    p.tx = a->tx.ptr; p.tx_sb = a->tx.stride_b; p.tx_sl = a->tx.stride_l; p.tx_sh = a->tx.stride_h;
    p.ty = a->ty.ptr; p.ty_sb = a->ty.stride_b; p.ty_sl = a->ty.stride_l; p.ty_sh = a->ty.stride_h;
  }
  p.w = a->weight;
  p.batch = a->batch; p.seqlen = a->seqlen; p.heads = a->heads; p.head_dim = a->head_dim;
  p.rows = static_cast<int64_t>(a->batch) * a->seqlen * a->heads;
  p.eps = a->eps;
  const int grid = rms_grid(p.rows, a->head_dim, rms_unroll_fwd(dual), sm_count);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  bool small = true;
  for (const dmf_attn_tensor* t : {&a->x, &a->tx, &a->y, &a->ty})
    small = small && rms_small(*t, a->batch, a->seqlen, a->heads, a->head_dim);
  const int chunks = a->head_dim / 8;
  if (a->dtype == DMF_ATTN_BF16) {
    if (small) rms_launch_fwd<__nv_bfloat16, int32_t>(chunks, dual, grid, stream, p);
    else rms_launch_fwd<__nv_bfloat16, int64_t>(chunks, dual, grid, stream, p);
  } else {
    if (small) rms_launch_fwd<__half, int32_t>(chunks, dual, grid, stream, p);
    else rms_launch_fwd<__half, int64_t>(chunks, dual, grid, stream, p);
  }
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

size_t rmsnorm_bwd_workspace_bytes(int d) {
  if (d < 8 || d > 128 || (d % 8) != 0) return 0;
  return static_cast<size_t>(kRmsMaxBlocks) * d * sizeof(float);
}

int run_rmsnorm_bwd(const dmf_rmsnorm_bwd_args* a) {
  if (a == nullptr || a->weight == nullptr || a->dweight == nullptr) return DMF_ATTN_ERR_NULL;
  int st = rms_check(a->batch, a->seqlen, a->heads, a->head_dim, a->dtype);
  if (st != DMF_ATTN_OK) return st;
  if ((st = check_tensor(a->dy, 2)) != DMF_ATTN_OK || (st = check_tensor(a->x, 2)) != DMF_ATTN_OK ||
      (st = check_tensor(a->dx, 2)) != DMF_ATTN_OK)
    return st;
  if (a->workspace == nullptr || a->workspace_bytes < rmsnorm_bwd_workspace_bytes(a->head_dim))
    return DMF_ATTN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 15u) != 0) return DMF_ATTN_ERR_ALIGN;
  int sm_count = 0;
  if ((st = device_info(&sm_count)) != DMF_ATTN_OK) return st;
  RmsParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = a->x.ptr; p.x_sb = a->x.stride_b; p.x_sl = a->x.stride_l; p.x_sh = a->x.stride_h;
  p.dy = a->dy.ptr; p.dy_sb = a->dy.stride_b; p.dy_sl = a->dy.stride_l; p.dy_sh = a->dy.stride_h;
  p.dx = a->dx.ptr; p.dx_sb = a->dx.stride_b; p.dx_sl = a->dx.stride_l; p.dx_sh = a->dx.stride_h;
  p.w = a->weight;
  p.dw_partial = static_cast<float*>(a->workspace);
  p.batch = a->batch; p.seqlen = a->seqlen; p.heads = a->heads; p.head_dim = a->head_dim;
  p.rows = static_cast<int64_t>(a->batch) * a->seqlen * a->heads;
  p.eps = a->eps;
  const int grid = rms_grid(p.rows, a->head_dim, kRmsUnrollBwd, sm_count);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  bool small = true;
  for (const dmf_attn_tensor* t : {&a->dy, &a->x, &a->dx})
    small = small && rms_small(*t, a->batch, a->seqlen, a->heads, a->head_dim);
  const int chunks = a->head_dim / 8;
  if (a->dtype == DMF_ATTN_BF16) {
    if (small) rms_launch_bwd<__nv_bfloat16, int32_t>(chunks, grid, stream, p);
    else rms_launch_bwd<__nv_bfloat16, int64_t>(chunks, grid, stream, p);
  } else {
    if (small) rms_launch_bwd<__half, int32_t>(chunks, grid, stream, p);
    else rms_launch_bwd<__half, int64_t>(chunks, grid, stream, p);
  }
  if (cudaGetLastError() != cudaSuccess) return DMF_ATTN_ERR_LAUNCH;
  rmsnorm_dw_reduce_kernel<<<(a->head_dim + 31) / 32, 1024, 0, stream>>>(p.dw_partial, a->dweight, grid, a->head_dim);
  return cudaGetLastError() == cudaSuccess ? DMF_ATTN_OK : DMF_ATTN_ERR_LAUNCH;
}

}  // namespace

#define DMF_API __attribute__((visibility("default")))

extern "C" {

DMF_API int dmf_attn_abi_version(void) { return DMF_ATTN_ABI_VERSION; }

DMF_API const char* dmf_attn_status_string(int status) {
  switch (status) {
    case DMF_ATTN_OK: return "ok";
    case DMF_ATTN_ERR_NULL: return "a required pointer is NULL";
    case DMF_ATTN_ERR_DTYPE: return "unsupported dtype (bf16 and fp16 only)";
    case DMF_ATTN_ERR_HEAD_DIM: return "unsupported head_dim (multiples of 8 in [64, 128])";
    case DMF_ATTN_ERR_SEQLEN: return "seqlen_q and seqlen_kv must be positive multiples of 128";
    case DMF_ATTN_ERR_SHAPE: return "bad batch / heads / scale";
    case DMF_ATTN_ERR_STRIDE: return "strides must be non-negative and a multiple of 16 bytes";
    case DMF_ATTN_ERR_ALIGN: return "base pointers must be 16-byte aligned";
    case DMF_ATTN_ERR_DEVICE: return "no usable sm_100 CUDA device";
    case DMF_ATTN_ERR_TENSOR_MAP: return "the driver rejected a TMA tensor map";
    case DMF_ATTN_ERR_LAUNCH: return "kernel launch failed";
    case DMF_ATTN_ERR_WORKSPACE: return "workspace missing or too small";
    case DMF_ATTN_ERR_TIMEOUT: return "a device-side wait ran out";
    case DMF_ATTN_ERR_TOO_LARGE: return "batch*heads*seqlen_q exceeds the built-in scratch of dmf_attn_bwd_static (1048576 rows)";
    default: return "unknown status";
  }
}

DMF_API int dmf_attn_fwd_dual(const dmf_attn_fwd_args* args) { return run_fwd(args, true); }

DMF_API int dmf_attn_fwd(const dmf_attn_fwd_args* args) { return run_fwd(args, false); }

DMF_API int dmf_attn_fwd_dual_f32out(const dmf_attn_fwd_args* args) { return run_fwd(args, true, true); }

DMF_API int dmf_attn_selftest_wait_limit(int64_t limit_cycles, int32_t* status_word, int32_t* result, void* stream) {
  return run_selftest_wait_limit(limit_cycles, status_word, result, stream);
}

#ifdef DMF_TRACE
// diagnostic builds only: copy the in-kernel timeline of the one-pass backward out (see attn_bwd_fused.cuh)
DMF_API int dmf_trace_read_bwd_fused(unsigned long long* out, size_t count) {
  const size_t have = sizeof(g_bwd_fused_trace) / sizeof(unsigned long long);
  if (cudaDeviceSynchronize() != cudaSuccess) return DMF_ATTN_ERR_DEVICE;
  if (cudaMemcpyFromSymbol(out, g_bwd_fused_trace, sizeof(unsigned long long) * (count < have ? count : have)) != cudaSuccess)
    return DMF_ATTN_ERR_DEVICE;
  return DMF_ATTN_OK;
}
#endif

DMF_API int dmf_attn_kernel_name(int32_t op, int32_t seqlen_q, int32_t seqlen_kv, int32_t head_dim, int32_t dtype,
                                 char* buf, size_t len) {
  return kernel_name(op, seqlen_q, seqlen_kv, head_dim, dtype, buf, len);
}

DMF_API int dmf_attn_validate_fwd(const dmf_attn_fwd_args* args, int dual) { return validate_fwd(args, dual != 0); }

DMF_API int dmf_attn_validate_bwd(const dmf_attn_bwd_args* args) { return validate_bwd(args); }

DMF_API int dmf_rmsnorm_fwd(const dmf_rmsnorm_args* args) { return run_rmsnorm_fwd(args); }

DMF_API size_t dmf_rmsnorm_bwd_workspace_bytes(int32_t head_dim) { return rmsnorm_bwd_workspace_bytes(head_dim); }

DMF_API int dmf_rmsnorm_bwd(const dmf_rmsnorm_bwd_args* args) { return run_rmsnorm_bwd(args); }

DMF_API size_t dmf_attn_bwd_workspace_bytes(int32_t batch, int32_t seqlen_q, int32_t seqlen_kv, int32_t heads,
                                    int32_t head_dim) {
  return bwd_workspace_bytes(batch, seqlen_q, seqlen_kv, heads, head_dim);
}

DMF_API int dmf_attn_bwd(const dmf_attn_bwd_args* args) { return run_bwd(args); }

DMF_API int dmf_attn_bwd_static(const dmf_attn_bwd_args* args) { return run_bwd_static(args); }

DMF_API int dmf_attn_check_status_word(const int32_t* status_word, void* stream, int32_t* raw) {
  if (status_word == nullptr) return DMF_ATTN_ERR_NULL;
  int32_t host = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&host, status_word, sizeof(host), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    (void)cudaGetLastError();
    return DMF_ATTN_ERR_DEVICE;
  }
  if (raw != nullptr) *raw = host;
  return host == 0 ? DMF_ATTN_OK : DMF_ATTN_ERR_TIMEOUT;
}

}  // extern "C"
