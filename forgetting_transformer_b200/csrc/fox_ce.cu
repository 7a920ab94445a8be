// Fused cross-entropy loss over a (rows, classes) logit matrix, forward and backward.  HBM-bound: the forward
// reads every logit once, the backward reads it once more and writes the gradient (in place if asked to).
//
// Stands in for upstream's Triton kernels cross_entropy_fwd_kernel / cross_entropy_bwd_kernel
// (src/forgetting_transformer/model/forgetting_transformer/fused_cross_entropy.py:24-134) behind
// FusedCrossEntropyLoss, as the model's loss uses it (modeling_forgetting_transformer.py:877-884,
// inplace_backward=True, reduction='none'):
//
//   z      = logit_scale * logits[row, :]                       (fp32)
//   lse    = log sum_c exp(z_c)
//   loss   = lse - (1 - eps) z_label - eps mean_c z_c + lse_square_scale lse^2        (0 where label == ignore_index)
//   z_loss = lse_square_scale lse^2                                                    (0 where label == ignore_index)
//   dlogits_c = dloss logit_scale ( exp(z_c - lse) (1 + 2 lse_square_scale lse) - (1 - eps) [c == label] - eps / C )
//
// With the classes split over ranks (upstream lines 150-151, 196-226: every rank holds n_cols of C = world * n_cols
// classes, starting at class_start) the forward writes the rank's own lse and the part of the loss that does not
// need the global one, -(1 - eps) z_label [label on this rank] - eps sum_c z_c / C; the host joins the ranks' lse
// (log-sum-exp of an all-gather), sums the parts and adds the global lse; the backward takes the global lse.
//
// One CTA per row.  Forward: every thread runs an online (maximum, sum) pair over its 16-byte pieces of the row
// (and the plain sum of the logits when label smoothing is on); the pairs are merged through shuffles and shared
// memory.  Logits are fp32, bf16 or fp16; the row stride is in elements and the rows must be 16-byte aligned.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int kCeThreads = 512;

template <int kDtype>   // 0 fp16, 1 bf16, 2 fp32
struct CeVec;
template <>
struct CeVec<2> {
  static constexpr int kElems = 4;
  __device__ static void load(const void* base, int64_t i, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + i);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  __device__ static void store(void* base, int64_t i, const float* f) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + i) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __device__ static float load1(const void* base, int64_t i) { return reinterpret_cast<const float*>(base)[i]; }
  __device__ static void store1(void* base, int64_t i, float v) { reinterpret_cast<float*>(base)[i] = v; }
};
template <int kDtype>
struct CeVec {
  static constexpr bool kBf16 = kDtype == 1;
  static constexpr int kElems = 8;
  __device__ static void load(const void* base, int64_t i, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2<kBf16>(w[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
  }
  __device__ static void store(void* base, int64_t i, const float* f) {
    uint4 v;
    v.x = pack2<kBf16>(f[0], f[1]);
    v.y = pack2<kBf16>(f[2], f[3]);
    v.z = pack2<kBf16>(f[4], f[5]);
    v.w = pack2<kBf16>(f[6], f[7]);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + i) = v;
  }
  __device__ static float load1(const void* base, int64_t i) {
    const uint32_t w = reinterpret_cast<const uint16_t*>(base)[i];
    return unpack2<kBf16>(w).x;
  }
  __device__ static void store1(void* base, int64_t i, float v) {
    reinterpret_cast<uint16_t*>(base)[i] = static_cast<uint16_t>(pack2<kBf16>(v, 0.f) & 0xffffu);
  }
};

// (m, s) <- merge of two online pairs: sum of exp(z - m)
__device__ __forceinline__ void ce_merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
  m = mn;
}

template <int kDtype>
__global__ void __launch_bounds__(kCeThreads)
fox_ce_fwd_kernel(const void* __restrict__ logits, int64_t row_stride, const int64_t* __restrict__ labels,
                  float* __restrict__ losses, float* __restrict__ z_losses, float* __restrict__ lse_out,
                  int64_t n_cols, float label_smoothing, float logit_scale, float lse_square_scale,
                  int64_t ignore_index, int64_t total_classes, int64_t class_start, int split) {
  using V = CeVec<kDtype>;
  constexpr int E = V::kElems;
  const int64_t row = blockIdx.x;
  const char* base = reinterpret_cast<const char*>(logits) + row * row_stride * (kDtype == 2 ? 4 : 2);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float m = -INFINITY, s = 0.f, tot = 0.f;
  const int64_t n_vec = n_cols / E;
  for (int64_t i = tid; i < n_vec; i += kCeThreads) {
    float f[E];
    V::load(base, i * E, f);
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      f[j] *= logit_scale;
      mx = fmaxf(mx, f[j]);
      tot += f[j];
    }
    const float mn = fmaxf(m, mx);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) acc += __expf(f[j] - mn);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + acc;
    m = mn;
  }
  for (int64_t c = n_vec * E + tid; c < n_cols; c += kCeThreads) {   // ragged end of the row
    const float z = V::load1(base, c) * logit_scale;
    tot += z;
    ce_merge(m, s, z, 1.f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    tot += __shfl_xor_sync(0xffffffffu, tot, o);
    ce_merge(m, s, m2, s2);
  }
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32], st[kCeThreads / 32];
  if (lane == 0) { sm[warp] = m; ss[warp] = s; st[warp] = tot; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kCeThreads / 32; ++w) {
      ce_merge(m, s, sm[w], ss[w]);
      tot += st[w];
    }
    const float lse = logf(s) + m;
    lse_out[row] = lse;
    const int64_t label = labels[row];
    const int64_t local = label - class_start;     // index among this rank's classes
    const bool mine = label != ignore_index && local >= 0 && local < n_cols;
    const float n_all = static_cast<float>(total_classes);
    float loss = 0.f, zl = 0.f;
    if (label != ignore_index && split) {
      // the part of the loss that needs no global lse (upstream lines 84-92)
      const float zlab = mine ? V::load1(base, local) * logit_scale : 0.f;
      loss = (label_smoothing > 0.f ? -label_smoothing * tot / n_all : 0.f) - (mine ? (1.f - label_smoothing) * zlab : 0.f);
    } else if (label != ignore_index) {
      if (mine) {
        const float zlab = V::load1(base, local) * logit_scale;
        loss = label_smoothing > 0.f ? lse - label_smoothing * tot / n_all - (1.f - label_smoothing) * zlab
                                     : lse - zlab;
      } else {   // a label outside the classes contributes only the smoothing term (upstream lines 74-78)
        loss = label_smoothing > 0.f ? label_smoothing * (lse - tot / n_all) : 0.f;
      }
      zl = lse_square_scale * lse * lse;
      loss += zl;
    }
    losses[row] = loss;
    if (z_losses) z_losses[row] = zl;
  }
}

template <int kDtype>
__global__ void __launch_bounds__(kCeThreads)
fox_ce_bwd_kernel(const void* __restrict__ logits, int64_t row_stride, const int64_t* __restrict__ labels,
                  const float* __restrict__ lse_in, const float* __restrict__ dloss, int64_t dloss_stride,
                  void* __restrict__ dlogits, int64_t d_row_stride, int64_t n_cols, float label_smoothing,
                  float logit_scale, float lse_square_scale, int64_t ignore_index, int64_t total_classes,
                  int64_t class_start) {
  using V = CeVec<kDtype>;
  constexpr int E = V::kElems;
  constexpr int kBytes = kDtype == 2 ? 4 : 2;
  const int64_t row = blockIdx.x;
  const char* base = reinterpret_cast<const char*>(logits) + row * row_stride * kBytes;
  char* dbase = reinterpret_cast<char*>(dlogits) + row * d_row_stride * kBytes;
  const int tid = threadIdx.x;
  const int64_t label_all = labels[row];
  const int64_t label = label_all - class_start;   // index among this rank's classes (outside [0, n_cols): none)
  const float dl = (label_all != ignore_index) ? dloss[row * dloss_stride] : 0.f;
  const float lse = lse_in[row];
  const float pscale = 1.f + 2.f * lse_square_scale * lse;
  const float g = dl * logit_scale;
  const float smooth_neg = label_smoothing / static_cast<float>(total_classes);
  const float at_label = 1.f - label_smoothing;
  const int64_t n_vec = n_cols / E;
  for (int64_t i = tid; i < n_vec; i += kCeThreads) {
    float f[E];
    V::load(base, i * E, f);
#pragma unroll
    for (int j = 0; j < E; ++j) {
      float pr = __expf(f[j] * logit_scale - lse) * pscale;
      if (i * E + j == label) pr -= at_label;
      f[j] = g * (pr - smooth_neg);
    }
    V::store(dbase, i * E, f);
  }
  for (int64_t c = n_vec * E + tid; c < n_cols; c += kCeThreads) {
    float pr = __expf(V::load1(base, c) * logit_scale - lse) * pscale;
    if (c == label) pr -= at_label;
    V::store1(dbase, c, g * (pr - smooth_neg));
  }
}

}  // namespace fox

static int ce_dtype_index(int dtype) {
  return dtype == FOX_DTYPE_FP16 ? 0 : dtype == FOX_DTYPE_BF16 ? 1 : dtype == FOX_DTYPE_FP32 ? 2 : -1;
}

static int ce_fwd_launch(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols, const void* logits,
                         int64_t row_stride, const int64_t* labels, float label_smoothing, float logit_scale,
                         float lse_square_scale, int64_t ignore_index, int64_t total_classes, int64_t class_start,
                         int split, float* losses, float* z_losses, float* lse) {
  using namespace fox;
  const int di = ce_dtype_index(dtype);
  if (!logits || !labels || !losses || (!z_losses && !split) || !lse || n_rows <= 0 || n_cols <= 0 || di < 0)
    return FOX_ERR_BAD_ARG;
  if (total_classes < n_cols || class_start < 0 || class_start + n_cols > total_classes) return FOX_ERR_BAD_ARG;
  if (n_rows > 2147483647LL) return FOX_ERR_TOO_LARGE;
  const int bytes = di == 2 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(logits) % 16 || (row_stride * bytes) % 16 || row_stride < n_cols) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(n_rows);
#define FOX_CE_FWD(DT)                                                                                              \
  fox_ce_fwd_kernel<DT><<<grid, kCeThreads, 0, st>>>(logits, row_stride, labels, losses, z_losses, lse, n_cols,       \
                                                     label_smoothing, logit_scale, lse_square_scale, ignore_index,   \
                                                     total_classes, class_start, split)
  if (di == 0) FOX_CE_FWD(0);
  else if (di == 1) FOX_CE_FWD(1);
  else FOX_CE_FWD(2);
#undef FOX_CE_FWD
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

static int ce_bwd_launch(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols, const void* logits,
                         int64_t row_stride, const int64_t* labels, const float* lse, const float* dloss,
                         int64_t dloss_stride, float label_smoothing, float logit_scale, float lse_square_scale,
                         int64_t ignore_index, int64_t total_classes, int64_t class_start, void* dlogits,
                         int64_t dlogits_row_stride) {
  using namespace fox;
  const int di = ce_dtype_index(dtype);
  if (!logits || !labels || !lse || !dloss || !dlogits || n_rows <= 0 || n_cols <= 0 || di < 0) return FOX_ERR_BAD_ARG;
  if (total_classes < n_cols || class_start < 0 || class_start + n_cols > total_classes) return FOX_ERR_BAD_ARG;
  if (n_rows > 2147483647LL) return FOX_ERR_TOO_LARGE;
  const int bytes = di == 2 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(logits) % 16 || (row_stride * bytes) % 16 || row_stride < n_cols ||
      reinterpret_cast<uintptr_t>(dlogits) % 16 || (dlogits_row_stride * bytes) % 16 || dlogits_row_stride < n_cols)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(n_rows);
#define FOX_CE_BWD(DT)                                                                                              \
  fox_ce_bwd_kernel<DT><<<grid, kCeThreads, 0, st>>>(logits, row_stride, labels, lse, dloss, dloss_stride, dlogits,   \
                                                     dlogits_row_stride, n_cols, label_smoothing, logit_scale,       \
                                                     lse_square_scale, ignore_index, total_classes, class_start)
  if (di == 0) FOX_CE_BWD(0);
  else if (di == 1) FOX_CE_BWD(1);
  else FOX_CE_BWD(2);
#undef FOX_CE_BWD
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

extern "C" int fox_cross_entropy_fwd(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols,
                                     const void* logits, int64_t row_stride, const int64_t* labels,
                                     float label_smoothing, float logit_scale, float lse_square_scale,
                                     int64_t ignore_index, float* losses, float* z_losses, float* lse) {
  return ce_fwd_launch(device, stream, dtype, n_rows, n_cols, logits, row_stride, labels, label_smoothing, logit_scale,
                       lse_square_scale, ignore_index, n_cols, 0, 0, losses, z_losses, lse);
}

extern "C" int fox_cross_entropy_bwd(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols,
                                     const void* logits, int64_t row_stride, const int64_t* labels, const float* lse,
                                     const float* dloss, int64_t dloss_stride, float label_smoothing,
                                     float logit_scale, float lse_square_scale, int64_t ignore_index, void* dlogits,
                                     int64_t dlogits_row_stride) {
  return ce_bwd_launch(device, stream, dtype, n_rows, n_cols, logits, row_stride, labels, lse, dloss, dloss_stride,
                       label_smoothing, logit_scale, lse_square_scale, ignore_index, n_cols, 0, dlogits,
                       dlogits_row_stride);
}

extern "C" int fox_cross_entropy_fwd_split(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols,
                                           const void* logits, int64_t row_stride, const int64_t* labels,
                                           float label_smoothing, float logit_scale, int64_t ignore_index,
                                           int64_t total_classes, int64_t class_start, float* loss_parts,
                                           float* lse_local) {
  // (the z-loss needs the global lse: the host forms it)
  return ce_fwd_launch(device, stream, dtype, n_rows, n_cols, logits, row_stride, labels, label_smoothing, logit_scale,
                       0.f, ignore_index, total_classes, class_start, 1, loss_parts, nullptr, lse_local);
}

extern "C" int fox_cross_entropy_bwd_split(int device, void* stream, int dtype, int64_t n_rows, int64_t n_cols,
                                           const void* logits, int64_t row_stride, const int64_t* labels,
                                           const float* lse_global, const float* dloss, int64_t dloss_stride,
                                           float label_smoothing, float logit_scale, float lse_square_scale,
                                           int64_t ignore_index, int64_t total_classes, int64_t class_start,
                                           void* dlogits, int64_t dlogits_row_stride) {
  return ce_bwd_launch(device, stream, dtype, n_rows, n_cols, logits, row_stride, labels, lse_global, dloss,
                       dloss_stride, label_smoothing, logit_scale, lse_square_scale, ignore_index, total_classes,
                       class_start, dlogits, dlogits_row_stride);
}
