// Row-wise RMSNorm with optional residual add, forward and backward: the FoX block's input norms
// (attn_norm(x); mlp_norm(x, residual, prenorm=True), modeling_forgetting_transformer.py:565, 580).
// HBM-bound: every element is read once and written once.
//
// Stands in for upstream's Triton layer_norm_fwd_kernel1 / layer_norm_bwd kernels with IS_RMS_NORM, a
// weight, no bias (src/forgetting_transformer/model/forgetting_transformer/layernorm.py:248-325, 328-423;
// host functions 426-520, LayerNormFunction 523-620):
//
//   forward : z = x + residual (fp32; residual optional); residual_out = z rounded (optional);
//             rstd = (mean z^2 + eps)^-1/2;  y = z rstd w
//   backward: xhat = z rstd; wdy = w dy; dx = (wdy - xhat mean(xhat wdy)) rstd + dresidual_in;
//             dw += dy xhat   (z is the saved, rounded residual_out, or x when there was no residual)
//
// Layout: rows of `hidden` 16-bit elements, contiguous; w (hidden) fp32; rstd (rows) fp32.  One warp per
// row, lane l owns the 16-byte vectors l, l+32, ... (VPL per lane, hidden = 256 VPL): coalesced loads, a
// shuffle reduction per row, the row stays in registers between the reduction and the store.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

template <bool kBf16>
__device__ __forceinline__ void rn_load8(const uint16_t* p, float* f) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack2<kBf16>(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <bool kBf16>
__device__ __forceinline__ void rn_store8(uint16_t* p, const float* f) {
  uint4 v;
  v.x = pack2<kBf16>(f[0], f[1]);
  v.y = pack2<kBf16>(f[2], f[3]);
  v.z = pack2<kBf16>(f[4], f[5]);
  v.w = pack2<kBf16>(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

constexpr int kRnWarps = 8;  // rows per CTA pass

template <bool kBf16, int VPL>
__global__ void __launch_bounds__(kRnWarps * 32)
fox_rmsnorm_fwd_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ res, const float* __restrict__ w,
                       uint16_t* __restrict__ y, uint16_t* __restrict__ res_out, float* __restrict__ rstd,
                       int64_t rows, float eps) {
  constexpr int hidden = 256 * VPL;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.f / static_cast<float>(hidden);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRnWarps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kRnWarps) {
    float z[VPL][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int64_t off = row * hidden + (v * 32 + lane) * 8;
      rn_load8<kBf16>(x + off, z[v]);
      if (res) {
        float r[8];
        rn_load8<kBf16>(res + off, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) z[v][j] += r[j];
      }
      if (res_out) rn_store8<kBf16>(res_out + off, z[v]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(z[v][j], z[v][j], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = 1.f / sqrtf(ss * inv_h + eps);
    if (lane == 0) rstd[row] = r;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int col = (v * 32 + lane) * 8;
      const float4 w0 = *reinterpret_cast<const float4*>(w + col), w1 = *reinterpret_cast<const float4*>(w + col + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = z[v][j] * r * wv[j];
      rn_store8<kBf16>(y + row * hidden + col, o);
    }
  }
}

template <bool kBf16, int VPL>
__global__ void __launch_bounds__(kRnWarps * 32)
fox_rmsnorm_bwd_kernel(const uint16_t* __restrict__ z_saved, const float* __restrict__ w, const float* __restrict__ rstd,
                       const uint16_t* __restrict__ dy, const uint16_t* __restrict__ dres_in, uint16_t* __restrict__ dx,
                       float* __restrict__ dw_partial, int64_t rows) {
  constexpr int hidden = 256 * VPL;
  __shared__ float s_dw[kRnWarps][32 * 8 + 8];  // one vector column at a time, padded against bank conflicts
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.f / static_cast<float>(hidden);
  float dwv[VPL][8];
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwv[v][j] = 0.f;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRnWarps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kRnWarps) {
    const float r = rstd[row];
    float xhat[VPL][8], wdy[VPL][8];
    float c1 = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int col = (v * 32 + lane) * 8;
      const int64_t off = row * hidden + col;
      float zz[8], d[8];
      rn_load8<kBf16>(z_saved + off, zz);
      rn_load8<kBf16>(dy + off, d);
      const float4 w0 = *reinterpret_cast<const float4*>(w + col), w1 = *reinterpret_cast<const float4*>(w + col + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xhat[v][j] = zz[j] * r;
        wdy[v][j] = wv[j] * d[j];
        dwv[v][j] = fmaf(d[j], xhat[v][j], dwv[v][j]);
        c1 = fmaf(xhat[v][j], wdy[v][j], c1);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c1 += __shfl_xor_sync(0xffffffffu, c1, o);
    c1 *= inv_h;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int64_t off = row * hidden + (v * 32 + lane) * 8;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (wdy[v][j] - xhat[v][j] * c1) * r;
      if (dres_in) {
        float dr[8];
        rn_load8<kBf16>(dres_in + off, dr);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += dr[j];
      }
      rn_store8<kBf16>(dx + off, o);
    }
  }
  // per-CTA weight-gradient partial: sum the warps' registers through shared memory, one vector column at a time
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) s_dw[warp][lane * 8 + j] = dwv[v][j];
    __syncthreads();
    for (int e = threadIdx.x; e < 256; e += kRnWarps * 32) {
      float acc = 0.f;
#pragma unroll
      for (int q = 0; q < kRnWarps; ++q) acc += s_dw[q][e];
      dw_partial[static_cast<int64_t>(blockIdx.x) * hidden + v * 256 + e] = acc;
    }
  }
}

template <bool kBf16, int VPL>
static int rn_launch_fwd(cudaStream_t st, unsigned grid, const void* x, const void* res, const float* w, void* y,
                         void* res_out, float* rstd, int64_t rows, float eps) {
  fox_rmsnorm_fwd_kernel<kBf16, VPL><<<grid, kRnWarps * 32, 0, st>>>((const uint16_t*)x, (const uint16_t*)res, w,
                                                                    (uint16_t*)y, (uint16_t*)res_out, rstd, rows, eps);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}
template <bool kBf16, int VPL>
static int rn_launch_bwd(cudaStream_t st, unsigned grid, const void* z, const float* w, const float* rstd,
                         const void* dy, const void* dres_in, void* dx, float* dw_partial, int64_t rows) {
  fox_rmsnorm_bwd_kernel<kBf16, VPL><<<grid, kRnWarps * 32, 0, st>>>((const uint16_t*)z, w, rstd, (const uint16_t*)dy,
                                                                    (const uint16_t*)dres_in, (uint16_t*)dx, dw_partial, rows);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

// hidden sizes built: 256 x {1, 2, 3, 4, 5, 6, 8} (a row's fp32 working set has to fit one warp's registers)
#define FOX_RN_DISPATCH(FN, BF, ...)                                 \
  switch (hidden / 256) {                                            \
    case 1: return FN<BF, 1>(__VA_ARGS__);                           \
    case 2: return FN<BF, 2>(__VA_ARGS__);                           \
    case 3: return FN<BF, 3>(__VA_ARGS__);                           \
    case 4: return FN<BF, 4>(__VA_ARGS__);                           \
    case 5: return FN<BF, 5>(__VA_ARGS__);                           \
    case 6: return FN<BF, 6>(__VA_ARGS__);                           \
    case 8: return FN<BF, 8>(__VA_ARGS__);                           \
    default: return FOX_ERR_HEAD_DIM;                                \
  }

static bool rn_hidden_ok(int64_t hidden) {
  if (hidden <= 0 || hidden % 256) return false;
  const int64_t v = hidden / 256;
  return v == 1 || v == 2 || v == 3 || v == 4 || v == 5 || v == 6 || v == 8;
}

}  // namespace fox

using namespace fox;

extern "C" int fox_rmsnorm_fwd(int device, void* stream, int dtype, int64_t rows, int64_t hidden, const void* x,
                               const void* residual, const float* w, float eps, void* y, void* residual_out,
                               float* rstd) {
  if (!x || !w || !y || !rstd || rows <= 0) return FOX_ERR_BAD_ARG;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (!rn_hidden_ok(hidden)) return FOX_ERR_HEAD_DIM;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(y) |
       reinterpret_cast<uintptr_t>(residual_out) | reinterpret_cast<uintptr_t>(w)) % 16)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const int64_t blocks = (rows + kRnWarps - 1) / kRnWarps;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FOX_DTYPE_BF16) {
    FOX_RN_DISPATCH(rn_launch_fwd, true, st, grid, x, residual, w, y, residual_out, rstd, rows, eps)
  } else {
    FOX_RN_DISPATCH(rn_launch_fwd, false, st, grid, x, residual, w, y, residual_out, rstd, rows, eps)
  }
}

extern "C" int fox_rmsnorm_bwd(int device, void* stream, int dtype, int64_t rows, int64_t hidden, const void* z,
                               const float* w, const float* rstd, const void* dy, const void* dresidual_in, void* dx,
                               float* dw_partial, int64_t n_partials) {
  if (!z || !w || !rstd || !dy || !dx || !dw_partial || rows <= 0 || n_partials <= 0) return FOX_ERR_BAD_ARG;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (!rn_hidden_ok(hidden)) return FOX_ERR_HEAD_DIM;
  if ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dresidual_in) |
       reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(w)) % 16)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const unsigned grid = (unsigned)n_partials;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FOX_DTYPE_BF16) {
    FOX_RN_DISPATCH(rn_launch_bwd, true, st, grid, z, w, rstd, dy, dresidual_in, dx, dw_partial, rows)
  } else {
    FOX_RN_DISPATCH(rn_launch_bwd, false, st, grid, z, w, rstd, dy, dresidual_in, dx, dw_partial, rows)
  }
}
