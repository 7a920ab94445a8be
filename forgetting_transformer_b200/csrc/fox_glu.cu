// SwiGLU elementwise kernels of the FoX MLP, forward and backward.  HBM-bound.
//
// Stand in for upstream's jiterator functions swiglu_fwd / swiglu_bwd / swiglu_bwd_with_output
// (src/forgetting_transformer/model/forgetting_transformer/glu_linear.py:64-92), used by SwiGLUFunction and
// SwiGLULinearFunction (glu_linear.py:95-146) behind ForgettingTransformerMLP (modeling_forgetting_transformer.py:505-516):
//
//   forward : z = x sigmoid(x) y
//   backward: s = sigmoid(x);  dx = s (1 + x (1 - s)) g y;  dy = x s g;  optionally z again (the linear layer
//             behind it does not keep z)
//
// All tensors are (rows, cols) 16-bit with unit inner stride and their own row stride (elements), so the two
// halves of a packed (rows, 2 cols) projection output, and of its gradient, are addressed in place.  Arithmetic
// in fp32, one rounding per output, as upstream's functions do.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

template <bool kBf16>
__device__ __forceinline__ void glu_load8(const uint16_t* p, float* f) {
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
__device__ __forceinline__ void glu_store8(uint16_t* p, const float* f) {
  uint4 v;
  v.x = pack2<kBf16>(f[0], f[1]);
  v.y = pack2<kBf16>(f[2], f[3]);
  v.z = pack2<kBf16>(f[4], f[5]);
  v.w = pack2<kBf16>(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
fox_swiglu_fwd_kernel(const uint16_t* __restrict__ x, int64_t x_sr, const uint16_t* __restrict__ y, int64_t y_sr,
                      uint16_t* __restrict__ z, int64_t z_sr, int64_t rows, int64_t cols) {
  const int64_t vec_per_row = cols >> 3;
  const int64_t n = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t r = i / vec_per_row, c = (i % vec_per_row) << 3;
    float xv[8], yv[8], o[8];
    glu_load8<kBf16>(x + r * x_sr + c, xv);
    glu_load8<kBf16>(y + r * y_sr + c, yv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __fdividef(xv[j] * yv[j], 1.0f + __expf(-xv[j]));   // approximate reciprocal: 2 ulp in fp32
    glu_store8<kBf16>(z + r * z_sr + c, o);
  }
}

template <bool kBf16, bool kWithZ>
__global__ void __launch_bounds__(256)
fox_swiglu_bwd_kernel(const uint16_t* __restrict__ x, int64_t x_sr, const uint16_t* __restrict__ y, int64_t y_sr,
                      const uint16_t* __restrict__ g, int64_t g_sr, uint16_t* __restrict__ dx, int64_t dx_sr,
                      uint16_t* __restrict__ dy, int64_t dy_sr, uint16_t* __restrict__ z, int64_t z_sr, int64_t rows,
                      int64_t cols) {
  const int64_t vec_per_row = cols >> 3;
  const int64_t n = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t r = i / vec_per_row, c = (i % vec_per_row) << 3;
    float xv[8], yv[8], gv[8], ox[8], oy[8], oz[8];
    glu_load8<kBf16>(x + r * x_sr + c, xv);
    glu_load8<kBf16>(y + r * y_sr + c, yv);
    glu_load8<kBf16>(g + r * g_sr + c, gv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = __fdividef(1.0f, 1.0f + __expf(-xv[j]));
      const float sw = xv[j] * s;
      ox[j] = s * (1.0f + xv[j] * (1.0f - s)) * gv[j] * yv[j];
      oy[j] = sw * gv[j];
      oz[j] = sw * yv[j];
    }
    glu_store8<kBf16>(dx + r * dx_sr + c, ox);
    glu_store8<kBf16>(dy + r * dy_sr + c, oy);
    if (kWithZ) glu_store8<kBf16>(z + r * z_sr + c, oz);
  }
}

static int glu_check(int64_t rows, int64_t cols, std::initializer_list<const void*> ptrs,
                     std::initializer_list<int64_t> strides) {
  if (rows <= 0 || cols <= 0 || cols % 8) return FOX_ERR_BAD_ARG;
  for (const void* p : ptrs)
    if (!p || reinterpret_cast<uintptr_t>(p) % 16) return p ? FOX_ERR_ALIGNMENT : FOX_ERR_BAD_ARG;
  for (int64_t s : strides)
    if (s % 8 || s < cols) return FOX_ERR_ALIGNMENT;
  return FOX_OK;
}
static unsigned glu_grid(int64_t rows, int64_t cols) {
  const int64_t blocks = (rows * (cols / 8) + 255) / 256;
  return (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
}

}  // namespace fox

using namespace fox;

extern "C" int fox_swiglu_fwd(int device, void* stream, int dtype, int64_t rows, int64_t cols, const void* x,
                              int64_t x_row_stride, const void* y, int64_t y_row_stride, void* z, int64_t z_row_stride) {
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (int rc = glu_check(rows, cols, {x, y, z}, {x_row_stride, y_row_stride, z_row_stride})) return rc;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const unsigned grid = glu_grid(rows, cols);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FOX_DTYPE_BF16)
    fox_swiglu_fwd_kernel<true><<<grid, 256, 0, st>>>((const uint16_t*)x, x_row_stride, (const uint16_t*)y, y_row_stride, (uint16_t*)z, z_row_stride, rows, cols);
  else
    fox_swiglu_fwd_kernel<false><<<grid, 256, 0, st>>>((const uint16_t*)x, x_row_stride, (const uint16_t*)y, y_row_stride, (uint16_t*)z, z_row_stride, rows, cols);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

extern "C" int fox_swiglu_bwd(int device, void* stream, int dtype, int64_t rows, int64_t cols, const void* x,
                              int64_t x_row_stride, const void* y, int64_t y_row_stride, const void* g,
                              int64_t g_row_stride, void* dx, int64_t dx_row_stride, void* dy, int64_t dy_row_stride,
                              void* z, int64_t z_row_stride) {
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (int rc = glu_check(rows, cols, {x, y, g, dx, dy}, {x_row_stride, y_row_stride, g_row_stride, dx_row_stride, dy_row_stride}))
    return rc;
  if (z && (reinterpret_cast<uintptr_t>(z) % 16 || z_row_stride % 8 || z_row_stride < cols)) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const unsigned grid = glu_grid(rows, cols);
  cudaStream_t st = (cudaStream_t)stream;
#define FOX_GLU_BWD(BF, WZ)                                                                                          \
  fox_swiglu_bwd_kernel<BF, WZ><<<grid, 256, 0, st>>>((const uint16_t*)x, x_row_stride, (const uint16_t*)y, y_row_stride, \
                                                     (const uint16_t*)g, g_row_stride, (uint16_t*)dx, dx_row_stride,  \
                                                     (uint16_t*)dy, dy_row_stride, (uint16_t*)z, z_row_stride, rows, cols)
  if (dtype == FOX_DTYPE_BF16) {
    if (z) FOX_GLU_BWD(true, true); else FOX_GLU_BWD(true, false);
  } else {
    if (z) FOX_GLU_BWD(false, true); else FOX_GLU_BWD(false, false);
  }
#undef FOX_GLU_BWD
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}
