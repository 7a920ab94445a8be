// Data-dependent token shift of the FoX-Pro key/value projections, forward and backward.
// HBM-bound: every element is read once (the previous token's row comes from L1/L2) and written once.
//
// Stands in for upstream's Triton `shift_fwd_kernel` / `shift_bwd_kernel`
// (src/forgetting_transformer/model/forgetting_transformer/token_shift.py:21-80, 82-157), called by
// ShiftLinear (modeling_forgetting_transformer.py:44-95) as token_shift(x, alpha, 1 - alpha):
//
//   forward : out[b,t,h,:] = x[b,t,h,:] curr[b,t,h] + x[b,t-1,h,:] prev[b,t,h]      (x[b,-1] = 0)
//   backward: dx[b,t,h,:]  = dout[b,t,h,:] curr[b,t,h] + dout[b,t+1,h,:] prev[b,t+1,h]
//             dcurr[b,t,h] = sum_d dout[b,t,h,d] x[b,t,h,d];  dprev[b,t,h] = sum_d dout[b,t,h,d] x[b,t-1,h,d]
//
// x, out, dout, dx: (B,T,H,D) 16-bit, unit stride on D, arbitrary element strides on B, T, H (all four share
// them, as upstream asserts); prev, curr, dprev, dcurr: (B,T,H) fp32 sharing one set of strides.  The two
// products and their sum are separate fp32 operations (no fused multiply-add) and the result is rounded once,
// which reproduces upstream's kernels in Triton's interpreter bit for bit.  Thread = 8 channels of one (b,t,h) row; the D/8
// lanes of a row are neighbours in a warp, so the two weight gradients are a shuffle reduction.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

template <bool kBf16>
__device__ __forceinline__ void shift_load8(const uint16_t* p, float* f) {
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
__device__ __forceinline__ void shift_store8(uint16_t* p, const float* f) {
  uint4 v;
  v.x = pack2<kBf16>(f[0], f[1]);
  v.y = pack2<kBf16>(f[2], f[3]);
  v.z = pack2<kBf16>(f[4], f[5]);
  v.w = pack2<kBf16>(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

struct ShiftParams {
  int64_t B, T, H;
  int D;
  int64_t x_sb, x_st, x_sh;  // element strides of x / out / dout / dx
  int64_t w_sb, w_st, w_sh;  // element strides of the four weight tensors
};

template <bool kBf16>
__global__ void __launch_bounds__(256)
fox_token_shift_fwd_kernel(const uint16_t* __restrict__ x, const float* __restrict__ prev, const float* __restrict__ curr,
                           uint16_t* __restrict__ out, const ShiftParams p) {
  const int lanes = p.D >> 3;
  const int rows_per_block = 256 / lanes;
  const int sub = threadIdx.x % lanes;
  const int64_t n_rows = p.B * p.T * p.H;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_block + threadIdx.x / lanes; row < n_rows;
       row += static_cast<int64_t>(gridDim.x) * rows_per_block) {
    // (b, t, h) of the row with 32-bit divisions (the launcher rejects more than 2^31 rows): 64-bit ones cost
    // more instructions than the row's arithmetic
    const uint32_t r32 = static_cast<uint32_t>(row), H32 = static_cast<uint32_t>(p.H), T32 = static_cast<uint32_t>(p.T);
    const uint32_t q32 = r32 / H32;
    const int64_t h = r32 - q32 * H32, b = q32 / T32, t = q32 - static_cast<uint32_t>(b) * T32;
    const int64_t xo = b * p.x_sb + t * p.x_st + h * p.x_sh + sub * 8;
    const int64_t wo = b * p.w_sb + t * p.w_st + h * p.w_sh;
    float xv[8], xp[8], o[8];
    shift_load8<kBf16>(x + xo, xv);
    if (t > 0) {
      shift_load8<kBf16>(x + xo - p.x_st, xp);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) xp[j] = 0.f;
    }
    const float cw = curr[wo], pw = prev[wo];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __fadd_rn(__fmul_rn(xv[j], cw), __fmul_rn(xp[j], pw));  // two products, one sum: no contraction
    shift_store8<kBf16>(out + xo, o);
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
fox_token_shift_bwd_kernel(const uint16_t* __restrict__ x, const float* __restrict__ prev, const float* __restrict__ curr,
                           const uint16_t* __restrict__ dout, uint16_t* __restrict__ dx, float* __restrict__ dprev,
                           float* __restrict__ dcurr, const ShiftParams p) {
  const int lanes = p.D >> 3;
  const int rows_per_block = 256 / lanes;
  const int sub = threadIdx.x % lanes;
  const int64_t n_rows = p.B * p.T * p.H;
  // every lane runs the same number of iterations (the shuffles need the whole warp)
  const int64_t n_iter = (n_rows + static_cast<int64_t>(gridDim.x) * rows_per_block - 1) /
                         (static_cast<int64_t>(gridDim.x) * rows_per_block);
  for (int64_t it = 0; it < n_iter; ++it) {
    const int64_t row = (it * gridDim.x + blockIdx.x) * rows_per_block + threadIdx.x / lanes;
    const bool in = row < n_rows;
    const int64_t rc = in ? row : 0;
    const uint32_t r32 = static_cast<uint32_t>(rc), H32 = static_cast<uint32_t>(p.H), T32 = static_cast<uint32_t>(p.T);
    const uint32_t q32 = r32 / H32;
    const int64_t h = r32 - q32 * H32, b = q32 / T32, t = q32 - static_cast<uint32_t>(b) * T32;
    const int64_t xo = b * p.x_sb + t * p.x_st + h * p.x_sh + sub * 8;
    const int64_t wo = b * p.w_sb + t * p.w_st + h * p.w_sh;
    float xv[8], xp[8], dv[8], dn[8], o[8];
    shift_load8<kBf16>(x + xo, xv);
    shift_load8<kBf16>(dout + xo, dv);
    if (t > 0) {
      shift_load8<kBf16>(x + xo - p.x_st, xp);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) xp[j] = 0.f;
    }
    float pw_next = 0.f;
    if (t + 1 < p.T) {
      shift_load8<kBf16>(dout + xo + p.x_st, dn);
      pw_next = prev[wo + p.w_st];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) dn[j] = 0.f;
    }
    const float cw = curr[wo];
    float sc = 0.f, sp = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j] = __fadd_rn(__fmul_rn(dv[j], cw), __fmul_rn(dn[j], pw_next));
      sc = fmaf(dv[j], xv[j], sc);
      sp = fmaf(dv[j], xp[j], sp);
    }
    for (int off = lanes >> 1; off > 0; off >>= 1) {
      sc += __shfl_xor_sync(0xffffffffu, sc, off);
      sp += __shfl_xor_sync(0xffffffffu, sp, off);
    }
    if (in) {
      shift_store8<kBf16>(dx + xo, o);
      if (sub == 0) {
        dcurr[wo] = sc;
        dprev[wo] = sp;
      }
    }
  }
}

static int shift_check(int64_t B, int64_t T, int64_t H, int64_t D, int64_t x_sb, int64_t x_st, int64_t x_sh,
                       std::initializer_list<const void*> ptrs16) {
  if (B <= 0 || T <= 0 || H <= 0) return FOX_ERR_BAD_ARG;
  if (B * T > (int64_t{1} << 31) / H) return FOX_ERR_TOO_LARGE;              // rows are indexed with 32 bits
  if (D != 16 && D != 32 && D != 64 && D != 128) return FOX_ERR_HEAD_DIM;  // token_shift.py:166
  if (x_sb % 8 || x_st % 8 || x_sh % 8) return FOX_ERR_ALIGNMENT;           // 16-byte rows
  for (const void* q : ptrs16)
    if (!q || reinterpret_cast<uintptr_t>(q) % 16) return q ? FOX_ERR_ALIGNMENT : FOX_ERR_BAD_ARG;
  return FOX_OK;
}

}  // namespace fox

using namespace fox;

extern "C" int fox_token_shift_fwd(int device, void* stream, int dtype, int64_t B, int64_t T, int64_t H, int64_t D,
                                   const void* x, int64_t x_sb, int64_t x_st, int64_t x_sh, const float* prev_weight,
                                   const float* curr_weight, int64_t w_sb, int64_t w_st, int64_t w_sh, void* out) {
  if (!prev_weight || !curr_weight) return FOX_ERR_BAD_ARG;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (int rc = shift_check(B, T, H, D, x_sb, x_st, x_sh, {x, out})) return rc;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const ShiftParams p{B, T, H, (int)D, x_sb, x_st, x_sh, w_sb, w_st, w_sh};
  const int64_t rows_per_block = 256 / (D / 8);
  const int64_t blocks = (B * T * H + rows_per_block - 1) / rows_per_block;
  const unsigned grid = (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
  if (dtype == FOX_DTYPE_BF16)
    fox_token_shift_fwd_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, prev_weight, curr_weight, (uint16_t*)out, p);
  else
    fox_token_shift_fwd_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, prev_weight, curr_weight, (uint16_t*)out, p);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

extern "C" int fox_token_shift_bwd(int device, void* stream, int dtype, int64_t B, int64_t T, int64_t H, int64_t D,
                                   const void* x, int64_t x_sb, int64_t x_st, int64_t x_sh, const float* prev_weight,
                                   const float* curr_weight, int64_t w_sb, int64_t w_st, int64_t w_sh, const void* dout,
                                   void* dx, float* dprev_weight, float* dcurr_weight) {
  if (!prev_weight || !curr_weight || !dprev_weight || !dcurr_weight) return FOX_ERR_BAD_ARG;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (int rc = shift_check(B, T, H, D, x_sb, x_st, x_sh, {x, dout, dx})) return rc;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const ShiftParams p{B, T, H, (int)D, x_sb, x_st, x_sh, w_sb, w_st, w_sh};
  const int64_t rows_per_block = 256 / (D / 8);
  const int64_t blocks = (B * T * H + rows_per_block - 1) / rows_per_block;
  const unsigned grid = (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
  if (dtype == FOX_DTYPE_BF16)
    fox_token_shift_bwd_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, prev_weight, curr_weight, (const uint16_t*)dout, (uint16_t*)dx, dprev_weight, dcurr_weight, p);
  else
    fox_token_shift_bwd_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, prev_weight, curr_weight, (const uint16_t*)dout, (uint16_t*)dx, dprev_weight, dcurr_weight, p);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}
