// Fused per-head RMSNorm + sigmoid output gate of the FoX-Pro layer, forward and
// backward.  HBM-bound: every element is read once and written once.
//
// Stands in for upstream's Triton `layer_norm_gated_fwd_kernel` /
// `layer_norm_gated_bwd_kernel` in the configuration the FoX layer uses
// (is_rms_norm, activation "sigmoid", weight, no bias, no residual):
// src/forgetting_transformer/model/forgetting_transformer/fuse_norm_gate.py:132-206, 309-421.
//
//   forward : rstd = (mean_d x^2 + eps)^-1/2 ;  y = x rstd w_h sigmoid(g)
//   backward: s = sigmoid(g); xhat = x rstd; dg = dy (xhat w) s (1-s); dy' = dy s;
//             dw_h += dy' xhat;  dx = (w dy' - xhat mean_d(xhat w dy')) rstd
//
// With g == NULL the gate is left out (y = x rstd w_h; no dg): the per-head RMSNorm that the FoX layer
// applies to q and k ("QK-norm", GroupNorm(num_groups=H, is_rms_norm=True) at
// modeling_forgetting_transformer.py:264-265, 314-316; Triton kernels at layernorm.py:183-245, 328-423).
//
// Layout: x, g, y, dy, dx, dg are contiguous (tokens, G*D) 16-bit arrays, w is
// (G*D) fp32, rstd is (tokens*G) fp32.  A CTA covers whole tokens: thread
// (h, sub) owns the 8 consecutive channels [h*D + 8 sub, +8) of every token the
// CTA visits, so its loads are 16-byte and coalesced across the CTA, the
// per-head reduction is a shuffle over D/8 neighbouring lanes, and its slice of
// dw stays in registers until the end.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

// 1 / (1 + e^-x) with the approximate reciprocal (2 ulp in fp32, far below a 16-bit ulp): an IEEE division here
// made the forward kernel instruction-bound (37 instructions per element, issue slots 69 % busy at 3 TB/s)
__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

template <bool kBf16>
__device__ __forceinline__ void load8(const uint16_t* p, float* f) {
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
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack2<kBf16>(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <bool kBf16>
__device__ __forceinline__ void store8(uint16_t* p, const float* f) {
  uint4 v;
  v.x = pack2<kBf16>(f[0], f[1]);
  v.y = pack2<kBf16>(f[2], f[3]);
  v.z = pack2<kBf16>(f[4], f[5]);
  v.w = pack2<kBf16>(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

template <bool kBf16, bool kGate>
__global__ void fox_normgate_fwd_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ g,
                                        const float* __restrict__ w, uint16_t* __restrict__ y,
                                        float* __restrict__ rstd, int64_t tokens, int G, int D, float eps) {
  const int lanes = D >> 3;
  const int tid = threadIdx.x;
  const int h = tid / lanes, sub = tid % lanes;
  const bool active = h < G;
  const int ch = active ? h * D + sub * 8 : 0;
  float wv[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) wv[j] = active ? w[ch + j] : 0.f;
  const int64_t GD = static_cast<int64_t>(G) * D;
  const float inv_d = 1.f / static_cast<float>(D);
  // kU tokens per iteration, their 16-byte loads issued (and kept packed) before the first reduction: with one
  // token per iteration a warp has 512 B in flight and the kernel is latency-bound
  constexpr int kU = 4;
  for (int64_t t0 = blockIdx.x; t0 < tokens; t0 += static_cast<int64_t>(kU) * gridDim.x) {
    uint4 xr[kU], gr[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t t = t0 + static_cast<int64_t>(u) * gridDim.x;
      xr[u] = gr[u] = make_uint4(0, 0, 0, 0);
      if (active && t < tokens) {
        xr[u] = *reinterpret_cast<const uint4*>(x + t * GD + ch);
        if (kGate) gr[u] = *reinterpret_cast<const uint4*>(g + t * GD + ch);
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t t = t0 + static_cast<int64_t>(u) * gridDim.x;
      float xv[8], gv[8];
      unpack8<kBf16>(xr[u], xv);
      if (kGate) unpack8<kBf16>(gr[u], gv);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(xv[j], xv[j], ss);
      for (int o = lanes >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss * inv_d + eps);
      if (active && t < tokens) {
        float out[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) out[j] = kGate ? xv[j] * r * wv[j] * sigmoidf_fast(gv[j]) : xv[j] * r * wv[j];
        store8<kBf16>(y + t * GD + ch, out);
        if (sub == 0) rstd[t * G + h] = r;
      }
    }
  }
}

template <bool kBf16, bool kGate>
__global__ void fox_normgate_bwd_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ g,
                                        const float* __restrict__ w, const float* __restrict__ rstd,
                                        const uint16_t* __restrict__ dy, uint16_t* __restrict__ dx,
                                        uint16_t* __restrict__ dg, float* __restrict__ dw_partial, int64_t tokens,
                                        int G, int D) {
  const int lanes = D >> 3;
  const int tid = threadIdx.x;
  const int h = tid / lanes, sub = tid % lanes;
  const bool active = h < G;
  const int ch = active ? h * D + sub * 8 : 0;
  float wv[8], dwv[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    wv[j] = active ? w[ch + j] : 0.f;
    dwv[j] = 0.f;
  }
  const int64_t GD = static_cast<int64_t>(G) * D;
  const float inv_d = 1.f / static_cast<float>(D);
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    float xv[8], gv[8], dyv[8];
    float r = 0.f;
    if (active) {
      load8<kBf16>(x + t * GD + ch, xv);
      if (kGate) load8<kBf16>(g + t * GD + ch, gv);
      load8<kBf16>(dy + t * GD + ch, dyv);
      r = rstd[t * G + h];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) xv[j] = gv[j] = dyv[j] = 0.f;
    }
    float xhat[8], wdy[8], dgv[8];
    float c1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = kGate ? sigmoidf_fast(gv[j]) : 1.f;
      xhat[j] = xv[j] * r;
      const float yv = xhat[j] * wv[j];
      dgv[j] = dyv[j] * yv * s * (1.f - s);
      const float dy2 = dyv[j] * s;
      wdy[j] = dy2 * wv[j];
      dwv[j] = fmaf(dy2, xhat[j], dwv[j]);
      c1 = fmaf(xhat[j], wdy[j], c1);
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) c1 += __shfl_xor_sync(0xffffffffu, c1, o);
    c1 *= inv_d;
    if (active) {
      float dxv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) dxv[j] = (wdy[j] - xhat[j] * c1) * r;
      store8<kBf16>(dx + t * GD + ch, dxv);
      if (kGate) store8<kBf16>(dg + t * GD + ch, dgv);
    }
  }
  if (active) {
    float* dst = dw_partial + static_cast<int64_t>(blockIdx.x) * GD + ch;
    *reinterpret_cast<float4*>(dst) = make_float4(dwv[0], dwv[1], dwv[2], dwv[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(dwv[4], dwv[5], dwv[6], dwv[7]);
  }
}

static inline int normgate_threads(int64_t G, int64_t D) {
  const int64_t n = G * (D / 8);
  return static_cast<int>((n + 31) / 32 * 32);
}

}  // namespace fox

using namespace fox;

extern "C" int fox_normgate_fwd(int device, void* stream, int dtype, int64_t tokens, int64_t G, int64_t D,
                                const void* x, const void* g, const float* w, float eps, void* y, float* rstd) {
  if (!x || !w || !y || !rstd || tokens <= 0 || G <= 0) return FOX_ERR_BAD_ARG;
  if (D % 8 || D < 8 || D > 256 || (D & (D - 1))) return FOX_ERR_HEAD_DIM;
  const int threads = normgate_threads(G, D);
  if (threads > 1024) return FOX_ERR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(y)) % 16)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const int64_t grid = tokens < 148 * 16 ? tokens : 148 * 16;
#define FOX_NG_FWD(BF, GATE)                                                                      \
  fox_normgate_fwd_kernel<BF, GATE><<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>(          \
      (const uint16_t*)x, (const uint16_t*)g, w, (uint16_t*)y, rstd, tokens, (int)G, (int)D, eps)
  if (dtype == FOX_DTYPE_BF16) {
    if (g) FOX_NG_FWD(true, true); else FOX_NG_FWD(true, false);
  } else {
    if (g) FOX_NG_FWD(false, true); else FOX_NG_FWD(false, false);
  }
#undef FOX_NG_FWD
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

extern "C" int fox_normgate_bwd(int device, void* stream, int dtype, int64_t tokens, int64_t G, int64_t D,
                                const void* x, const void* g, const float* w, const float* rstd, const void* dy,
                                void* dx, void* dg, float* dw_partial, int64_t n_partials) {
  if (!x || !w || !rstd || !dy || !dx || !dw_partial || tokens <= 0 || G <= 0 || n_partials <= 0)
    return FOX_ERR_BAD_ARG;
  if ((g == nullptr) != (dg == nullptr)) return FOX_ERR_BAD_ARG;
  if (D % 8 || D < 8 || D > 256 || (D & (D - 1))) return FOX_ERR_HEAD_DIM;
  const int threads = normgate_threads(G, D);
  if (threads > 1024) return FOX_ERR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(dy) |
       reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dg) | reinterpret_cast<uintptr_t>(dw_partial)) % 16)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
#define FOX_NG_BWD(BF, GATE)                                                                          \
  fox_normgate_bwd_kernel<BF, GATE><<<(unsigned)n_partials, threads, 0, (cudaStream_t)stream>>>(        \
      (const uint16_t*)x, (const uint16_t*)g, w, rstd, (const uint16_t*)dy, (uint16_t*)dx, (uint16_t*)dg, \
      dw_partial, tokens, (int)G, (int)D)
  if (dtype == FOX_DTYPE_BF16) {
    if (g) FOX_NG_BWD(true, true); else FOX_NG_BWD(true, false);
  } else {
    if (g) FOX_NG_BWD(false, true); else FOX_NG_BWD(false, false);
  }
#undef FOX_NG_BWD
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}
