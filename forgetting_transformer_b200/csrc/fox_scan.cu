// HBM-bound helpers around the attention kernels: log-gate prefix sum with the
// seq_start masking folded in, block-pruning index scans, reverse prefix sum
// for the gate gradient, max row norms for the automatic threshold, the
// delta = rowsum(O * dO) pre-pass and the fp32 -> 16-bit dQ conversion.
//
// Upstream counterparts (src/forgetting_transformer/ops/forgetting_attention.py):
//   masked clone + torch.cumsum ............ lines 117-127
//   _find_start_index_kernel ............... lines 695-745
//   _find_end_index_kernel ................. lines 747-795
//   _bwd_preprocess ........................ lines 902-943
//   reverse cumsum of dlog_lambda .......... lines 390-392
//   vector_norm(...).max(...) .............. lines 95-96
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

// ------------------------------------------------------------------ block scan
constexpr int kScanThreads = 1024;
constexpr int kScanPerThread = 4;
constexpr int kScanChunk = kScanThreads * kScanPerThread;

// inclusive scan of one value per thread across the CTA; returns the inclusive
// prefix and (via total) the CTA total.  red[] holds 32 floats.
__device__ __forceinline__ float block_inclusive_scan(float v, float* red, float& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = red[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    red[lane] = w;
  }
  __syncthreads();
  const float prefix = warp > 0 ? red[warp - 1] : 0.f;
  total = red[31];
  __syncthreads();
  return v + prefix;
}

// One gate value: kIn = 3 reads an fp32 log gate; kIn = 0 / 1 / 2 reads an fp16 / bf16 / fp32 gate LOGIT and
// returns log sigmoid(x) = min(x, 0) - log1p(exp(-|x|)) in fp32 (the F.logsigmoid(fgate_logit.float()) of
// upstream's layer, modeling_forgetting_transformer.py:343-346).
template <int kIn>
__device__ __forceinline__ float load_gate(const void* base, int64_t idx) {
  if constexpr (kIn == 3) {
    return reinterpret_cast<const float*>(base)[idx];
  } else {
    float x;
    if constexpr (kIn == 2) x = reinterpret_cast<const float*>(base)[idx];
    else x = unpack2<kIn == 1>(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(base)[idx])).x;
    return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
  }
}

// log_lambda[b,h,t] = carry_in[b,h] + sum_{u<=t, u>=seq_start[b]} log_fgate[b,h,u]
// One CTA per (b,h); chunks of 4096 elements with a carried running total.  With gate logits as input
// (kIn < 3) the log gates themselves are formed on the fly and, if lf_out is given, written out (unmasked).
template <int kIn>
__global__ void __launch_bounds__(kScanThreads)
fox_cumsum_kernel(const void* __restrict__ lf, int64_t sb, int64_t sh, int64_t sn,
                  const int64_t* __restrict__ seq_start, const float* __restrict__ carry_in,
                  float* __restrict__ out, float* __restrict__ total_out, float* __restrict__ lf_out, int H, int N) {
  __shared__ float red[32];
  const int bh = blockIdx.x, b = bh / H, h = bh % H;
  const int64_t src0 = b * sb + h * sh;
  float* dst = out + static_cast<int64_t>(bh) * N;
  const int s0 = seq_start ? static_cast<int>(seq_start[b]) : 0;
  float carry = carry_in ? carry_in[bh] : 0.f;
  for (int base = 0; base < N; base += kScanChunk) {
    const int t0 = base + threadIdx.x * kScanPerThread;
    float x[kScanPerThread];
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
      const int t = t0 + j;
      float g = 0.f;
      if (t < N && (t >= s0 || (kIn < 3 && lf_out))) g = load_gate<kIn>(lf, src0 + static_cast<int64_t>(t) * sn);
      if (kIn < 3 && lf_out && t < N) lf_out[static_cast<int64_t>(bh) * N + t] = g;
      x[j] = (t < N && t >= s0) ? g : 0.f;
    }
#pragma unroll
    for (int j = 1; j < kScanPerThread; ++j) x[j] += x[j - 1];
    float total;
    const float incl = block_inclusive_scan(x[kScanPerThread - 1], red, total);
    const float excl = incl - x[kScanPerThread - 1] + carry;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
      const int t = t0 + j;
      if (t < N) dst[t] = x[j] + excl;
    }
    carry += total;
  }
  if (total_out && threadIdx.x == 0) total_out[bh] = carry;
}

// dlog_fgate[t] = carry_in + sum_{u >= t} (dcol[u] + drow[u - P] if u >= P)
// Reverse inclusive scan, one CTA per (b,h).  kIn < 3: the chain rule through log sigmoid is applied on the way
// out, dlogit[t] = dlog_fgate[t] * sigmoid(-logit[t]), written in the logits' dtype with the logits' strides.
template <int kIn>
__global__ void __launch_bounds__(kScanThreads)
fox_revcumsum_kernel(const float* __restrict__ dcol, const float* __restrict__ drow,
                     const float* __restrict__ carry_in, float* __restrict__ out,
                     float* __restrict__ total_out, int M, int N, const void* __restrict__ logit,
                     void* __restrict__ dlogit, int64_t sb, int64_t sh, int64_t sn, int H) {
  __shared__ float red[32];
  const int bh = blockIdx.x;
  const float* c = dcol + static_cast<int64_t>(bh) * N;
  const float* r = drow ? drow + static_cast<int64_t>(bh) * M : nullptr;
  float* dst = out + static_cast<int64_t>(bh) * N;
  const int P = N - M;
  float carry = carry_in ? carry_in[bh] : 0.f;
  // walk chunks from the right; inside a chunk index i runs right-to-left
  for (int base = 0; base < N; base += kScanChunk) {
    const int i0 = base + threadIdx.x * kScanPerThread;
    float x[kScanPerThread];
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
      const int t = N - 1 - (i0 + j);
      float v = 0.f;
      if (t >= 0) {
        v = c[t];
        if (r && t >= P) v += r[t - P];
      }
      x[j] = v;
    }
#pragma unroll
    for (int j = 1; j < kScanPerThread; ++j) x[j] += x[j - 1];
    float total;
    const float incl = block_inclusive_scan(x[kScanPerThread - 1], red, total);
    const float excl = incl - x[kScanPerThread - 1] + carry;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
      const int t = N - 1 - (i0 + j);
      if (t >= 0) {
        const float gsum = x[j] + excl;
        if constexpr (kIn == 3) {
          dst[t] = gsum;
        } else {
          const int64_t idx = static_cast<int64_t>(bh / H) * sb + static_cast<int64_t>(bh % H) * sh + static_cast<int64_t>(t) * sn;
          float xl;
          if constexpr (kIn == 2) xl = reinterpret_cast<const float*>(logit)[idx];
          else xl = unpack2<kIn == 1>(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(logit)[idx])).x;
          const float dl = gsum / (1.f + expf(xl));     // d/dx log sigmoid(x) = sigmoid(-x)
          if constexpr (kIn == 2) reinterpret_cast<float*>(dlogit)[idx] = dl;
          else reinterpret_cast<uint16_t*>(dlogit)[idx] = static_cast<uint16_t>(pack2<kIn == 1>(dl, 0.f) & 0xffffu);
        }
      }
    }
    carry += total;
  }
  if (total_out && threadIdx.x == 0) total_out[bh] = carry;
}

// ------------------------------------------------------------ pruning indices
// One CTA per (b,h).  The scans only look at log_lambda on block boundaries, so
// those values are staged in shared memory and one thread replays upstream's
// carried sequential scan on them (bit-identical decisions, no dependent global
// loads).  start != nullptr: start_index (B,H,ceil(M/BM)); end != nullptr:
// end_index (B,H,ceil(N/BN)).
__global__ void __launch_bounds__(256)
fox_find_index_kernel(const float* __restrict__ lam, const float* __restrict__ thr, int64_t thr_sb,
                      int64_t thr_sh, int64_t* __restrict__ start, int64_t* __restrict__ end, int H, int M,
                      int N, int BM, int BN, int nmb, int nnb) {
  extern __shared__ float sm[];
  float* row_first = sm;        // lam[P + mb*BM]            (nmb)
  float* col_last = sm + nmb;   // lam[min(N-1, nb*BN+BN-1)] (nnb)
  float* row_e = col_last + nnb;  // lam[min(mb*BM, M-1)], mb in [0, nmb]  (nmb + 1)
  const int bh = blockIdx.x, b = bh / H, h = bh % H;
  const float* l = lam + static_cast<int64_t>(bh) * N;
  const int P = N - M;
  for (int i = threadIdx.x; i < nmb; i += blockDim.x) row_first[i] = l[P + i * BM];
  for (int i = threadIdx.x; i < nnb; i += blockDim.x) col_last[i] = l[min(N - 1, i * BN + BN - 1)];
  for (int i = threadIdx.x; i <= nmb; i += blockDim.x) row_e[i] = l[min(min(i * BM, M), M - 1)];
  __syncthreads();
  const float t = thr[b * thr_sb + h * thr_sh];
  if (threadIdx.x == 0 && start) {
    int64_t* dst = start + static_cast<int64_t>(bh) * nmb;
    int s = 0;  // in blocks of BN
    for (int mb = 0; mb < nmb; ++mb) {
      const float lo = row_first[mb];
      // upstream: while (lo - lam[min(N-1, s+BN-1)] < thr) s += BN.  Past the last
      // block the clamped column stays N-1, which is col_last[nnb-1].
      int guard = 0;
      while (lo - col_last[min(s, nnb - 1)] < t && guard < nnb + 2) {
        ++s;
        if (s >= nnb) ++guard;
      }
      dst[mb] = static_cast<int64_t>(s) * BN;
    }
  }
  if (threadIdx.x == 32 && end) {
    int64_t* dst = end + static_cast<int64_t>(bh) * nnb;
    int e = 0;  // row index, multiple of BM or M
    for (int nb = 0; nb < nnb; ++nb) {
      const float li = col_last[nb];
      while (e < M) {
        const int eb = (e + BM - 1) / BM;  // e is k*BM (eb = k) or M (eb = nmb, handled by e < M)
        if (!(row_e[eb] - li >= t)) break;
        e = min(e + BM, M);
      }
      dst[nb] = e;
    }
  }
}

// ----------------------------------------------------------- max row L2 norm
// out[b,h] = max_t ||x[b,h,t,:]||_2 as fp32 (the caller rounds to the input dtype,
// which commutes with the max).  out must be zero-initialised; the maximum is
// taken with an integer atomicMax on the non-negative float bit pattern.
template <bool kBf16>
__global__ void __launch_bounds__(256)
fox_max_row_norm_kernel(const uint16_t* __restrict__ x, int64_t sb, int64_t sh, int64_t st, int H, int T, int D,
                        float* __restrict__ out) {
  const int lanes_per_row = D / 8;              // one 16-byte load per lane
  const int rows_per_block = 256 / lanes_per_row;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int sub = threadIdx.x % lanes_per_row;
  const int r_in = threadIdx.x / lanes_per_row;
  const uint16_t* base = x + b * sb + h * sh;
  float best = 0.f;
  // every lane runs the same number of iterations (the shuffles below need the full warp)
  // four rows per iteration with their loads issued first; the maximum is taken over the squared norms and the
  // square root once at the end (sqrt is monotone and correctly rounded: same result as the maximum of the roots)
  constexpr int kU = 4;
  for (int t0 = blockIdx.x * rows_per_block; t0 < T; t0 += kU * gridDim.x * rows_per_block) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int t = t0 + u * gridDim.x * rows_per_block + r_in;
      v[u] = make_uint4(0, 0, 0, 0);
      if (t < T) v[u] = *reinterpret_cast<const uint4*>(base + static_cast<int64_t>(t) * st + sub * 8);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack2<kBf16>(w[j]);
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
      }
      for (int o = lanes_per_row / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      best = fmaxf(best, acc);
    }
  }
  best = sqrtf(best);
  for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out + bh), __float_as_int(best));
}

// ------------------------------------------------------ delta = rowsum(O * dO)
// D / 8 lanes share a row (16 bytes each); a thread takes kDeltaRows rows a block-stride apart and issues all
// its loads before using any (two loads per thread left the kernel at a third of the copy rate).
constexpr int kDeltaRows = 4;
template <bool kBf16>
__global__ void __launch_bounds__(256)
fox_delta_kernel(const uint16_t* __restrict__ o, int64_t o_sb, int64_t o_sh, int64_t o_st,
                 const uint16_t* __restrict__ d_o, int64_t d_sb, int64_t d_sh, int64_t d_st, int H, int M, int D,
                 float* __restrict__ delta) {
  const int lanes_per_row = D / 8;
  const int rows_per_pass = 256 / lanes_per_row;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int sub = threadIdx.x % lanes_per_row;
  const int row0 = blockIdx.x * rows_per_pass * kDeltaRows + threadIdx.x / lanes_per_row;
  const uint16_t* ob = o + b * o_sb + h * o_sh + sub * 8;
  const uint16_t* gb = d_o + b * d_sb + h * d_sh + sub * 8;
  uint4 a[kDeltaRows], g[kDeltaRows];
#pragma unroll
  for (int i = 0; i < kDeltaRows; ++i) {
    const int row = row0 + i * rows_per_pass;
    a[i] = g[i] = make_uint4(0, 0, 0, 0);
    if (row < M) {
      a[i] = *reinterpret_cast<const uint4*>(ob + static_cast<int64_t>(row) * o_st);
      g[i] = *reinterpret_cast<const uint4*>(gb + static_cast<int64_t>(row) * d_st);
    }
  }
#pragma unroll
  for (int i = 0; i < kDeltaRows; ++i) {
    const int row = row0 + i * rows_per_pass;
    const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, gw[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = unpack2<kBf16>(aw[j]), fg = unpack2<kBf16>(gw[j]);
      acc = fmaf(fa.x, fg.x, acc);
      acc = fmaf(fa.y, fg.y, acc);
    }
    for (int o2 = lanes_per_row / 2; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
    if (row < M && sub == 0) delta[static_cast<int64_t>(bh) * M + row] = acc;
  }
}

// ------------------------------------------- dq = (fp32 accumulator) * scale
template <bool kBf16>
__global__ void __launch_bounds__(256)
fox_dq_convert_kernel(const float* __restrict__ acc, uint16_t* __restrict__ dq, int64_t sb, int64_t sh, int64_t st,
                      int H, int M, int D, float scale) {
  const int lanes_per_row = D / 8;
  const int rows_per_block = 256 / lanes_per_row;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int sub = threadIdx.x % lanes_per_row;
  const int row = blockIdx.x * rows_per_block + threadIdx.x / lanes_per_row;
  if (row >= M) return;
  const float4* src = reinterpret_cast<const float4*>(acc + (static_cast<int64_t>(bh) * M + row) * D + sub * 8);
  const float4 a = src[0], c = src[1];
  uint4 w;
  w.x = pack2<kBf16>(a.x * scale, a.y * scale);
  w.y = pack2<kBf16>(a.z * scale, a.w * scale);
  w.z = pack2<kBf16>(c.x * scale, c.y * scale);
  w.w = pack2<kBf16>(c.z * scale, c.w * scale);
  *reinterpret_cast<uint4*>(dq + b * sb + h * sh + static_cast<int64_t>(row) * st + sub * 8) = w;
}

static inline bool head_dim_ok(int64_t D) { return D == 16 || D == 32 || D == 64 || D == 128; }
static inline bool aligned16(const fox_tensor4* t) {
  return t && t->ptr && reinterpret_cast<uintptr_t>(t->ptr) % 16 == 0 && (t->sb * 2) % 16 == 0 &&
         (t->sh * 2) % 16 == 0 && (t->st * 2) % 16 == 0;
}
static inline int launch_rc() { return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH; }

}  // namespace fox

using namespace fox;

extern "C" const char* fox_version(void) { return "fox_b200 0.1 (sm_100a; tcgen05 + TMA)"; }

extern "C" int fox_cumsum_fwd(int device, void* stream, int64_t B, int64_t H, int64_t N, const float* log_fgate,
                              int64_t sb, int64_t sh, int64_t sn, const int64_t* seq_start,
                              const float* carry_in, float* log_lambda, float* total_out) {
  if (!log_fgate || !log_lambda || B <= 0 || H <= 0 || N <= 0) return FOX_ERR_BAD_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  fox_cumsum_kernel<3><<<(unsigned)(B * H), kScanThreads, 0, (cudaStream_t)stream>>>(
      log_fgate, sb, sh, sn, seq_start, carry_in, log_lambda, total_out, nullptr, (int)H, (int)N);
  return launch_rc();
}

extern "C" int fox_gate_prefix_fwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t N,
                                   const void* fgate_logit, int64_t sb, int64_t sh, int64_t sn,
                                   const int64_t* seq_start, float* log_fgate_out, float* log_lambda) {
  if (!fgate_logit || !log_lambda || B <= 0 || H <= 0 || N <= 0) return FOX_ERR_BAD_ARG;
  if (dtype != FOX_DTYPE_FP16 && dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP32) return FOX_ERR_BAD_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const unsigned grid = (unsigned)(B * H);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FOX_DTYPE_FP16)
    fox_cumsum_kernel<0><<<grid, kScanThreads, 0, st>>>(fgate_logit, sb, sh, sn, seq_start, nullptr, log_lambda, nullptr, log_fgate_out, (int)H, (int)N);
  else if (dtype == FOX_DTYPE_BF16)
    fox_cumsum_kernel<1><<<grid, kScanThreads, 0, st>>>(fgate_logit, sb, sh, sn, seq_start, nullptr, log_lambda, nullptr, log_fgate_out, (int)H, (int)N);
  else
    fox_cumsum_kernel<2><<<grid, kScanThreads, 0, st>>>(fgate_logit, sb, sh, sn, seq_start, nullptr, log_lambda, nullptr, log_fgate_out, (int)H, (int)N);
  return launch_rc();
}

extern "C" int fox_revcumsum(int device, void* stream, int64_t B, int64_t H, int64_t M, int64_t N,
                             const float* dlam_col, const float* dlam_row, const float* carry_in,
                             float* dlog_fgate, float* total_out) {
  if (!dlam_col || !dlog_fgate || B <= 0 || H <= 0 || N <= 0 || M <= 0 || M > N) return FOX_ERR_BAD_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  fox_revcumsum_kernel<3><<<(unsigned)(B * H), kScanThreads, 0, (cudaStream_t)stream>>>(
      dlam_col, dlam_row, carry_in, dlog_fgate, total_out, (int)M, (int)N, nullptr, nullptr, 0, 0, 0, (int)H);
  return launch_rc();
}

extern "C" int fox_gate_prefix_bwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                                   const float* dlam_col, const float* dlam_row, const void* fgate_logit,
                                   int64_t sb, int64_t sh, int64_t sn, void* dfgate_logit) {
  if (!dlam_col || !fgate_logit || !dfgate_logit || B <= 0 || H <= 0 || N <= 0 || M <= 0 || M > N) return FOX_ERR_BAD_ARG;
  if (dtype != FOX_DTYPE_FP16 && dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP32) return FOX_ERR_BAD_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const unsigned grid = (unsigned)(B * H);
  cudaStream_t st = (cudaStream_t)stream;
#define FOX_GPB(K) fox_revcumsum_kernel<K><<<grid, kScanThreads, 0, st>>>(dlam_col, dlam_row, nullptr, nullptr, nullptr, (int)M, (int)N, fgate_logit, dfgate_logit, sb, sh, sn, (int)H)
  if (dtype == FOX_DTYPE_FP16) FOX_GPB(0);
  else if (dtype == FOX_DTYPE_BF16) FOX_GPB(1);
  else FOX_GPB(2);
#undef FOX_GPB
  return launch_rc();
}

extern "C" int fox_find_index(int device, void* stream, int64_t B, int64_t H, int64_t M, int64_t N,
                              int64_t block_m, int64_t block_n, const float* log_lambda, const float* threshold,
                              int64_t thr_sb, int64_t thr_sh, int64_t* start_index, int64_t* end_index) {
  if (!log_lambda || !threshold || B <= 0 || H <= 0 || N <= 0 || M <= 0 || M > N || block_m <= 0 || block_n <= 0)
    return FOX_ERR_BAD_ARG;
  if (!start_index && !end_index) return FOX_OK;
  const int64_t nmb = (M + block_m - 1) / block_m, nnb = (N + block_n - 1) / block_n;
  const size_t smem = sizeof(float) * (size_t)(2 * nmb + nnb + 1);
  if (smem > 200 * 1024) return FOX_ERR_TOO_LARGE;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(fox_find_index_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return FOX_ERR_LAUNCH;
  }
  fox_find_index_kernel<<<(unsigned)(B * H), 256, smem, (cudaStream_t)stream>>>(
      log_lambda, threshold, thr_sb, thr_sh, start_index, end_index, (int)H, (int)M, (int)N, (int)block_m,
      (int)block_n, (int)nmb, (int)nnb);
  return launch_rc();
}

extern "C" int fox_max_row_norm(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t T, int64_t D,
                                const fox_tensor4* x, float* out_zeroed) {
  if (!x || !out_zeroed || B <= 0 || H <= 0 || T <= 0) return FOX_ERR_BAD_ARG;
  if (B > 65535 || H > 65535 || B * H > 65535) return FOX_ERR_TOO_LARGE;   // (b, h) is the grid's y index
  if (!head_dim_ok(D)) return FOX_ERR_HEAD_DIM;
  if (!aligned16(x)) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const int rows_per_block = 256 / (int)(D / 8);
  // one wave of resident blocks (8 of 256 threads per SM on 148 SMs) shared among the (b, h) rows of the grid:
  // more blocks than that run as a second, partly filled wave
  int64_t gx = (T + rows_per_block - 1) / rows_per_block;
  const int64_t per_unit = (148 * 8) / (B * H) > 0 ? (148 * 8) / (B * H) : 1;
  if (gx > per_unit) gx = per_unit;
  dim3 grid((unsigned)gx, (unsigned)(B * H));
  if (dtype == FOX_DTYPE_BF16)
    fox_max_row_norm_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x->ptr, x->sb, x->sh, x->st, (int)H, (int)T, (int)D, out_zeroed);
  else
    fox_max_row_norm_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x->ptr, x->sb, x->sh, x->st, (int)H, (int)T, (int)D, out_zeroed);
  return launch_rc();
}

extern "C" int fox_bwd_delta(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t D,
                             const fox_tensor4* o, const fox_tensor4* d_o, float* delta) {
  if (!o || !d_o || !delta || B <= 0 || H <= 0 || M <= 0) return FOX_ERR_BAD_ARG;
  if (B > 65535 || H > 65535 || B * H > 65535) return FOX_ERR_TOO_LARGE;   // (b, h) is the grid's y index
  if (!head_dim_ok(D)) return FOX_ERR_HEAD_DIM;
  if (!aligned16(o) || !aligned16(d_o)) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const int rows_per_block = kDeltaRows * 256 / (int)(D / 8);
  dim3 grid((unsigned)((M + rows_per_block - 1) / rows_per_block), (unsigned)(B * H));
  if (dtype == FOX_DTYPE_BF16)
    fox_delta_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)o->ptr, o->sb, o->sh, o->st, (const uint16_t*)d_o->ptr, d_o->sb, d_o->sh, d_o->st, (int)H, (int)M, (int)D, delta);
  else
    fox_delta_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)o->ptr, o->sb, o->sh, o->st, (const uint16_t*)d_o->ptr, d_o->sb, d_o->sh, d_o->st, (int)H, (int)M, (int)D, delta);
  return launch_rc();
}

extern "C" int fox_dq_convert(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t D,
                              const float* dq_accum, float scale, const fox_tensor4* dq) {
  if (!dq_accum || !dq || B <= 0 || H <= 0 || M <= 0) return FOX_ERR_BAD_ARG;
  if (B > 65535 || H > 65535 || B * H > 65535) return FOX_ERR_TOO_LARGE;   // (b, h) is the grid's y index
  if (!head_dim_ok(D)) return FOX_ERR_HEAD_DIM;
  if (!aligned16(dq)) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  const int rows_per_block = 256 / (int)(D / 8);
  dim3 grid((unsigned)((M + rows_per_block - 1) / rows_per_block), (unsigned)(B * H));
  if (dtype == FOX_DTYPE_BF16)
    fox_dq_convert_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(dq_accum, (uint16_t*)dq->ptr, dq->sb, dq->sh, dq->st, (int)H, (int)M, (int)D, scale);
  else
    fox_dq_convert_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(dq_accum, (uint16_t*)dq->ptr, dq->sb, dq->sh, dq->st, (int)H, (int)M, (int)D, scale);
  return launch_rc();
}
