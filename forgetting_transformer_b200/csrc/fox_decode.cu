// Single-query ("decode") forgetting attention: one new token against a cache of N keys.
//
// The path upstream's generation loop takes through the same _fwd_kernel with seqlen_q = 1
// (src/forgetting_transformer/ops/forgetting_attention.py:148-153, 591-693; the cache that feeds it is
// fgate_cache.py:77-116).  With one query row the work is a pair of matrix-vector products, bound by reading
// K and V once, so it is spread over `splits` CTAs per (b,h) that each reduce a slice of the keys to a partial
// (m, l, o) triple on the CUDA cores; a second small kernel merges the triples:
//
//   u_j = (q.k_j) sm_scale log2e + (Lambda_{N-1} - Lambda_j) log2e      (j >= seq_start, j >= start_index)
//   m = max u_j;  l = sum 2^(u_j - m);  o = sum 2^(u_j - m) v_j;   out = o / l;   L = m ln2 + ln l
//
// Thread = one key at a time for a 64-wide slice of the head dimension (D = 128: two neighbouring lanes
// share a key); q, the running o and (m, l) live in registers.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int kDecThreads = 128;
constexpr float kDecLog2e = 1.4426950408889634f;

template <bool kBf16>
__device__ __forceinline__ void dec_load8(const uint16_t* p, float* f) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack2<kBf16>(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

struct DecodeParams {
  const uint16_t *q, *k, *v;
  int64_t q_sb, q_sh, k_sb, k_sh, k_st, v_sb, v_sh, v_st;
  const float* lam;            // (B,H,N)
  const int64_t* seq_start;    // (B,) or nullptr
  const int64_t* start_index;  // (B,H,1) or nullptr
  float* part;                 // (B,H,splits, D + 2): o[D], m, l
  int H, N, splits;
  float qk_scale;              // sm_scale * log2(e)
};

// TPK threads share one key (D = 64 TPK)
template <bool kBf16, int TPK>
__global__ void __launch_bounds__(kDecThreads)
fox_decode_partial_kernel(const DecodeParams p) {
  constexpr int D = 64 * TPK;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int sub = tid % TPK;              // which 64-wide slice of the head dimension
  const int kslot = tid / TPK;            // key slot inside the CTA
  constexpr int kKeysPerPass = kDecThreads / TPK;
  const int64_t bh = static_cast<int64_t>(b) * p.H + h;
  const int N = p.N;
  int lo = p.seq_start ? static_cast<int>(p.seq_start[b]) : 0;
  if (p.start_index) {
    const int64_t si = p.start_index[bh];
    lo = max(lo, static_cast<int>(si < N ? si : N));
  }
  lo = min(lo, N);
  // this CTA's slice of [lo, N)
  const int span = N - lo;
  const int per = (span + p.splits - 1) / p.splits;
  const int j0 = lo + split * per, j1 = min(N, j0 + per);

  float qv[64];
  {
    const uint16_t* qp = p.q + b * p.q_sb + h * p.q_sh + sub * 64;
#pragma unroll
    for (int c = 0; c < 8; ++c) dec_load8<kBf16>(qp + c * 8, &qv[c * 8]);
  }
  const float* lam = p.lam + bh * N;
  const float a = lam[N - 1];   // (the difference of two prefixes is formed before the scaling by log2(e))
  float m = -INFINITY, l = 0.f;
  float acc[64];
#pragma unroll
  for (int d = 0; d < 64; ++d) acc[d] = 0.f;

  for (int jb = j0; jb < j1; jb += kKeysPerPass) {
    const int j = jb + kslot;
    const bool in = j < j1;
    const int jc = in ? j : j0;
    const uint16_t* kp = p.k + b * p.k_sb + h * p.k_sh + static_cast<int64_t>(jc) * p.k_st + sub * 64;
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float kv[8];
      dec_load8<kBf16>(kp + c * 8, kv);
#pragma unroll
      for (int e = 0; e < 8; ++e) s = fmaf(qv[c * 8 + e], kv[e], s);
    }
    if (TPK == 2) s += __shfl_xor_sync(0xffffffffu, s, 1);
    const float u = in ? fmaf(s, p.qk_scale, (a - lam[jc]) * kDecLog2e) : -INFINITY;
    const float m_new = fmaxf(m, u);
    if (m_new > -INFINITY) {  // (warp-divergent, but only until every lane has seen its first key)
      const float alpha = fast_exp2(m - m_new);   // 0 when m was -inf
      const float pj = fast_exp2(u - m_new);      // 0 for a lane without a key
      l = l * alpha + pj;
      const uint16_t* vp = p.v + b * p.v_sb + h * p.v_sh + static_cast<int64_t>(jc) * p.v_st + sub * 64;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float vv[8];
        dec_load8<kBf16>(vp + c * 8, vv);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[c * 8 + e] = fmaf(acc[c * 8 + e], alpha, pj * vv[e]);
      }
      m = m_new;
    }
  }

  // ---- merge the CTA's key slots: first (m, l), then the weighted accumulators through shared memory ----
  __shared__ float s_m[kDecThreads], s_w[kDecThreads];
  __shared__ float s_acc[kDecThreads / 32][2][64];
  __shared__ float s_ml[2];
  s_m[tid] = m;
  __syncthreads();
  float mx = -INFINITY;
  for (int t = 0; t < kDecThreads; ++t) mx = fmaxf(mx, s_m[t]);
  const float w = (m == -INFINITY) ? 0.f : fast_exp2(m - mx);
  s_w[tid] = (sub == 0) ? l * w : 0.f;
  // warp-level sum of the weighted accumulators per head-dimension slice
#pragma unroll
  for (int d = 0; d < 64; ++d) {
    float x = acc[d] * w;
#pragma unroll
    for (int o = 16; o >= TPK; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    if ((tid & 31) < TPK) s_acc[tid >> 5][sub][d] = x;
  }
  __syncthreads();
  float* out = p.part + (bh * p.splits + split) * (D + 2);
  if (tid < D) {
    const int sl = tid / 64, d = tid % 64;
    float x = 0.f;
#pragma unroll
    for (int wq = 0; wq < kDecThreads / 32; ++wq) x += s_acc[wq][sl][d];
    out[tid] = x;
  }
  if (tid == 0) {
    float lt = 0.f;
    for (int t = 0; t < kDecThreads; ++t) lt += s_w[t];
    out[D] = mx;
    out[D + 1] = lt;
  }
  (void)s_ml;
}

template <bool kBf16>
__global__ void fox_decode_merge_kernel(const float* __restrict__ part, int splits, int D, uint16_t* __restrict__ o,
                                        int64_t o_sb, int64_t o_sh, float* __restrict__ L, int H) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int64_t bh = static_cast<int64_t>(b) * H + h;
  const float* base = part + bh * splits * (D + 2);
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, base[s * (D + 2) + D]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = base[s * (D + 2) + D];
    l += (ms == -INFINITY) ? 0.f : base[s * (D + 2) + D + 1] * fast_exp2(ms - mx);
  }
  const bool empty = !(l > 0.f);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float x = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = base[s * (D + 2) + D];
      if (ms != -INFINITY) x += base[s * (D + 2) + d] * fast_exp2(ms - mx);
    }
    const float r = empty ? 0.f : x / l;
    const uint32_t pk = pack2<kBf16>(r, 0.f);
    o[b * o_sb + h * o_sh + d] = static_cast<uint16_t>(pk & 0xffffu);
  }
  if (threadIdx.x == 0) L[bh] = empty ? -INFINITY : mx * 0.6931471805599453f + __logf(l);
}

}  // namespace fox

using namespace fox;

extern "C" int64_t fox_attn_decode_workspace_floats(int64_t B, int64_t H, int64_t D, int64_t splits) {
  return B * H * splits * (D + 2);
}

extern "C" int fox_attn_decode(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t N, int64_t D,
                               const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                               const float* log_lambda, const int64_t* seq_start, const int64_t* start_index,
                               float sm_scale, const fox_tensor4* o, float* L, float* workspace, int64_t splits) {
  if (!q || !k || !v || !o || !q->ptr || !k->ptr || !v->ptr || !o->ptr || !log_lambda || !L || !workspace)
    return FOX_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || N <= 0 || H > 65535 || B > 65535 || splits <= 0 || splits > 1024) return FOX_ERR_BAD_ARG;
  if (D != 64 && D != 128) return FOX_ERR_HEAD_DIM;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  auto bad = [](const fox_tensor4* t) {
    return reinterpret_cast<uintptr_t>(t->ptr) % 16 || t->sb % 8 || t->sh % 8 || t->st % 8;
  };
  if (bad(q) || bad(k) || bad(v)) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  DecodeParams p;
  p.q = (const uint16_t*)q->ptr; p.k = (const uint16_t*)k->ptr; p.v = (const uint16_t*)v->ptr;
  p.q_sb = q->sb; p.q_sh = q->sh; p.k_sb = k->sb; p.k_sh = k->sh; p.k_st = k->st;
  p.v_sb = v->sb; p.v_sh = v->sh; p.v_st = v->st;
  p.lam = log_lambda; p.seq_start = seq_start; p.start_index = start_index; p.part = workspace;
  p.H = (int)H; p.N = (int)N; p.splits = (int)splits;
  p.qk_scale = sm_scale * kDecLog2e;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)splits, (unsigned)H, (unsigned)B);
  const bool bf = dtype == FOX_DTYPE_BF16;
  if (D == 64) {
    if (bf) fox_decode_partial_kernel<true, 1><<<grid, kDecThreads, 0, st>>>(p);
    else fox_decode_partial_kernel<false, 1><<<grid, kDecThreads, 0, st>>>(p);
  } else {
    if (bf) fox_decode_partial_kernel<true, 2><<<grid, kDecThreads, 0, st>>>(p);
    else fox_decode_partial_kernel<false, 2><<<grid, kDecThreads, 0, st>>>(p);
  }
  if (cudaGetLastError() != cudaSuccess) return FOX_ERR_LAUNCH;
  dim3 grid2((unsigned)H, (unsigned)B);
  if (bf) fox_decode_merge_kernel<true><<<grid2, 128, 0, st>>>(workspace, (int)splits, (int)D, (uint16_t*)o->ptr, o->sb, o->sh, L, (int)H);
  else fox_decode_merge_kernel<false><<<grid2, 128, 0, st>>>(workspace, (int)splits, (int)D, (uint16_t*)o->ptr, o->sb, o->sh, L, (int)H);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}
