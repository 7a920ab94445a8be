// Forgetting Attention backward, query side: dQ and the query-side log-gate gradient.
//
// Stands in for upstream's Triton `_bwd_q_kernel`
// (src/forgetting_transformer/ops/forgetting_attention.py:1156-1344).  Used at D = 128, where the one-pass
// backward kernel's dQ partials (64 KB of fp32 per tile pair, add-reduced into L2 at the L2's chip-wide rate)
// cost more than recomputing S and dP: there the key side runs without a dQ product and this kernel owns dQ.
//
// Two kernels: fox_attn_bwd_dq2_kernel (further down; one CTA per SM, 128-column tiles, products of the
// next tile under the elementwise passes of this one), the default, and the first form (debug hook):
// one CTA = one (batch, head, 128-row query tile), two CTAs per SM, same roles as the forward kernel:
//   warps 0-3 : thread t owns query row t (TMEM lane t): p = 2^(s c + e_i - b_j), dS = p (dP - delta_i),
//               16-bit dS written over S, running rowsum(dS) (of the fp32 values, like the key side's colsum)
//   warp 4    : TMA producer (Q, dO once; K, V tiles of 64 rows; also stages the tile's gate prefixes)
//   warp 5    : tcgen05.mma issuer: S = Q K^T, dP = dO V^T (smem x smem), dQ += dS K (TMEM x smem)
// TMEM (256 columns): S fp32 [0,64), dP fp32 [64,128), dQ fp32 [128, 128 + D).
// KV tiles are walked from the diagonal leftwards over the same range as the forward (lines 1239-1261).
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int kDqBM = 128, kDqBN = 64;
constexpr float kDqLog2e = 1.4426950408889634f;

struct DqParams {
  const float* lam;            // (B,H,N)
  const float* L;              // (B,H,M)
  const float* delta;          // (B,H,M)
  const int64_t* seq_start;    // (B,) or nullptr
  const int64_t* start_index;  // (B,H,ceil(M/128)) or nullptr
  void* dq;
  int64_t dq_sb, dq_sh, dq_st;
  float* dlam_row;             // (B,H,M), fully written
  int* status;
  int H, M, N;
  float qk_scale;              // sm_scale * log2(e)
  float sm_scale;
};

#ifdef FOX_DQ_TRACE
__device__ long long g_dq_trace[24 * 8 * 16];
#define DQSTAMP(role, ev, it) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (it) >= 32 && (it) < 48) g_dq_trace[((role) * 8 + (ev)) * 16 + (it) - 32] = clock64(); } while (0)
extern "C" int fox_debug_read_dq_trace(long long* host) { return cudaMemcpyFromSymbol(host, g_dq_trace, sizeof(g_dq_trace)); }
#else
#define DQSTAMP(role, ev, it)
#endif

#ifdef FOX_DEBUG   // the first form is kept in debug builds only
enum DqWaitSite { kDqSiteQ = 41, kDqSiteK = 42, kDqSiteV = 43, kDqSiteKE = 44, kDqSiteVE = 45, kDqSiteS = 46,
                  kDqSiteDS = 47, kDqSiteDone = 48, kDqSiteNegB = 49 };

template <int D, bool kBf16>
__global__ void __launch_bounds__(192, 2)
fox_attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                       const DqParams p) {
  constexpr int BN = kDqBN;
  constexpr int kQBytes = 128 * D * 2;
  constexpr int kTileBytes = BN * D * 2;
  constexpr int kSubBytes = BN * 128;
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  constexpr uint32_t kColS = 0, kColDP = BN, kColDQ = 2 * BN;
  constexpr uint32_t kTmemCols = 256;
  static_assert(2 * BN + D <= 256, "TMEM budget");
  constexpr int kTmaWarp = 4, kMmaWarp = 5;

  // (1024-byte aligned by declaration: two CTAs of 112 KB of tiles each fill the SM's shared memory to within
  // a few hundred bytes, there is no room for an alignment slack)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full, bar_k_full[2], bar_k_empty[2], bar_v_full, bar_v_empty, bar_sdp_full, bar_ds_full, bar_done;
  __shared__ uint64_t bar_negb[3];
  __shared__ __align__(16) float s_negb[3][BN];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* sQ = smem_raw;
  uint8_t* sDO = sQ + kQBytes;
  uint8_t* sK = sDO + kQBytes;
  uint8_t* sV = sK + 2 * kTileBytes;  // K in two stages (it is read by S and, a whole elementwise pass later, by dQ), V in one

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int M = p.M, N = p.N, P = N - M;
  const int64_t bh = static_cast<int64_t>(b) * p.H + h;

  const int hi = min(N, P + (mb + 1) * kDqBM);
  const int seq0 = p.seq_start ? static_cast<int>(p.seq_start[b]) : 0;
  int lo = min(seq0, hi);
  if (p.start_index) {
    const int64_t si = p.start_index[bh * gridDim.x + mb];
    lo = max(lo, static_cast<int>(si < static_cast<int64_t>(hi) ? si : static_cast<int64_t>(hi)));
  }
  lo = (lo / 128) * 128;
  const int nb_lo = lo / BN;
  const int nb_hi = (hi + BN - 1) / BN;
  const int n_tiles = max(nb_hi - nb_lo, 0);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_k_full[i], 1);
      mbar_init(&bar_k_empty[i], 1);
    }
    mbar_init(&bar_v_full, 1);
    mbar_init(&bar_v_empty, 1);
    mbar_init(&bar_sdp_full, 1);
    mbar_init(&bar_ds_full, 128);
    mbar_init(&bar_done, 1);
    for (int i = 0; i < 3; ++i) mbar_init(&bar_negb[i], 1);
    mbar_fence_init();
  }
  if (warp == kTmaWarp) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == kTmaWarp) {
    // ===================== TMA producer =====================
    if (n_tiles > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmDO);
        mbar_expect_tx(&bar_q_full, 2 * kQBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
          tma_load_4d(sQ + s * 16384, &tmQ, &bar_q_full, s * 64, mb * kDqBM, h, b);
          tma_load_4d(sDO + s * 16384, &tmDO, &bar_q_full, s * 64, mb * kDqBM, h, b);
        }
      }
      __syncwarp();
      const float* lam = p.lam + bh * N;
      float lamv[2] = {0.f, 0.f};   // lane l holds columns 2l, 2l+1 of a tile
      auto fetch_lam = [&](int it) {
        const int c0 = (nb_hi - 1 - it) * BN + 2 * lane;
#pragma unroll
        for (int e = 0; e < 2; ++e) lamv[e] = (c0 + e < N) ? ldg_f32_here(lam + c0 + e) : 0.f;
      };
      auto stage_negb = [&](int it) {
        const int slot = it % 3;
        const float lam_ref = lam[min(P + mb * kDqBM, N - 1)];
        *reinterpret_cast<float2*>(&s_negb[slot][2 * lane]) =
            make_float2((lam_ref - lamv[0]) * kDqLog2e, (lam_ref - lamv[1]) * kDqLog2e);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_negb[slot]);
        __syncwarp();
      };
      fetch_lam(0);
      stage_negb(0);
      if (n_tiles > 1) fetch_lam(1);
      int issued_k = 0, issued_v = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int nb = nb_hi - 1 - it;
        const int ks = it & 1;
        if (!mbar_wait_warp(&bar_k_empty[ks], ((it >> 1) & 1) ^ 1, abortp, p.status, kDqSiteKE, it)) break;
        if (elect_one()) {
          mbar_expect_tx(&bar_k_full[ks], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(sK + ks * kTileBytes + s * kSubBytes, &tmK, &bar_k_full[ks], s * 64, nb * BN, h, b);
        }
        __syncwarp();
        issued_k = it + 1;
        if (!mbar_wait_warp(&bar_v_empty, (it & 1) ^ 1, abortp, p.status, kDqSiteVE, it)) break;  // dS(it-1) done
        if (elect_one()) {
          mbar_expect_tx(&bar_v_full, kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s) tma_load_4d(sV + s * kSubBytes, &tmV, &bar_v_full, s * 64, nb * BN, h, b);
        }
        __syncwarp();
        issued_v = it + 1;
        if (it + 1 < n_tiles) {   // (the slot of tile it+1 was last read for tile it-2, which has long retired)
          stage_negb(it + 1);
          if (it + 2 < n_tiles) fetch_lam(it + 2);
        }
      }
      if (*abortp && lane == 0) {
        // error path only: let the copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_q_full, 0) && clock64() - t0 < 200000000LL) {
        }
        for (int c = max(issued_k - 2, 0); c < issued_k; ++c)
          while (!mbar_try_wait(&bar_k_full[c & 1], (c >> 1) & 1) && clock64() - t0 < 200000000LL) {
          }
        if (issued_v > 0)
          while (!mbar_try_wait(&bar_v_full, (issued_v - 1) & 1) && clock64() - t0 < 200000000LL) {
          }
      }
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    if (n_tiles > 0) {
      constexpr uint32_t idS = umma_idesc(kFmt, 128, BN, 0, 0);
      constexpr uint32_t idDQ = umma_idesc(kFmt, 128, D, 0, 1);
      const uint64_t dQd = umma_desc_kmajor(smem_u32(sQ));
      const uint64_t dDOd = umma_desc_kmajor(smem_u32(sDO));
      const uint64_t dKk = umma_desc_kmajor(smem_u32(sK));
      const uint64_t dVk = umma_desc_kmajor(smem_u32(sV));
      const uint64_t dKmn = umma_desc_mnmajor(smem_u32(sK), kSubBytes);
      bool ok = mbar_wait_warp(&bar_q_full, 0, abortp, p.status, kDqSiteQ);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const uint32_t ph = it & 1;
        const int ks = it & 1;
        DQSTAMP(5, 5, it);
        ok = mbar_wait_warp(&bar_k_full[ks], (it >> 1) & 1, abortp, p.status, kDqSiteK, it);
        if (!ok) break;
        const uint64_t dKk_s = umma_desc_advance(dKk, ks * kTileBytes);
        const uint64_t dKmn_s = umma_desc_advance(dKmn, ks * kTileBytes);
        DQSTAMP(5, 0, it);
        ok = mbar_wait_warp(&bar_v_full, ph, abortp, p.status, kDqSiteV, it);
        if (!ok) break;
        DQSTAMP(5, 1, it);
        tc_fence_after();
        // S(it) overwrites dS(it-1): ordered behind dQ(it-1) in the tensor pipe
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t offq = (kk >> 2) * 16384 + (kk & 3) * 32, offk = (kk >> 2) * kSubBytes + (kk & 3) * 32;
            mma_ss_raw(tbase + kColS, umma_desc_advance(dQd, offq), umma_desc_advance(dKk_s, offk), idS, kk > 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t offq = (kk >> 2) * 16384 + (kk & 3) * 32, offk = (kk >> 2) * kSubBytes + (kk & 3) * 32;
            mma_ss_raw(tbase + kColDP, umma_desc_advance(dDOd, offq), umma_desc_advance(dVk, offk), idS, kk > 0);
          }
          tc_commit_raw(&bar_sdp_full);
          tc_commit_raw(&bar_v_empty);
        }
        __syncwarp();
        DQSTAMP(5, 2, it);
        ok = mbar_wait_warp(&bar_ds_full, ph, abortp, p.status, kDqSiteDS, it);
        if (!ok) break;
        DQSTAMP(5, 3, it);
        tc_fence_after();
        if (elect_one()) {
          // dQ += dS[:, 0:64] K[0:64, :]; the 16-bit dS sits at the S columns
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            mma_ts_raw(tbase + kColDQ, tbase + kColS + kk * 8, umma_desc_advance(dKmn_s, kk * 2048), idDQ,
                       (it > 0 || kk > 0) ? 1u : 0u);
          tc_commit_raw(&bar_k_empty[ks]);
        }
        __syncwarp();
        DQSTAMP(5, 4, it);
      }
      if (ok) tc_commit(&bar_done);
    }
  } else {
    // ===================== elementwise / epilogue =====================
    const int r = tid & 127;
    const int row = mb * kDqBM + r;
    const bool row_ok = row < M;
    float e_i = -INFINITY, delta_i = 0.f;
    if (row_ok) {
      const float Li = p.L[bh * M + row];
      e_i = (Li == -INFINITY) ? -INFINITY
                              : ((p.lam[bh * N + P + row] - p.lam[bh * N + min(P + mb * kDqBM, N - 1)]) - Li) * kDqLog2e;
      delta_i = p.delta[bh * M + row];
    }
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tbase + lane_base + kColS, tDP = tbase + lane_base + kColDP, tDQ = tbase + lane_base + kColDQ;
    const float2 scale2 = make_float2(p.qk_scale, p.qk_scale);
    const float2 e2 = make_float2(e_i, e_i);
    const float2 nd2 = make_float2(-delta_i, -delta_i);
    float2 rowsum2 = make_float2(0.f, 0.f);
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int nb = nb_hi - 1 - it;
      const int col0 = nb * BN;
      DQSTAMP(warp, 0, it);
      ok = mbar_wait(&bar_negb[it % 3], (it / 3) & 1, abortp, p.status, kDqSiteNegB, it);
      ok = mbar_wait(&bar_sdp_full, it & 1, abortp, p.status, kDqSiteS, it) && ok;
      DQSTAMP(warp, 1, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float4* nb4 = reinterpret_cast<const float4*>(&s_negb[it % 3][0]);
      const bool need_mask = (col0 + BN - 1 > P + mb * kDqBM) || (col0 < seq0) || (col0 + BN > N);
      const int c_lo = need_mask ? max(seq0 - col0, 0) : 0;
      const int c_hi = need_mask ? (row_ok ? min(min(P + row, N - 1) - col0, BN - 1) : -1) : BN - 1;
#pragma unroll
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t sreg[32], dreg[32], pk[16];
        tmem_ld32(tS + ch * 32, sreg);
        tmem_ld32(tDP + ch * 32, dreg);
        tmem_ld_wait();
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 nbv = nb4[ch * 8 + c4];
          float2 x01 = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4]), __uint_as_float(sreg[4 * c4 + 1])), scale2,
                                  __fadd2_rn(make_float2(nbv.x, nbv.y), e2));
          float2 x23 = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4 + 2]), __uint_as_float(sreg[4 * c4 + 3])), scale2,
                                  __fadd2_rn(make_float2(nbv.z, nbv.w), e2));
          if (need_mask) {
            const int cc = ch * 32 + 4 * c4;
            x01.x = (cc >= c_lo && cc <= c_hi) ? x01.x : -INFINITY;
            x01.y = (cc + 1 >= c_lo && cc + 1 <= c_hi) ? x01.y : -INFINITY;
            x23.x = (cc + 2 >= c_lo && cc + 2 <= c_hi) ? x23.x : -INFINITY;
            x23.y = (cc + 3 >= c_lo && cc + 3 <= c_hi) ? x23.y : -INFINITY;
          }
          const float2 p01 = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
          const float2 p23 = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
          const float2 ds01 = __fmul2_rn(p01, __fadd2_rn(make_float2(__uint_as_float(dreg[4 * c4]), __uint_as_float(dreg[4 * c4 + 1])), nd2));
          const float2 ds23 = __fmul2_rn(p23, __fadd2_rn(make_float2(__uint_as_float(dreg[4 * c4 + 2]), __uint_as_float(dreg[4 * c4 + 3])), nd2));
          const uint32_t d01 = pack2<kBf16>(ds01.x, ds01.y), d23 = pack2<kBf16>(ds23.x, ds23.y);
          pk[2 * c4] = d01;
          pk[2 * c4 + 1] = d23;
          rowsum2 = __fadd2_rn(rowsum2, __fadd2_rn(ds01, ds23));   // fp32 values, as the key-side kernel's column sums
        }
        tmem_st16(tS + ch * 16, pk);
      }
      DQSTAMP(warp, 2, it);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_ds_full);
      DQSTAMP(warp, 3, it);
    }
    // ---- epilogue: dQ * sm_scale -> 16-bit -> global; rowsum(dS) ----
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_done, 0, abortp, p.status, kDqSiteDone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_sb + h * p.dq_sh + static_cast<int64_t>(row) * p.dq_st;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t t0[32];
        if (n_tiles > 0) {
          tmem_ld32(tDQ + c, t0);
          tmem_ld_wait();
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w = make_uint4(0, 0, 0, 0);
            if (n_tiles > 0) {
              w.x = pack2<kBf16>(__uint_as_float(t0[j + 0]) * p.sm_scale, __uint_as_float(t0[j + 1]) * p.sm_scale);
              w.y = pack2<kBf16>(__uint_as_float(t0[j + 2]) * p.sm_scale, __uint_as_float(t0[j + 3]) * p.sm_scale);
              w.z = pack2<kBf16>(__uint_as_float(t0[j + 4]) * p.sm_scale, __uint_as_float(t0[j + 5]) * p.sm_scale);
              w.w = pack2<kBf16>(__uint_as_float(t0[j + 6]) * p.sm_scale, __uint_as_float(t0[j + 7]) * p.sm_scale);
            }
            *reinterpret_cast<uint4*>(orow + c + j) = w;
          }
        }
      }
      if (row_ok) p.dlam_row[bh * M + row] = rowsum2.x + rowsum2.y;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tbase, kTmemCols);
}

#endif  // FOX_DEBUG

// ---------------------------------------------------------------------------------------------------------------
// Pipelined form: one CTA per SM, 128-row KV tiles, four elementwise warpgroups (thread = query row x
// 32 of the tile's 128 columns; four warps on every scheduler), S double-buffered in TMEM so that the products of
// the next tile run under the elementwise passes of this one:
//   issuer, tile t:  S(t+1) = Q K(t+1)^T | wait dS(t) | dP(t+1) = dO V(t+1)^T | dQ += dS(t) K(t)
//   elementwise, t:  phase A: wait S(t):  p = 2^(s c + e_i - b_j) kept in registers
//                    phase B: wait dP(t): dS = p (dP - delta_i) -> 16 bit over the warpgroup's own S columns
// TMEM (512 columns): S [0,128) and [128,256), dP [256,384), dQ [384,512).  Shared memory: Q, dO resident (64 KB),
// K in three stages (read by S(t) and, two tiles of products later, by dQ(t)), V in one.
// A 128-column S / dP product re-reads Q / dO from shared memory once per 128 columns instead of once per 64.
constexpr int kDq2BN = 128;
enum Dq2WaitSite { kDq2SiteQ = 51, kDq2SiteK = 52, kDq2SiteV = 53, kDq2SiteKE = 54, kDq2SiteVE = 55, kDq2SiteS = 56,
                   kDq2SiteDP = 57, kDq2SiteDS = 58, kDq2SiteDone = 59, kDq2SiteNegB = 60, kDq2SiteRow = 61, kDq2SiteEpi = 62 };

template <int D, bool kBf16>
__global__ void __launch_bounds__(576, 1)
fox_attn_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                        const __grid_constant__ CUtensorMap tmDQ, const DqParams p) {
  static_assert(D == 64 || D == 128, "head dim");
  constexpr int BN = kDq2BN;
  constexpr int kWG = 4, CW = BN / kWG;          // 32 columns of every tile per warpgroup
  constexpr int kKS = 3;                         // K stages
  constexpr int kQBytes = 128 * D * 2;
  constexpr int kTileBytes = BN * D * 2;
  constexpr int kSubBytes = BN * 128;            // one [128 rows][64 x 16 bit] sub-tile
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  constexpr uint32_t kColS = 0, kColDP = 2 * BN, kColDQ = 3 * BN;
  constexpr uint32_t kTmemCols = 512;
  constexpr int kTmaWarp = 4 * kWG, kMmaWarp = 4 * kWG + 1;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full, bar_k_full[kKS], bar_k_empty[kKS], bar_v_full, bar_v_empty, bar_s_full[2], bar_dp_full,
      bar_ds_full, bar_done, bar_rowsum, bar_epi;
  __shared__ uint64_t bar_negb[3];
  __shared__ __align__(16) float s_negb[3][BN];
  __shared__ float s_rowsum[kWG - 1][128];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* sQ = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sDO = sQ + kQBytes;
  uint8_t* sK = sDO + kQBytes;
  uint8_t* sV = sK + kKS * kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int M = p.M, N = p.N, P = N - M;
  const int64_t bh = static_cast<int64_t>(b) * p.H + h;

  const int hi = min(N, P + (mb + 1) * kDqBM);
  const int seq0 = p.seq_start ? static_cast<int>(p.seq_start[b]) : 0;
  int lo = min(seq0, hi);
  if (p.start_index) {
    const int64_t si = p.start_index[bh * gridDim.x + mb];
    lo = max(lo, static_cast<int>(si < static_cast<int64_t>(hi) ? si : static_cast<int64_t>(hi)));
  }
  const int nb_lo = lo / BN;
  const int nb_hi = (hi + BN - 1) / BN;
  const int n_tiles = max(nb_hi - nb_lo, 0);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_q_full, 1);
    for (int i = 0; i < kKS; ++i) {
      mbar_init(&bar_k_full[i], 1);
      mbar_init(&bar_k_empty[i], 1);
    }
    mbar_init(&bar_v_full, 1);
    mbar_init(&bar_v_empty, 1);
    mbar_init(&bar_s_full[0], 1);
    mbar_init(&bar_s_full[1], 1);
    mbar_init(&bar_dp_full, 1);
    mbar_init(&bar_ds_full, 128 * kWG);
    mbar_init(&bar_done, 1);
    mbar_init(&bar_rowsum, 128 * (kWG - 1));
    mbar_init(&bar_epi, 128 * kWG);
    for (int i = 0; i < 3; ++i) mbar_init(&bar_negb[i], 1);
    mbar_fence_init();
  }
  if (warp == kTmaWarp) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == kTmaWarp) {
    // ===================== TMA producer =====================
    if (n_tiles > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmDO);
        mbar_expect_tx(&bar_q_full, 2 * kQBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
          tma_load_4d(sQ + s * 16384, &tmQ, &bar_q_full, s * 64, mb * kDqBM, h, b);
          tma_load_4d(sDO + s * 16384, &tmDO, &bar_q_full, s * 64, mb * kDqBM, h, b);
        }
      }
      __syncwarp();
      const float* lam = p.lam + bh * N;
      // Prefixes enter the logits as Lambda_i - Lambda_j; both are taken relative to the prefix of this query
      // tile's first row before the scaling by log2(e) (a prefix of -1e4 scaled first costs 2e-3 per logit)
      const float lam_ref = lam[min(P + mb * kDqBM, N - 1)];
      float lamv[4] = {0.f, 0.f, 0.f, 0.f};   // lane l holds columns 4l .. 4l+3 of a tile
      auto fetch_lam = [&](int it) {
        const int c0 = (nb_hi - 1 - it) * BN + 4 * lane;
#pragma unroll
        for (int e = 0; e < 4; ++e) lamv[e] = (c0 + e < N) ? ldg_f32_here(lam + c0 + e) : 0.f;
      };
      auto stage_negb = [&](int it) {
        const int slot = it % 3;
        *reinterpret_cast<float4*>(&s_negb[slot][4 * lane]) =
            make_float4((lam_ref - lamv[0]) * kDqLog2e, (lam_ref - lamv[1]) * kDqLog2e,
                        (lam_ref - lamv[2]) * kDqLog2e, (lam_ref - lamv[3]) * kDqLog2e);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_negb[slot]);
        __syncwarp();
      };
      fetch_lam(0);
      stage_negb(0);
      if (n_tiles > 1) fetch_lam(1);
      int issued_k = 0, issued_v = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int nb = nb_hi - 1 - it;
        const int ks = it % kKS;
        if (!mbar_wait_warp(&bar_k_empty[ks], ((it / kKS) & 1) ^ 1, abortp, p.status, kDq2SiteKE, it)) break;
        if (elect_one()) {
          mbar_expect_tx(&bar_k_full[ks], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(sK + ks * kTileBytes + s * kSubBytes, &tmK, &bar_k_full[ks], s * 64, nb * BN, h, b);
        }
        __syncwarp();
        issued_k = it + 1;
        if (!mbar_wait_warp(&bar_v_empty, (it & 1) ^ 1, abortp, p.status, kDq2SiteVE, it)) break;  // dP(it-1) done
        if (elect_one()) {
          mbar_expect_tx(&bar_v_full, kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s) tma_load_4d(sV + s * kSubBytes, &tmV, &bar_v_full, s * 64, nb * BN, h, b);
        }
        __syncwarp();
        issued_v = it + 1;
        if (it + 1 < n_tiles) {   // (the slot of tile it+1 was last read for tile it-2: dP(it-1) done => phase A(it-2) done)
          stage_negb(it + 1);
          if (it + 2 < n_tiles) fetch_lam(it + 2);
        }
      }
      if (*abortp && lane == 0) {
        // error path only: let the copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_q_full, 0) && clock64() - t0 < 200000000LL) {
        }
        for (int c = max(issued_k - kKS, 0); c < issued_k; ++c)
          while (!mbar_try_wait(&bar_k_full[c % kKS], (c / kKS) & 1) && clock64() - t0 < 200000000LL) {
          }
        if (issued_v > 0)
          while (!mbar_try_wait(&bar_v_full, (issued_v - 1) & 1) && clock64() - t0 < 200000000LL) {
          }
      }
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    if (n_tiles > 0) {
      constexpr uint32_t idS = umma_idesc(kFmt, 128, BN, 0, 0);
      constexpr uint32_t idDQ = umma_idesc(kFmt, 128, D, 0, 1);
      const uint64_t dQd = umma_desc_kmajor(smem_u32(sQ));
      const uint64_t dDOd = umma_desc_kmajor(smem_u32(sDO));
      const uint64_t dKk = umma_desc_kmajor(smem_u32(sK));
      const uint64_t dVk = umma_desc_kmajor(smem_u32(sV));
      const uint64_t dKmn = umma_desc_mnmajor(smem_u32(sK), kSubBytes);
      auto issue_s = [&](int t) {      // S(t) -> buffer t & 1
        if (elect_one()) {
          const uint64_t dK_s = umma_desc_advance(dKk, (t % kKS) * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            mma_ss_raw(tbase + kColS + (t & 1) * BN, umma_desc_advance(dQd, off), umma_desc_advance(dK_s, off), idS, kk > 0);
          }
          tc_commit_raw(&bar_s_full[t & 1]);
        }
        __syncwarp();
      };
      auto issue_dp = [&]() {
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            mma_ss_raw(tbase + kColDP, umma_desc_advance(dDOd, off), umma_desc_advance(dVk, off), idS, kk > 0);
          }
          tc_commit_raw(&bar_dp_full);
          tc_commit_raw(&bar_v_empty);
        }
        __syncwarp();
      };
      bool ok = mbar_wait_warp(&bar_q_full, 0, abortp, p.status, kDq2SiteQ);
      if (ok) ok = mbar_wait_warp(&bar_k_full[0], 0, abortp, p.status, kDq2SiteK, 0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = mbar_wait_warp(&bar_v_full, 0, abortp, p.status, kDq2SiteV, 0);
      }
      if (ok) {
        tc_fence_after();
        issue_dp();
      }
      for (int it = 0; it < n_tiles && ok; ++it) {
        DQSTAMP(17, 0, it);
        if (it + 1 < n_tiles) {
          ok = mbar_wait_warp(&bar_k_full[(it + 1) % kKS], ((it + 1) / kKS) & 1, abortp, p.status, kDq2SiteK, it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        DQSTAMP(17, 1, it);
        ok = mbar_wait_warp(&bar_ds_full, it & 1, abortp, p.status, kDq2SiteDS, it);
        if (!ok) break;
        DQSTAMP(17, 2, it);
        if (it + 1 < n_tiles) {
          ok = mbar_wait_warp(&bar_v_full, (it + 1) & 1, abortp, p.status, kDq2SiteV, it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_dp();
        }
        tc_fence_after();
        if (elect_one()) {
          // dQ += dS(it) K(it); warpgroup g's 16-bit dS sits in the first 16 of its own 32 S columns
          const uint64_t dKmn_s = umma_desc_advance(dKmn, (it % kKS) * kTileBytes);
          const uint32_t tA = tbase + kColS + (it & 1) * BN;
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            mma_ts_raw(tbase + kColDQ, tA + (kk >> 1) * CW + (kk & 1) * 8, umma_desc_advance(dKmn_s, kk * 2048), idDQ,
                       (it > 0 || kk > 0) ? 1u : 0u);
          tc_commit_raw(&bar_k_empty[it % kKS]);
        }
        __syncwarp();
        DQSTAMP(17, 3, it);
      }
      if (ok) tc_commit(&bar_done);
    }
  } else {
    // ===================== elementwise / epilogue =====================
    const int g = warp >> 2;
    const int r = tid & 127;
    const int row = mb * kDqBM + r;
    const bool row_ok = row < M;
    float e_i = -INFINITY, delta_i = 0.f;
    if (row_ok) {
      const float Li = p.L[bh * M + row];
      e_i = (Li == -INFINITY) ? -INFINITY
                              : ((p.lam[bh * N + P + row] - p.lam[bh * N + min(P + mb * kDqBM, N - 1)]) - Li) * kDqLog2e;
      delta_i = p.delta[bh * M + row];
    }
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tDP = tbase + lane_base + kColDP + g * CW, tDQ = tbase + lane_base + kColDQ;
    const float2 scale2 = make_float2(p.qk_scale, p.qk_scale);
    const float2 e2 = make_float2(e_i, e_i);
    const float2 nd2 = make_float2(-delta_i, -delta_i);
    float2 rowsum2 = make_float2(0.f, 0.f);
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int nb = nb_hi - 1 - it;
      const int col0 = nb * BN;
      const uint32_t tS = tbase + lane_base + kColS + (it & 1) * BN + g * CW;
      // ---------------- phase A: p ----------------
      DQSTAMP(warp, 0, it);
      ok = mbar_wait(&bar_negb[it % 3], (it / 3) & 1, abortp, p.status, kDq2SiteNegB, it);
      ok = mbar_wait(&bar_s_full[it & 1], (it >> 1) & 1, abortp, p.status, kDq2SiteS, it) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      DQSTAMP(warp, 1, it);
      tc_fence_after();
      uint32_t sreg[32];
      float2 pf[16];
      tmem_ld32(tS, sreg);
      tmem_ld_wait();
      const float4* nb4 = reinterpret_cast<const float4*>(&s_negb[it % 3][g * CW]);
      const bool need_mask = (col0 + BN - 1 > P + mb * kDqBM) || (col0 < seq0) || (col0 + BN > N);
      const int c_lo = need_mask ? max(seq0 - col0, 0) : 0;
      const int c_hi = need_mask ? (row_ok ? min(min(P + row, N - 1) - col0, BN - 1) : -1) : BN - 1;
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 nbv = nb4[c4];
        float2 x01 = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4]), __uint_as_float(sreg[4 * c4 + 1])), scale2,
                                __fadd2_rn(make_float2(nbv.x, nbv.y), e2));
        float2 x23 = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4 + 2]), __uint_as_float(sreg[4 * c4 + 3])), scale2,
                                __fadd2_rn(make_float2(nbv.z, nbv.w), e2));
        if (need_mask) {
          const int cc = g * CW + 4 * c4;
          x01.x = (cc >= c_lo && cc <= c_hi) ? x01.x : -INFINITY;
          x01.y = (cc + 1 >= c_lo && cc + 1 <= c_hi) ? x01.y : -INFINITY;
          x23.x = (cc + 2 >= c_lo && cc + 2 <= c_hi) ? x23.x : -INFINITY;
          x23.y = (cc + 3 >= c_lo && cc + 3 <= c_hi) ? x23.y : -INFINITY;
        }
        pf[2 * c4] = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
        pf[2 * c4 + 1] = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
      }
      DQSTAMP(warp, 2, it);
      // ---------------- phase B: dS ----------------
      ok = mbar_wait(&bar_dp_full, it & 1, abortp, p.status, kDq2SiteDP, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      DQSTAMP(warp, 3, it);
      tc_fence_after();
      uint32_t pk[16];
      tmem_ld32(tDP, sreg);
      tmem_ld_wait();
#pragma unroll
      for (int c2 = 0; c2 < 16; ++c2) {
        const float2 ds = __fmul2_rn(pf[c2], __fadd2_rn(make_float2(__uint_as_float(sreg[2 * c2]), __uint_as_float(sreg[2 * c2 + 1])), nd2));
        pk[c2] = pack2<kBf16>(ds.x, ds.y);
        rowsum2 = __fadd2_rn(rowsum2, ds);   // fp32 values, as the key-side kernel's column sums
      }
      tmem_st16(tS, pk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_ds_full);
      DQSTAMP(warp, 4, it);
    }
    // ---- epilogue: dQ * sm_scale -> 16-bit -> global (each warpgroup a quarter of the columns); rowsum(dS) ----
    if (g > 0) {
      s_rowsum[g - 1][r] = rowsum2.x + rowsum2.y;
      mbar_arrive(&bar_rowsum);
    } else {
      ok = mbar_wait(&bar_rowsum, 0, abortp, p.status, kDq2SiteRow) && ok;
      ok = __all_sync(0xffffffffu, ok);
    }
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_done, 0, abortp, p.status, kDq2SiteDone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      // With pruning on, a CTA lives for a few tiles and this epilogue weighs: the 16-bit tile then goes through
      // shared memory (Q is idle: every product has retired) and leaves as TMA stores, which write whole lines
      // and clip the rows past M.  Without pruning the direct stores measured 2 % faster for the whole kernel.
      constexpr int kCols = D / kWG;   // 32 or 16
      const bool via_tma = p.start_index != nullptr;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_sb + h * p.dq_sh + static_cast<int64_t>(row) * p.dq_st + g * kCols;
      uint32_t t0[kCols];
      if (n_tiles > 0) {
        if constexpr (kCols == 32) tmem_ld32(tDQ + g * kCols, t0); else tmem_ld16(tDQ + g * kCols, t0);
        tmem_ld_wait();
      }
#pragma unroll
      for (int j = 0; j < kCols; j += 8) {
        uint4 w = make_uint4(0, 0, 0, 0);
        if (n_tiles > 0) {
          w.x = pack2<kBf16>(__uint_as_float(t0[j + 0]) * p.sm_scale, __uint_as_float(t0[j + 1]) * p.sm_scale);
          w.y = pack2<kBf16>(__uint_as_float(t0[j + 2]) * p.sm_scale, __uint_as_float(t0[j + 3]) * p.sm_scale);
          w.z = pack2<kBf16>(__uint_as_float(t0[j + 4]) * p.sm_scale, __uint_as_float(t0[j + 5]) * p.sm_scale);
          w.w = pack2<kBf16>(__uint_as_float(t0[j + 6]) * p.sm_scale, __uint_as_float(t0[j + 7]) * p.sm_scale);
        }
        const int col = g * kCols + j;
        if (via_tma) *reinterpret_cast<uint4*>(sQ + (col >> 6) * 16384 + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4)) = w;
        else if (row_ok) *reinterpret_cast<uint4*>(orow + j) = w;
      }
      if (via_tma) {
        fence_proxy_async_smem();
        mbar_arrive(&bar_epi);
      }
      if (via_tma && warp == 0) {
        // (a bounded wait like every other one: a warp that gave up elsewhere never arrives)
        if (mbar_wait_warp(&bar_epi, 0, abortp, p.status, kDq2SiteEpi) && elect_one()) {
#pragma unroll
          for (int sub = 0; sub < D / 64; ++sub)
            tma_store_4d(&tmDQ, sQ + sub * 16384, sub * 64, mb * kDqBM, h, b);
          tma_store_commit();
          tma_store_wait_read<0>();   // the tile must stay in shared memory until it has been read
        }
        __syncwarp();
      }
      if (g == 0 && row_ok)
        p.dlam_row[bh * M + row] = (rowsum2.x + rowsum2.y) + (s_rowsum[0][r] + s_rowsum[1][r]) + s_rowsum[2][r];
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tbase, kTmemCols);
}

#ifdef FOX_DEBUG
static int g_dq_variant = 1;   // 0: two CTAs per SM, 64-column tiles; 1: pipelined form

template <int D, bool kBf16>
static int launch_dq(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
                     const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o, const DqParams& prm) {
  CUtensorMap tmQ, tmK, tmV, tmDO;
  Tensor4 tq{q->ptr, B, H, M, D, q->sb, q->sh, q->st};
  Tensor4 tk{k->ptr, B, H, N, D, k->sb, k->sh, k->st};
  Tensor4 tv{v->ptr, B, H, N, D, v->sb, v->sh, v->st};
  Tensor4 tdo{d_o->ptr, B, H, M, D, d_o->sb, d_o->sh, d_o->st};
  if (!tma_compatible(tq, 2) || !tma_compatible(tk, 2) || !tma_compatible(tv, 2) || !tma_compatible(tdo, 2))
    return FOX_ERR_ALIGNMENT;
  int rc;
  if ((rc = cached_tmap_4d(&tmQ, tq, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmDO, tdo, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmK, tk, 2, false, kBf16, 64, kDqBN, true))) return rc;
  if ((rc = cached_tmap_4d(&tmV, tv, 2, false, kBf16, 64, kDqBN, true))) return rc;
  constexpr int smem = 2 * 128 * D * 2 + 3 * kDqBN * D * 2;
  auto kern = fox_attn_bwd_dq_kernel<D, kBf16>;
  static bool configured[64] = {};
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[device] = true;
  }
  dim3 grid((unsigned)((M + kDqBM - 1) / kDqBM), (unsigned)H, (unsigned)B);
  kern<<<grid, 192, smem, stream>>>(tmQ, tmK, tmV, tmDO, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

#endif  // FOX_DEBUG

template <int D, bool kBf16>
static int launch_dq2(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
                      const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o, const DqParams& prm) {
  CUtensorMap tmQ, tmK, tmV, tmDO;
  Tensor4 tq{q->ptr, B, H, M, D, q->sb, q->sh, q->st};
  Tensor4 tk{k->ptr, B, H, N, D, k->sb, k->sh, k->st};
  Tensor4 tv{v->ptr, B, H, N, D, v->sb, v->sh, v->st};
  Tensor4 tdo{d_o->ptr, B, H, M, D, d_o->sb, d_o->sh, d_o->st};
  if (!tma_compatible(tq, 2) || !tma_compatible(tk, 2) || !tma_compatible(tv, 2) || !tma_compatible(tdo, 2))
    return FOX_ERR_ALIGNMENT;
  int rc;
  if ((rc = cached_tmap_4d(&tmQ, tq, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmDO, tdo, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmK, tk, 2, false, kBf16, 64, kDq2BN, true))) return rc;
  if ((rc = cached_tmap_4d(&tmV, tv, 2, false, kBf16, 64, kDq2BN, true))) return rc;
  CUtensorMap tmDQ;
  Tensor4 tdq{prm.dq, B, H, M, D, prm.dq_sb, prm.dq_sh, prm.dq_st};
  if (!tma_compatible(tdq, 2)) return FOX_ERR_ALIGNMENT;
  if ((rc = cached_tmap_4d(&tmDQ, tdq, 2, false, kBf16, 64, 128, true))) return rc;
  constexpr int smem = 2 * 128 * D * 2 + 4 * kDq2BN * D * 2 + 1024;
  auto kern = fox_attn_bwd_dq2_kernel<D, kBf16>;
  static bool configured[64] = {};
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[device] = true;
  }
  dim3 grid((unsigned)((M + kDqBM - 1) / kDqBM), (unsigned)H, (unsigned)B);
  kern<<<grid, 576, smem, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

}  // namespace fox

#ifdef FOX_DEBUG
// Debug builds only: 0 selects the two-CTA form at every head dim, 1 (default) the pipelined form.
extern "C" void fox_debug_set_dq_variant(int v) { fox::g_dq_variant = v; }
#endif

extern "C" int fox_attn_bwd_dq(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N, int64_t D,
                               const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o,
                               const float* log_lambda, const float* L, const float* delta, const int64_t* seq_start,
                               const int64_t* start_index, float sm_scale, const fox_tensor4* dq, float* dlam_row,
                               int32_t* status) {
  using namespace fox;
  if (!q || !k || !v || !d_o || !dq || !q->ptr || !k->ptr || !v->ptr || !d_o->ptr || !dq->ptr || !log_lambda || !L ||
      !delta || !dlam_row || !status)
    return FOX_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || M <= 0 || N <= 0 || M > N || H > 65535 || B > 65535) return FOX_ERR_BAD_ARG;
  if (N > 2147483647LL) return FOX_ERR_TOO_LARGE;   // row indices are 32-bit inside the kernels (M <= N)
  if (D != 64 && D != 128) return FOX_ERR_HEAD_DIM;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(dq->ptr) % 16 || (dq->sb * 2) % 16 || (dq->sh * 2) % 16 || (dq->st * 2) % 16)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  DqParams prm;
  prm.lam = log_lambda; prm.L = L; prm.delta = delta; prm.seq_start = seq_start; prm.start_index = start_index;
  prm.dq = dq->ptr; prm.dq_sb = dq->sb; prm.dq_sh = dq->sh; prm.dq_st = dq->st;
  prm.dlam_row = dlam_row; prm.status = status;
  prm.H = (int)H; prm.M = (int)M; prm.N = (int)N;
  prm.qk_scale = sm_scale * kDqLog2e;
  prm.sm_scale = sm_scale;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = dtype == FOX_DTYPE_BF16;
#ifdef FOX_DEBUG
  if (g_dq_variant != 1) {
    if (D == 64)
      return bf ? launch_dq<64, true>(device, st, B, H, M, N, q, k, v, d_o, prm) : launch_dq<64, false>(device, st, B, H, M, N, q, k, v, d_o, prm);
    return bf ? launch_dq<128, true>(device, st, B, H, M, N, q, k, v, d_o, prm) : launch_dq<128, false>(device, st, B, H, M, N, q, k, v, d_o, prm);
  }
#endif
  if (D == 64)
    return bf ? launch_dq2<64, true>(device, st, B, H, M, N, q, k, v, d_o, prm) : launch_dq2<64, false>(device, st, B, H, M, N, q, k, v, d_o, prm);
  return bf ? launch_dq2<128, true>(device, st, B, H, M, N, q, k, v, d_o, prm) : launch_dq2<128, false>(device, st, B, H, M, N, q, k, v, d_o, prm);
}
