// Forgetting Attention forward for sm_100a: TMA-staged Q/K/V tiles, tcgen05 MMAs
// with TMEM accumulators, decay bias from the log-gate prefix, causal /
// seq_start / tail masking, online softmax with lazy rescaling, block pruning.
//
// Stands in for upstream's Triton `_fwd_kernel`
// (src/forgetting_transformer/ops/forgetting_attention.py:505-693).
//
// One CTA = one (batch, head, 128-row query tile); two CTAs share an SM so that
// one CTA's softmax overlaps the other's matrix products.
//   warps 0-3 : softmax / correction / epilogue, thread t owns query row t and
//               TMEM lane t (no cross-thread reductions)
//   warp 4    : TMA producer (one elected lane)
//   warp 5    : tcgen05.mma issuer (one elected lane)
// TMEM (256 columns): S = Q K^T fp32 in columns [0,128); the probabilities are
// written back over S as packed 16-bit pairs (columns [0,64)) and consumed as the
// TMEM A operand of P V; O accumulates in columns [128, 128+D).
//
// KV tiles are visited from the diagonal leftwards: with forget gates the
// largest logits sit next to the diagonal, so the running row maximum is found
// on the first tile and the O accumulator hardly ever needs rescaling.
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int kFwdBM = FOX_FWD_BLOCK_M;
constexpr int kFwdBN = FOX_FWD_BLOCK_N;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// the reference maximum is only moved when it is off by more than 2^kLazyShift
constexpr float kLazyShift = 8.0f;

struct FwdParams {
  const float* lam;            // (B,H,N) inclusive prefix of the log gates
  const int64_t* seq_start;    // (B,) or nullptr
  const int64_t* start_index;  // (B,H,ceil(M/128)) or nullptr
  void* o;
  int64_t o_sb, o_sh, o_st;
  float* L;                    // (B,H,M)
  int* status;
  int H, M, N;
  float qk_scale;              // sm_scale * log2(e)
};

enum FwdWaitSite {
  kSiteQFull = 11, kSiteKFull = 12, kSiteVFull = 13, kSiteKEmpty = 14, kSiteVEmpty = 15,
  kSiteSFull = 16, kSitePFull = 17, kSiteODone = 18, kSiteDrain = 19, kSiteNegB = 20, kSiteMerge = 21
};

template <int D, bool kBf16, int BN, int STAGES, int CTAS, bool SPLIT, bool TWOPASS>
__global__ void __launch_bounds__(SPLIT ? 320 : 192, CTAS)
fox_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  // KV tiles of BN rows (64 or 128; the pruning grid stays 128 wide, BN = 64 just walks it in halves).
  // SPLIT: two softmax warpgroups per CTA, each owning half of the tile's columns with its own running
  // maximum, row sum and O accumulator (two independent online-softmax streams, merged in the epilogue),
  // so that four softmax warps per scheduler hide each other's ex2 / TMEM latency without any exchange
  // between the warpgroups inside the loop.
  constexpr int kWG = SPLIT ? 2 : 1;
  constexpr int CW = BN / kWG;              // columns per softmax thread
  constexpr int kQBytes = 128 * D * 2;      // Q tile: D/64 swizzled [128][64] sub-tiles
  constexpr int kTileBytes = BN * D * 2;    // K / V tile: D/64 swizzled [BN][64] sub-tiles
  constexpr int kSubBytes = BN * 128;       // one K / V sub-tile
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  constexpr uint32_t kColO = BN;            // S (fp32) in columns [0, BN), O_g in [BN + g D, BN + (g+1) D)
  constexpr uint32_t kTmemCols = (BN + kWG * D <= 128) ? 128 : ((BN + kWG * D <= 256) ? 256 : 512);
  constexpr int kTmaWarp = 4 * kWG, kMmaWarp = 4 * kWG + 1;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full, bar_s_full, bar_o_done, bar_merge;
  __shared__ uint64_t bar_p_full[2];
  __shared__ uint64_t bar_k_full[STAGES], bar_k_empty[STAGES], bar_v_full[STAGES], bar_v_empty[STAGES];
  __shared__ uint64_t bar_negb[2];
  __shared__ __align__(16) float s_negb[2][BN];  // read as float4
  __shared__ float s_m1[128], s_l1[128];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;
  uint8_t* sV = sK + STAGES * kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int M = p.M, N = p.N, P = N - M;

  // ---- KV range of this query tile (upstream lines 591-613) ----
  const int hi = min(N, P + (mb + 1) * kFwdBM);
  const int seq0 = p.seq_start ? static_cast<int>(p.seq_start[b]) : 0;
  int lo = min(seq0, hi);
  if (p.start_index) {
    const int64_t si = p.start_index[(static_cast<int64_t>(b) * p.H + h) * gridDim.x + mb];
    lo = max(lo, static_cast<int>(si < static_cast<int64_t>(hi) ? si : static_cast<int64_t>(hi)));
  }
  lo = (lo / kFwdBN) * kFwdBN;
  const int nb_lo = lo / BN;
  const int nb_hi = (hi + BN - 1) / BN;  // exclusive
  const int n_tiles = max(nb_hi - nb_lo, 0);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_q_full, 1);
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_p_full[0], 128);
    mbar_init(&bar_p_full[1], 128);
    mbar_init(&bar_o_done, 1);
    mbar_init(&bar_merge, 128);
    mbar_init(&bar_negb[0], 128);
    mbar_init(&bar_negb[1], 128);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_k_full[s], 1);
      mbar_init(&bar_k_empty[s], 1);
      mbar_init(&bar_v_full[s], 1);
      mbar_init(&bar_v_empty[s], 1);
    }
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
    // ===================== TMA producer (whole warp converged, one elected lane issues) =====================
    if (n_tiles > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_expect_tx(&bar_q_full, kQBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) tma_load_4d(sQ + s * 16384, &tmQ, &bar_q_full, s * 64, mb * kFwdBM, h, b);
      }
      __syncwarp();
      int issued = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int nb = nb_hi - 1 - it;
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait_warp(&bar_k_empty[st], ph ^ 1, abortp, p.status, kSiteKEmpty, it)) break;
        if (elect_one()) {
          mbar_expect_tx(&bar_k_full[st], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(sK + st * kTileBytes + s * kSubBytes, &tmK, &bar_k_full[st], s * 64, nb * BN, h, b);
        }
        __syncwarp();
        issued = it * 2 + 1;
        if (!mbar_wait_warp(&bar_v_empty[st], ph ^ 1, abortp, p.status, kSiteVEmpty, it)) break;
        if (elect_one()) {
          mbar_expect_tx(&bar_v_full[st], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(sV + st * kTileBytes + s * kSubBytes, &tmV, &bar_v_full[st], s * 64, nb * BN, h, b);
        }
        __syncwarp();
        issued = it * 2 + 2;
      }
      if (*abortp && lane == 0) {
        // error path only: let the copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_q_full, 0) && clock64() - t0 < 200000000LL) {
        }
        for (int c = max(issued - 2 * STAGES, 0); c < issued; ++c) {
          const int it = c >> 1, st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          uint64_t* bar = (c & 1) ? &bar_v_full[st] : &bar_k_full[st];
          while (!mbar_try_wait(bar, ph) && clock64() - t0 < 200000000LL) {
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer (whole warp converged, one elected lane issues) =====================
    if (n_tiles > 0) {
      constexpr uint32_t idQK = umma_idesc(kFmt, 128, BN, 0, 0);
      constexpr uint32_t idPV = umma_idesc(kFmt, 128, D, 0, 1);
      // descriptors are built once; the loops only move the start-address field
      const uint64_t dQ = umma_desc_kmajor(smem_u32(sQ));
      const uint64_t dK0 = umma_desc_kmajor(smem_u32(sK));
      const uint64_t dV0 = umma_desc_mnmajor(smem_u32(sV), kSubBytes);
      bool ok = mbar_wait_warp(&bar_q_full, 0, abortp, p.status, kSiteQFull);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        ok = mbar_wait_warp(&bar_k_full[st], ph, abortp, p.status, kSiteKFull, it);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dK = umma_desc_advance(dK0, st * kTileBytes);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_ss_raw(tbase, umma_desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32),
                       umma_desc_advance(dK, (kk >> 2) * kSubBytes + (kk & 3) * 32), idQK, kk > 0);
          tc_commit_raw(&bar_s_full);
          tc_commit_raw(&bar_k_empty[st]);
        }
        __syncwarp();
        ok = mbar_wait_warp(&bar_v_full[st], ph, abortp, p.status, kSiteVFull, it);
        if (!ok) break;
        const uint64_t dV = umma_desc_advance(dV0, st * kTileBytes);
#pragma unroll
        for (int g = 0; g < kWG; ++g) {
          ok = mbar_wait_warp(&bar_p_full[g], it & 1, abortp, p.status, kSitePFull, it);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            // O_g += P[:, g CW : (g+1) CW] V[g CW : (g+1) CW, :]; the 16-bit P sits at S columns g CW ...
#pragma unroll
            for (int kk = 0; kk < CW / 16; ++kk)
              mma_ts_raw(tbase + kColO + g * D, tbase + g * CW + kk * 8,
                         umma_desc_advance(dV, (g * (CW / 16) + kk) * 2048), idPV, (it > 0 || kk > 0) ? 1u : 0u);
            if (g == kWG - 1) tc_commit_raw(&bar_v_empty[st]);
          }
          __syncwarp();
        }
        if (!ok) break;
      }
      if (ok) tc_commit(&bar_o_done);
    }
  } else {
    // ===================== softmax / correction / epilogue =====================
    const int g = SPLIT ? (warp >> 2) : 0;    // column half owned by this warpgroup
    const int r = tid & 127;                  // query row inside the tile == TMEM lane
    const int row = mb * kFwdBM + r;
    const bool row_ok = row < M;
    const int64_t bh = static_cast<int64_t>(b) * p.H + h;
    const float* lam = p.lam + bh * N;
    const float a_i = row_ok ? lam[P + row] * kLog2e : 0.f;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tbase + lane_base + g * CW;
    const uint32_t tO = tbase + lane_base + kColO + g * D;

    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    float negb_next = 0.f;
    const bool stager = (g == 0) && (r < BN);  // these threads stage one -b_j each per tile
    if (n_tiles > 0 && stager) {
      const int col = (nb_hi - 1) * BN + r;
      negb_next = col < N ? -lam[col] * kLog2e : 0.f;
    }
    for (int it = 0; it < n_tiles; ++it) {
      const int nb = nb_hi - 1 - it;
      const int col0 = nb * BN + g * CW;  // first column of this thread's slice
      if (g == 0) {
        if (stager) s_negb[it & 1][r] = negb_next;
        mbar_arrive(&bar_negb[it & 1]);
      }
      ok = mbar_wait(&bar_negb[it & 1], (it >> 1) & 1, abortp, p.status, kSiteNegB, it);
      ok = mbar_wait(&bar_s_full, it & 1, abortp, p.status, kSiteSFull, it) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (it + 1 < n_tiles && stager) {
        const int col = (nb - 1) * BN + r;
        negb_next = -lam[col] * kLog2e;  // nb-1 >= nb_lo >= 0 and this tile lies left of the tail
      }
      // Two passes over this thread's slice of S, 32 columns at a time.  TWOPASS reads S from TMEM in both
      // (a TMEM load costs ~50 cycles; holding a 64/128-column slice in registers costs spills):
      //   pass 1: u = s*scale - b_j (masked on boundary tiles), row maximum
      //   pass 2: the same u again, p = 2^(u + a_i - m), row sum, pack, write back over S
      const float4* nb4 = reinterpret_cast<const float4*>(&s_negb[it & 1][g * CW]);
      const bool need_mask = (col0 + CW - 1 > P + mb * kFwdBM) || (col0 < seq0) || (col0 + CW > N);
      // valid columns of this row inside the slice: [c_lo, c_hi]
      const int c_lo = need_mask ? max(seq0 - col0, 0) : 0;
      const int c_hi = need_mask ? (row_ok ? min(min(P + row, N - 1) - col0, CW - 1) : -1) : CW - 1;
      auto load_u = [&](int ch, float* u) {
        uint32_t sreg[32];
        tmem_ld32(tS + ch * 32, sreg);
        tmem_ld_wait();
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 nbv = nb4[ch * 8 + c4];
          u[4 * c4 + 0] = fmaf(__uint_as_float(sreg[4 * c4 + 0]), p.qk_scale, nbv.x);
          u[4 * c4 + 1] = fmaf(__uint_as_float(sreg[4 * c4 + 1]), p.qk_scale, nbv.y);
          u[4 * c4 + 2] = fmaf(__uint_as_float(sreg[4 * c4 + 2]), p.qk_scale, nbv.z);
          u[4 * c4 + 3] = fmaf(__uint_as_float(sreg[4 * c4 + 3]), p.qk_scale, nbv.w);
        }
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int cc = ch * 32 + c;
            u[c] = (cc >= c_lo && cc <= c_hi) ? u[c] : -INFINITY;
          }
        }
      };
      float umax = -INFINITY;
      float ukeep[TWOPASS ? 1 : CW];  // one-pass form: u stays in registers between the passes
#pragma unroll
      for (int ch = 0; ch < CW / 32; ++ch) {
        float utmp[32];
        float* u = TWOPASS ? utmp : &ukeep[TWOPASS ? 0 : ch * 32];
        load_u(ch, u);
#pragma unroll
        for (int c = 0; c < 32; c += 4) umax = fmaxf(umax, fmaxf(fmaxf(u[c], u[c + 1]), fmaxf(u[c + 2], u[c + 3])));
      }
      // ---- running maximum with lazy rescaling ----
      const float m_new = fmaxf(m_ref, a_i + umax);
      const bool need = (m_new - m_ref) > kLazyShift;  // false when both are -inf (NaN compare)
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_ref - m_new);
        l_sum *= alpha;
        if (it > 0) {
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32(tO + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st32(tO + c, o);
          }
        }
        m_ref = m_new;
      }
      const float off = a_i - ((m_ref == -INFINITY) ? 0.f : m_ref);
      float psum = 0.f;
#pragma unroll
      for (int ch = 0; ch < CW / 32; ++ch) {
        float utmp[32];
        float* u = TWOPASS ? utmp : &ukeep[TWOPASS ? 0 : ch * 32];
        if (TWOPASS) load_u(ch, u);
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float p0 = fast_exp2(u[2 * j] + off);
          const float p1 = fast_exp2(u[2 * j + 1] + off);
          psum += p0 + p1;
          pk[j] = pack2<kBf16>(p0, p1);
        }
        tmem_st16(tS + ch * 16, pk);  // columns already consumed by this thread
      }
      l_sum += psum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_p_full[g]);
    }

    // ---- epilogue: merge the streams, O / l -> 16-bit -> global, L = m ln2 + ln l ----
    if (SPLIT && g == 1) {
      s_m1[r] = m_ref;
      s_l1[r] = l_sum;
      mbar_arrive(&bar_merge);
    }
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_o_done, 0, abortp, p.status, kSiteODone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (SPLIT && g == 0 && ok) {
      ok = mbar_wait(&bar_merge, 0, abortp, p.status, kSiteMerge);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && g == 0) {
      tc_fence_after();
      float w0 = 1.f, w1 = 0.f;
      if (SPLIT) {
        const float m1 = s_m1[r], l1 = s_l1[r];
        const float m = fmaxf(m_ref, m1);
        w0 = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m);
        w1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - m);
        l_sum = l_sum * w0 + l1 * w1;
        m_ref = m;
      }
      const bool empty = (n_tiles == 0) || (P + row < seq0) || !(l_sum > 0.f);
      const float inv_l = empty ? 0.f : 1.f / l_sum;
      w0 *= inv_l;
      w1 *= inv_l;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + b * p.o_sb + h * p.o_sh + static_cast<int64_t>(row) * p.o_st;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        float o[32];
        if (n_tiles > 0) {
          uint32_t t0[32];
          tmem_ld32(tO + c, t0);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(t0[j]) * w0;
          if (SPLIT) {
            uint32_t t1[32];
            tmem_ld32(tO + D + c, t1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = fmaf(__uint_as_float(t1[j]), w1, o[j]);
          }
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w = make_uint4(0, 0, 0, 0);
            if (!empty) {
              w.x = pack2<kBf16>(o[j + 0], o[j + 1]);
              w.y = pack2<kBf16>(o[j + 2], o[j + 3]);
              w.z = pack2<kBf16>(o[j + 4], o[j + 5]);
              w.w = pack2<kBf16>(o[j + 6], o[j + 7]);
            }
            *reinterpret_cast<uint4*>(orow + c + j) = w;
          }
        }
      }
      if (row_ok) p.L[bh * M + row] = empty ? -INFINITY : m_ref * kLn2 + __logf(l_sum);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tbase, kTmemCols);
}

// Shapes: D=64 -> 128-row KV tiles, two softmax warpgroups with independent streams, S re-read from TMEM;
// D=128 -> 64-row KV tiles, two stages, one softmax warpgroup.  Tuning hook: 1 = D=64 with one warpgroup.
static int g_fwd_variant = 0;

template <int D, bool kBf16, int BN, int STAGES, int CTAS, bool SPLIT, bool TWOPASS>
static int launch_fwd(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
                      const fox_tensor4* k, const fox_tensor4* v, const FwdParams& prm) {
  CUtensorMap tmQ, tmK, tmV;
  Tensor4 tq{q->ptr, B, H, M, D, q->sb, q->sh, q->st};
  Tensor4 tk{k->ptr, B, H, N, D, k->sb, k->sh, k->st};
  Tensor4 tv{v->ptr, B, H, N, D, v->sb, v->sh, v->st};
  if (!tma_compatible(tq, 2) || !tma_compatible(tk, 2) || !tma_compatible(tv, 2)) return FOX_ERR_ALIGNMENT;
  int rc;
  if ((rc = cached_tmap_4d(&tmQ, tq, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmK, tk, 2, false, kBf16, 64, BN, true))) return rc;
  if ((rc = cached_tmap_4d(&tmV, tv, 2, false, kBf16, 64, BN, true))) return rc;
  constexpr int smem = 128 * D * 2 + 2 * STAGES * BN * D * 2 + 1024;
  auto kern = fox_attn_fwd_kernel<D, kBf16, BN, STAGES, CTAS, SPLIT, TWOPASS>;
  static bool configured[64] = {};  // per template instance and device
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[device] = true;
  }
  dim3 grid((unsigned)((M + kFwdBM - 1) / kFwdBM), (unsigned)H, (unsigned)B);
  kern<<<grid, SPLIT ? 320 : 192, smem, stream>>>(tmQ, tmK, tmV, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

}  // namespace fox

extern "C" void fox_debug_set_fwd_variant(int v) { fox::g_fwd_variant = v; }

extern "C" int fox_attn_fwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                            int64_t D, const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                            const float* log_lambda, const int64_t* seq_start, const int64_t* start_index,
                            float sm_scale, const fox_tensor4* o, float* L, int32_t* status) {
  using namespace fox;
  if (!q || !k || !v || !o || !q->ptr || !k->ptr || !v->ptr || !o->ptr || !log_lambda || !L || !status)
    return FOX_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || M <= 0 || N <= 0 || M > N || H > 65535 || B > 65535) return FOX_ERR_BAD_ARG;
  if (D != 64 && D != 128) return FOX_ERR_HEAD_DIM;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(o->ptr) % 16 || (o->sb * 2) % 16 || (o->sh * 2) % 16 || (o->st * 2) % 16)
    return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  FwdParams prm;
  prm.lam = log_lambda;
  prm.seq_start = seq_start;
  prm.start_index = start_index;
  prm.o = o->ptr; prm.o_sb = o->sb; prm.o_sh = o->sh; prm.o_st = o->st;
  prm.L = L;
  prm.status = status;
  prm.H = (int)H; prm.M = (int)M; prm.N = (int)N;
  prm.qk_scale = sm_scale * 1.4426950408889634f;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = dtype == FOX_DTYPE_BF16;
  const int variant = g_fwd_variant;
  if (D == 64) {
    if (variant == 1)
      return bf ? launch_fwd<64, true, 128, 2, 2, false, true>(device, st, B, H, M, N, q, k, v, prm)
                : launch_fwd<64, false, 128, 2, 2, false, true>(device, st, B, H, M, N, q, k, v, prm);
    return bf ? launch_fwd<64, true, 128, 2, 2, true, true>(device, st, B, H, M, N, q, k, v, prm)
              : launch_fwd<64, false, 128, 2, 2, true, true>(device, st, B, H, M, N, q, k, v, prm);
  }
  return bf ? launch_fwd<128, true, 64, 2, 2, false, false>(device, st, B, H, M, N, q, k, v, prm)
            : launch_fwd<128, false, 64, 2, 2, false, false>(device, st, B, H, M, N, q, k, v, prm);
}
