// Forgetting Attention forward for sm_100a: TMA-staged Q/K/V tiles, tcgen05 MMAs
// with TMEM accumulators, decay bias from the log-gate prefix, causal /
// seq_start / tail masking, online softmax with lazy rescaling, block pruning.
//
// Stands in for upstream's Triton `_fwd_kernel`
// (src/forgetting_transformer/ops/forgetting_attention.py:505-693).
//
// One CTA = one (batch, head, 128-row query tile); two CTAs share an SM so that
// one CTA's softmax overlaps the other's matrix products.
//   warps 0 .. 4 NWG-1 : NWG softmax warpgroups; warpgroup g owns a BN / NWG wide column slice of every KV
//                        tile with its own running maximum, row sum and O accumulator; thread t of a
//                        warpgroup owns query row t and TMEM lane t (no cross-thread reductions)
//   next warp          : TMA producer (one elected lane); also stages the tile's gate prefixes
//   last warp          : tcgen05.mma issuer (one elected lane)
// TMEM: S = Q K^T fp32 in columns [0,BN); each slice's probabilities are written back over the slice's own
// S columns as packed 16-bit pairs and consumed as the TMEM A operand of P V; O_g accumulates in columns
// [BN + g D, BN + (g+1) D).  D = 64: BN = 128, NWG = 2 (256 columns); D = 128: BN = 128, NWG = 1 (256 columns).
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
// A tile whose logits are provably below (reference maximum + this many octaves) skips the maximum pass
// altogether: p <= 2^shift stays far inside fp32 / bf16 range (fp16 P: 2^14 < 65504).
constexpr float kSkipShiftBf16 = 32.0f, kSkipShiftFp16 = 14.0f;

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
  const float* k_norm_max;     // (B,H) max_t ||k[b,h,t,:]||_2, or nullptr: lets a tile skip its maximum pass
};

// How many of every 4 column pairs take the FMA-pipe exponential instead of the ex2 unit (measured best:
// a quarter at D=64, where four softmax warps share a scheduler, half at D=128 with two).
#ifndef FOX_POLYQ64
#define FOX_POLYQ64 1
#endif
#ifndef FOX_POLYQ128
#define FOX_POLYQ128 2
#endif

// Debug builds with -DFOX_FWD_TRACE record clock64 stamps of CTA (0,0,0), tiles 32..47:
// trace[(role * 8 + event) * 16 + tile - 32], role = softmax warp index or 8 for the MMA issuer.
#ifdef FOX_FWD_TRACE
__device__ long long g_fwd_trace[16 * 8 * 16];
#define STAMP(role, ev, it) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (it) >= 32 && (it) < 48) g_fwd_trace[((role) * 8 + (ev)) * 16 + (it) - 32] = clock64(); } while (0)
#else
#define STAMP(role, ev, it)
#endif

enum FwdWaitSite {
  kSiteQFull = 11, kSiteKFull = 12, kSiteVFull = 13, kSiteKEmpty = 14, kSiteVEmpty = 15,
  kSiteSFull = 16, kSitePFull = 17, kSiteODone = 18, kSiteDrain = 19, kSiteNegB = 20, kSiteMerge = 21, kSiteEpi = 22
};

template <int D, bool kBf16, int BN, int STAGES, int CTAS, int NWG, bool PREF>
__global__ void __launch_bounds__(128 * NWG + 64, CTAS)
fox_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                    const FwdParams p) {
  // KV tiles of BN rows (64 or 128; the pruning grid stays 128 wide, BN = 64 just walks it in halves).
  // NWG softmax warpgroups per CTA, each owning a BN / NWG wide column slice of every tile with its own
  // running maximum, row sum and O accumulator (independent online-softmax streams, merged in the
  // epilogue), so that several softmax warps per scheduler hide each other's ex2 / TMEM latency without
  // any exchange between the warpgroups inside the loop.
  constexpr int kWG = NWG;
  constexpr int CW = BN / kWG;              // columns per softmax thread
  constexpr int kQBytes = 128 * D * 2;      // Q tile: D/64 swizzled [128][64] sub-tiles
  constexpr int kTileBytes = BN * D * 2;    // K / V tile: D/64 swizzled [BN][64] sub-tiles
  constexpr int kSubBytes = BN * 128;       // one K / V sub-tile
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  constexpr uint32_t kColO = BN;            // S (fp32) in columns [0, BN), O_g in [BN + g D, BN + (g+1) D)
  constexpr uint32_t kTmemCols = (kColO + kWG * D <= 128) ? 128 : ((kColO + kWG * D <= 256) ? 256 : 512);
  static_assert(kColO + kWG * D <= 512, "TMEM budget");
  constexpr int kTmaWarp = 4 * kWG, kMmaWarp = 4 * kWG + 1;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full, bar_o_done, bar_merge, bar_epi;
  __shared__ uint64_t bar_s_full[NWG], bar_p_full[NWG];  // per warpgroup
  __shared__ uint64_t bar_k_full[STAGES], bar_k_empty[STAGES], bar_v_full[STAGES], bar_v_empty[STAGES];
  // -b_j = -Lambda_j log2(e) of a tile's columns and the maximum over each warpgroup's slice, staged by the
  // producer warp one tile ahead in a ring of three (slot of tile t is reused for t+3, which the producer
  // stages only after O += P V of tile t+1 or later has retired, i.e. after every reader of tile t is done)
  __shared__ uint64_t bar_negb[3];
  __shared__ __align__(16) float s_negb[3][BN];  // read as float4
  __shared__ float s_nbmax[3][NWG];
  __shared__ float s_mg[NWG][128], s_lg[NWG][128];  // every stream's (m, l) for the merge
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
    for (int g = 0; g < NWG; ++g) {
      mbar_init(&bar_s_full[g], 1);
      mbar_init(&bar_p_full[g], 128);
    }
    for (int i = 0; i < 3; ++i) mbar_init(&bar_negb[i], 1);
    mbar_init(&bar_o_done, 1);
    mbar_init(&bar_merge, 128 * NWG);
    mbar_init(&bar_epi, 128 * NWG);
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
      // K(it), V(it) per tile, each into stage it % STAGES once the product that read its previous
      // occupant has retired
      auto load_kv = [&](bool is_v, int it) -> bool {
        const int nb = nb_hi - 1 - it;
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        uint64_t* empty = is_v ? &bar_v_empty[st] : &bar_k_empty[st];
        uint64_t* full = is_v ? &bar_v_full[st] : &bar_k_full[st];
        STAMP(9, is_v ? 2 : 0, it);
        if (!mbar_wait_warp(empty, ph ^ 1, abortp, p.status, is_v ? kSiteVEmpty : kSiteKEmpty, it)) return false;
        STAMP(9, is_v ? 3 : 1, it);
        if (elect_one()) {
          mbar_expect_tx(full, kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d((is_v ? sV : sK) + st * kTileBytes + s * kSubBytes, is_v ? &tmV : &tmK, full, s * 64, nb * BN, h, b);
        }
        __syncwarp();
        return true;
      };
      // gate prefixes of a tile's columns: lane l holds columns 4l .. 4l+3 (lanes < BN/4)
      const float* lam = p.lam + (static_cast<int64_t>(b) * p.H + h) * N;
      // Prefixes enter the logits as differences Lambda_i - Lambda_j.  Both are taken relative to the prefix of
      // this query tile's first row BEFORE the scaling by log2(e): far into a strongly decaying sequence the
      // prefix reaches -1e4 and beyond, where scaling it first costs an absolute 2e-3 per logit.
      const float lam_ref = lam[min(P + mb * kFwdBM, N - 1)];
      float lamv[4] = {0.f, 0.f, 0.f, 0.f};
      auto fetch_lam = [&](int it) {
        const int c0 = (nb_hi - 1 - it) * BN + 4 * lane;
#pragma unroll
        for (int e = 0; e < 4; ++e) lamv[e] = (4 * lane < BN && c0 + e < N) ? ldg_f32_here(lam + c0 + e) : 0.f;
      };
      auto stage_negb = [&](int it) {  // from lamv, fetched earlier for this tile
        const int slot = it % 3;
        float4 nbv = make_float4((lam_ref - lamv[0]) * kLog2e, (lam_ref - lamv[1]) * kLog2e,
                                 (lam_ref - lamv[2]) * kLog2e, (lam_ref - lamv[3]) * kLog2e);
        if (4 * lane < BN) *reinterpret_cast<float4*>(&s_negb[slot][4 * lane]) = nbv;
        float mx = fmaxf(fmaxf(nbv.x, nbv.y), fmaxf(nbv.z, nbv.w));
#pragma unroll
        for (int o = CW / 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (4 * lane < BN && (4 * lane) % CW == 0) s_nbmax[slot][(4 * lane) / CW] = mx;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_negb[slot]);
        __syncwarp();
      };
      fetch_lam(0);
      stage_negb(0);
      if (n_tiles > 1) fetch_lam(1);
      for (int it = 0; it < n_tiles; ++it) {
        if (!load_kv(false, it)) break;
        ++issued;
        if (!load_kv(true, it)) break;  // waits for O += P V of tile it-STAGES
        ++issued;
        if (it + 1 < n_tiles) {
          stage_negb(it + 1);
          if (it + 2 < n_tiles) fetch_lam(it + 2);
        }
      }
      if (*abortp && lane == 0) {
        // error path only: let the copies already in flight land before the CTA retires (at most 2 STAGES
        // are outstanding; a wait on a phase that completed earlier returns at once or runs into the limit)
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_q_full, 0) && clock64() - t0 < 200000000LL) {
        }
        const int last = (issued + 1) / 2;  // tiles with at least one copy issued
        for (int it = max(last - STAGES - 1, 0); it < last; ++it) {
          const int st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          while (!mbar_try_wait(&bar_k_full[st], ph) && clock64() - t0 < 200000000LL) {
          }
          while (!mbar_try_wait(&bar_v_full[st], ph) && clock64() - t0 < 200000000LL) {
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer (whole warp converged, one elected lane issues) =====================
    if (n_tiles > 0) {
      constexpr uint32_t idPV = umma_idesc(kFmt, 128, D, 0, 1);
      // descriptors are built once; the loops only move the start-address field
      const uint64_t dQ = umma_desc_kmajor(smem_u32(sQ));
      const uint64_t dK0 = umma_desc_kmajor(smem_u32(sK));
      const uint64_t dV0 = umma_desc_mnmajor(smem_u32(sV), kSubBytes);
      bool ok = mbar_wait_warp(&bar_q_full, 0, abortp, p.status, kSiteQFull);
      {
        // Every softmax warpgroup g has its own chain S_g -> P_g -> O_g += P_g V_g -> S_g(next tile): the S
        // product is issued per column slice right behind the P V product that frees the slice, so a
        // warpgroup never waits for the other one.
        constexpr uint32_t idQK = umma_idesc(kFmt, 128, CW, 0, 0);
        auto issue_s = [&](int g, int st) {  // S[:, g CW : (g+1) CW] = Q K[g CW : (g+1) CW, :]^T
          const uint64_t dK = umma_desc_advance(dK0, st * kTileBytes + g * CW * 128);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_ss_raw(tbase + g * CW, umma_desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32),
                       umma_desc_advance(dK, (kk >> 2) * kSubBytes + (kk & 3) * 32), idQK, kk > 0);
          tc_commit_raw(&bar_s_full[g]);
        };
        ok = ok && mbar_wait_warp(&bar_k_full[0], 0, abortp, p.status, kSiteKFull, 0);
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int g = 0; g < kWG; ++g) issue_s(g, 0);
            tc_commit_raw(&bar_k_empty[0]);
          }
          __syncwarp();
        }
        for (int it = 0; it < n_tiles && ok; ++it) {
          const int st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const bool more = it + 1 < n_tiles;
          const int st1 = (it + 1) % STAGES;
          ok = mbar_wait_warp(&bar_v_full[st], ph, abortp, p.status, kSiteVFull, it);
          if (!ok) break;
          if (more) {
            ok = mbar_wait_warp(&bar_k_full[st1], ((it + 1) / STAGES) & 1, abortp, p.status, kSiteKFull, it + 1);
            if (!ok) break;
          }
          const uint64_t dV = umma_desc_advance(dV0, st * kTileBytes);
#pragma unroll
          for (int g = 0; g < kWG; ++g) {
            STAMP(8, (g & 1) * 3 + 0, it);
            ok = mbar_wait_warp(&bar_p_full[g], it & 1, abortp, p.status, kSitePFull, it);
            if (!ok) break;
            STAMP(8, (g & 1) * 3 + 1, it);
            tc_fence_after();
            if (elect_one()) {
              // O_g += P[:, g CW : (g+1) CW] V[g CW : (g+1) CW, :]; the 16-bit P sits at S columns g CW ...
#pragma unroll
              for (int kk = 0; kk < CW / 16; ++kk)
                mma_ts_raw(tbase + kColO + g * D, tbase + g * CW + kk * 8,
                           umma_desc_advance(dV, (g * (CW / 16) + kk) * 2048), idPV, (it > 0 || kk > 0) ? 1u : 0u);
              if (more) issue_s(g, st1);
              if (g == kWG - 1) {
                tc_commit_raw(&bar_v_empty[st]);
                if (more) tc_commit_raw(&bar_k_empty[st1]);
              }
            }
            __syncwarp();
            STAMP(8, (g & 1) * 3 + 2, it);
          }
          if (!ok) break;
        }
      }
      if (ok) tc_commit(&bar_o_done);
    }
  } else {
    // ===================== softmax / correction / epilogue =====================
    const int g = warp >> 2;                  // column slice owned by this warpgroup
    const int r = tid & 127;                  // query row inside the tile == TMEM lane
    const int row = mb * kFwdBM + r;
    const bool row_ok = row < M;
    const int64_t bh = static_cast<int64_t>(b) * p.H + h;
    const float* lam = p.lam + bh * N;
    const float a_i = row_ok ? (lam[P + row] - lam[min(P + mb * kFwdBM, N - 1)]) * kLog2e : 0.f;  // (see the producer)
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tbase + lane_base + g * CW;
    const uint32_t tO = tbase + lane_base + kColO + g * D;

    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    // Upper bound of this row's scaled logits q_i.k_j*c <= ||q_i|| max_j||k_j|| c (Cauchy-Schwarz): with the
    // largest -b_j of a tile it tells, before S is even read, that no logit of the tile can exceed the
    // reference maximum by more than the skip shift; then the maximum pass over S is not run.
    const bool dead = !row_ok || (P + row < seq0);  // rows without any valid column never need a maximum
    float qbound = INFINITY;
    if (p.k_norm_max != nullptr && n_tiles > 1) {
      ok = mbar_wait(&bar_q_full, 0, abortp, p.status, kSiteQFull);
      float ss = 0.f;
#pragma unroll
      for (int sub = 0; sub < kSub; ++sub) {
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 w = *reinterpret_cast<const uint4*>(sQ + sub * 16384 + r * 128 + ((ch ^ (r & 7)) << 4));
          const float2 f0 = unpack2<kBf16>(w.x), f1 = unpack2<kBf16>(w.y), f2 = unpack2<kBf16>(w.z), f3 = unpack2<kBf16>(w.w);
          ss = fmaf(f0.x, f0.x, ss); ss = fmaf(f0.y, f0.y, ss);
          ss = fmaf(f1.x, f1.x, ss); ss = fmaf(f1.y, f1.y, ss);
          ss = fmaf(f2.x, f2.x, ss); ss = fmaf(f2.y, f2.y, ss);
          ss = fmaf(f3.x, f3.x, ss); ss = fmaf(f3.y, f3.y, ss);
        }
      }
      qbound = sqrtf(ss) * p.k_norm_max[bh] * fabsf(p.qk_scale) * 1.0001f + a_i;
    }
    constexpr float kSkipShift = kBf16 ? kSkipShiftBf16 : kSkipShiftFp16;
    constexpr int kPolyQ = (D == 64) ? FOX_POLYQ64 : FOX_POLYQ128;
    const float2 scale2 = make_float2(p.qk_scale, p.qk_scale);
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int nb = nb_hi - 1 - it;
      const int col0 = nb * BN + g * CW;  // first column of this thread's slice
      STAMP(warp & 7, 0, it);
      ok = mbar_wait(&bar_negb[it % 3], (it / 3) & 1, abortp, p.status, kSiteNegB, it);
      ok = mbar_wait(&bar_s_full[g], it & 1, abortp, p.status, kSiteSFull, it) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      STAMP(warp & 7, 1, it);
      tc_fence_after();
      // Two passes over this thread's slice of S, 32 columns at a time, in packed two-wide fp32 arithmetic.
      // Both read S from TMEM (a TMEM load costs ~50 cycles; holding a 64/128-column slice in registers
      // costs spills):
      //   pass 1: u = s*scale - b_j (masked on boundary tiles), row maximum
      //   pass 2: p = 2^(s*scale - b_j + a_i - m), row sum, pack, write back over S
      const float4* nb4 = reinterpret_cast<const float4*>(&s_negb[it % 3][g * CW]);
      const bool need_mask = (col0 + CW - 1 > P + mb * kFwdBM) || (col0 < seq0) || (col0 + CW > N);
      // valid columns of this row inside the slice: [c_lo, c_hi]
      const int c_lo = need_mask ? max(seq0 - col0, 0) : 0;
      const int c_hi = need_mask ? (row_ok ? min(min(P + row, N - 1) - col0, CW - 1) : -1) : CW - 1;
      // S chunks of 32 columns go through two register buffers: with PREF the load of chunk ch+1 is issued
      // before chunk ch is worked on, which hides the TMEM latency at the price of 32 registers
      uint32_t sbuf[PREF ? 2 : 1][32];
      auto fetch = [&](int ch) { tmem_ld32(tS + ch * 32, sbuf[PREF ? (ch & 1) : 0]); };
      auto load_u = [&](int ch, float2* u, const bool with_add, const float2 add) {  // u[16] = 32 columns
        if (!PREF || ch == 0) fetch(ch);
        tmem_ld_wait();
        if (PREF && ch + 1 < CW / 32) fetch(ch + 1);
        const uint32_t* sreg = sbuf[PREF ? (ch & 1) : 0];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 nbv = nb4[ch * 8 + c4];
          float2 n0 = make_float2(nbv.x, nbv.y), n1 = make_float2(nbv.z, nbv.w);
          if (with_add) {
            n0 = __fadd2_rn(n0, add);
            n1 = __fadd2_rn(n1, add);
          }
          u[2 * c4 + 0] = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4 + 0]), __uint_as_float(sreg[4 * c4 + 1])), scale2, n0);
          u[2 * c4 + 1] = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4 + 2]), __uint_as_float(sreg[4 * c4 + 3])), scale2, n1);
        }
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const int cc = ch * 32 + 2 * c;
            u[c].x = (cc >= c_lo && cc <= c_hi) ? u[c].x : -INFINITY;
            u[c].y = (cc + 1 >= c_lo && cc + 1 <= c_hi) ? u[c].y : -INFINITY;
          }
        }
      };
      const float nbmax = s_nbmax[it % 3][g];
      // (NaN or -inf reference -> false -> the maximum pass runs)
      const bool skip1 = __all_sync(0xffffffffu, dead || (qbound + nbmax <= m_ref + kSkipShift));
      if (!skip1) {
        float umax = -INFINITY;
#pragma unroll
        for (int ch = 0; ch < CW / 32; ++ch) {
          float2 u[16];
          load_u(ch, u, false, make_float2(0.f, 0.f));
#pragma unroll
          for (int c = 0; c < 16; ++c) umax = fmax3(umax, u[c].x, u[c].y);
        }
        STAMP(warp & 7, 2, it);
        // ---- running maximum with lazy rescaling ----
        const float m_new = fmaxf(m_ref, a_i + umax);
        const bool need = (m_new - m_ref) > kLazyShift;  // false when both are -inf (NaN compare)
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_ref - m_new);
          l_sum *= alpha;
          if (it > 0) {
            const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
            for (int c = 0; c < D; c += 32) {
              uint32_t o[32];
              tmem_ld32(tO + c, o);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float2 t = __fmul2_rn(make_float2(__uint_as_float(o[j]), __uint_as_float(o[j + 1])), alpha2);
                o[j] = __float_as_uint(t.x);
                o[j + 1] = __float_as_uint(t.y);
              }
              tmem_st32(tO + c, o);
            }
          }
          m_ref = m_new;
        }
      }
      STAMP(warp & 7, 3, it);
      const float off = a_i - ((m_ref == -INFINITY) ? 0.f : m_ref);
      const float2 off2 = make_float2(off, off);
      float2 psum = make_float2(0.f, 0.f);
#pragma unroll
      for (int ch = 0; ch < CW / 32; ++ch) {
        float2 u[16];
        load_u(ch, u, true, off2);
        uint32_t pk[16];
        if (kPolyQ > 0 && !need_mask) {
          // kPolyQ of every 4 column pairs take the FMA-pipe exponential instead of the ex2 unit
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 pp = ((j & 3) < kPolyQ) ? poly_exp2_x2(u[j]) : make_float2(fast_exp2(u[j].x), fast_exp2(u[j].y));
            psum = __fadd2_rn(psum, pp);
            pk[j] = pack2<kBf16>(pp.x, pp.y);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 pp = make_float2(fast_exp2(u[j].x), fast_exp2(u[j].y));
            psum = __fadd2_rn(psum, pp);
            pk[j] = pack2<kBf16>(pp.x, pp.y);
          }
        }
        tmem_st16(tS + ch * 16, pk);  // columns already consumed by this thread
      }
      l_sum += psum.x + psum.y;
      STAMP(warp & 7, 4, it);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_p_full[g]);
      STAMP(warp & 7, 5, it);
    }

    // ---- epilogue: merge the streams, O / l -> 16-bit -> global, L = m ln2 + ln l ----
    // every warpgroup publishes its (m, l); all of them form the same merge weights and each writes the
    // 32-column chunks c with (c / 32) % NWG == g
    if (NWG > 1) {
      s_mg[g][r] = m_ref;
      s_lg[g][r] = l_sum;
      mbar_arrive(&bar_merge);
    }
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_o_done, 0, abortp, p.status, kSiteODone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (NWG > 1 && ok) {
      ok = mbar_wait(&bar_merge, 0, abortp, p.status, kSiteMerge);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      float w[NWG];
      w[0] = 1.f;
      if (NWG > 1) {
        float m = -INFINITY;
#pragma unroll
        for (int q = 0; q < NWG; ++q) m = fmaxf(m, s_mg[q][r]);
        float l = 0.f;
#pragma unroll
        for (int q = 0; q < NWG; ++q) {
          const float mq = s_mg[q][r];
          w[q] = (mq == -INFINITY) ? 0.f : fast_exp2(mq - m);
          l = fmaf(s_lg[q][r], w[q], l);
        }
        l_sum = l;
        m_ref = m;
      }
      const bool empty = (n_tiles == 0) || (P + row < seq0) || !(l_sum > 0.f);
      const float inv_l = empty ? 0.f : 1.f / l_sum;
#pragma unroll
      for (int q = 0; q < NWG; ++q) w[q] *= inv_l;
      // The 16-bit tile goes through shared memory (Q is idle: every product has retired) and leaves as TMA
      // stores, which write whole lines and clip the rows past M.
      const uint32_t tO0 = tbase + lane_base + kColO;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        if ((c / 32) % NWG != g) continue;  // (with more warpgroups than chunks the surplus ones write nothing)
        float o[32];
        if (n_tiles > 0) {
#pragma unroll
          for (int q = 0; q < NWG; ++q) {
            uint32_t t0[32];
            tmem_ld32(tO0 + q * D + c, t0);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = q == 0 ? __uint_as_float(t0[j]) * w[0] : fmaf(__uint_as_float(t0[j]), w[q], o[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 wv = make_uint4(0, 0, 0, 0);
          if (!empty) {
            wv.x = pack2<kBf16>(o[j + 0], o[j + 1]);
            wv.y = pack2<kBf16>(o[j + 2], o[j + 3]);
            wv.z = pack2<kBf16>(o[j + 4], o[j + 5]);
            wv.w = pack2<kBf16>(o[j + 6], o[j + 7]);
          }
          *reinterpret_cast<uint4*>(sQ + (c >> 6) * 16384 + r * 128 + (((((c & 63) + j) >> 3) ^ (r & 7)) << 4)) = wv;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&bar_epi);
      if (warp == 0) {
        // (a bounded wait like every other one: a warp that gave up elsewhere never arrives)
        if (mbar_wait_warp(&bar_epi, 0, abortp, p.status, kSiteEpi) && elect_one()) {
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) tma_store_4d(&tmO, sQ + sub * 16384, sub * 64, mb * kFwdBM, h, b);
          tma_store_commit();
          tma_store_wait_read<0>();   // the tile must stay in shared memory until it has been read
        }
        __syncwarp();
      }
      if (row_ok && g == 0) p.L[bh * M + row] = empty ? -INFINITY : m_ref * kLn2 + __logf(l_sum);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tbase, kTmemCols);
}

// Shapes: D=64 -> 128-row KV tiles in two stages, two softmax warpgroups with independent streams;
// D=128 -> 128-row KV tiles in a single K and a single V buffer (K is free again once S is computed, V once
// P V is, so the next tile's copies overlap the softmax), one softmax warpgroup, S chunks prefetched.
#ifdef FOX_DEBUG
// Debug builds (-DFOX_DEBUG) only, tuning hook: 1 = D=64 with one warpgroup, 2 = D=128 with 64-row KV tiles in two stages.
static int g_fwd_variant = 0;
#endif
#ifdef FOX_FWD_TRACE
extern "C" int fox_debug_read_fwd_trace(long long* host) {
  return cudaMemcpyFromSymbol(host, g_fwd_trace, sizeof(g_fwd_trace));
}
#endif

template <bool kBf16, int D, int BN, int STAGES, int CTAS, int NWG, bool PREF>
static int launch_fwd_t(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
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
  CUtensorMap tmO;
  Tensor4 to{prm.o, B, H, M, D, prm.o_sb, prm.o_sh, prm.o_st};
  if (!tma_compatible(to, 2)) return FOX_ERR_ALIGNMENT;
  if ((rc = cached_tmap_4d(&tmO, to, 2, false, kBf16, 64, 128, true))) return rc;
  constexpr int smem = 128 * D * 2 + 2 * STAGES * BN * D * 2 + 1024;
  auto kern = fox_attn_fwd_kernel<D, kBf16, BN, STAGES, CTAS, NWG, PREF>;
  static bool configured[64] = {};  // per template instance and device
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[device] = true;
  }
  dim3 grid((unsigned)((M + kFwdBM - 1) / kFwdBM), (unsigned)H, (unsigned)B);
  kern<<<grid, 128 * NWG + 64, smem, stream>>>(tmQ, tmK, tmV, tmO, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

template <int... A>
static int launch_fwd(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
                      const fox_tensor4* k, const fox_tensor4* v, const FwdParams& prm) {
  return launch_fwd_t<true, A...>(device, stream, B, H, M, N, q, k, v, prm);
}
template <int... A>
static int launch_fwd_fp16(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
                           const fox_tensor4* k, const fox_tensor4* v, const FwdParams& prm) {
  return launch_fwd_t<false, A...>(device, stream, B, H, M, N, q, k, v, prm);
}

}  // namespace fox

#ifdef FOX_DEBUG
extern "C" void fox_debug_set_fwd_variant(int v) { fox::g_fwd_variant = v; }
#endif

extern "C" int fox_attn_fwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                            int64_t D, const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                            const float* log_lambda, const int64_t* seq_start, const int64_t* start_index,
                            float sm_scale, const fox_tensor4* o, float* L, const float* k_norm_max,
                            int32_t* status) {
  using namespace fox;
  if (!q || !k || !v || !o || !q->ptr || !k->ptr || !v->ptr || !o->ptr || !log_lambda || !L || !status)
    return FOX_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || M <= 0 || N <= 0 || M > N || H > 65535 || B > 65535) return FOX_ERR_BAD_ARG;
  if (N > 2147483647LL) return FOX_ERR_TOO_LARGE;   // row indices are 32-bit inside the kernels (M <= N)
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
  prm.k_norm_max = k_norm_max;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = dtype == FOX_DTYPE_BF16;
#ifdef FOX_DEBUG
  const int variant = g_fwd_variant;
#endif
#define FOX_FWD_LAUNCH(...) \
  (bf ? launch_fwd<__VA_ARGS__>(device, st, B, H, M, N, q, k, v, prm) : launch_fwd_fp16<__VA_ARGS__>(device, st, B, H, M, N, q, k, v, prm))
  //                 D  BN  STAGES CTAS NWG PREF
#ifdef FOX_DEBUG
  if (D == 64 && variant == 1) return FOX_FWD_LAUNCH(64, 128, 2, 2, 1, false);
  if (D == 128 && variant == 2) return FOX_FWD_LAUNCH(128, 64, 2, 2, 1, false);
#endif
  if (D == 64) return FOX_FWD_LAUNCH(64, 128, 2, 2, 2, false);
  return FOX_FWD_LAUNCH(128, 128, 1, 2, 1, true);
#undef FOX_FWD_LAUNCH
}
