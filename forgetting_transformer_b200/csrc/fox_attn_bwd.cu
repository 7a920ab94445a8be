// Forgetting Attention backward for sm_100a: one pass over the (query tile, KV
// tile) pairs with five tcgen05 matrix products per pair and a single exp2.
//
// Stands in for upstream's Triton `_bwd_kv_kernel` and `_bwd_q_kernel`
// (src/forgetting_transformer/ops/forgetting_attention.py:956-1143, 1156-1344),
// which recompute S and dP twice (seven products per pair).
//
// One CTA = one (batch, head, 128-row KV tile); it keeps K and V resident and
// streams the query tiles from the causal diagonal downwards.  704 threads:
//   warps 0-15 : compute.  Warp (g = warp/4, quarter = warp%4) owns KV rows [32 quarter, +32) (TMEM lanes of
//                S^T / dP^T) x query columns [32g, 32g+32) of the tile and reads them as matrix fragments
//                (tcgen05.ld 16x256b): a thread holds 4 KV rows x 4 column pairs.  Four warps per scheduler
//                are what it takes to keep the ex2 unit busy.
//   warp  16   : TMA producer (also stages the per-row vectors)    warp 17 : tcgen05.mma issuer
//   warps 18-21: dQ drain.  Thread owns one query row of the dQ tile accumulator: TMEM ->
//                swizzled shared memory -> TMA add-reduction into the fp32 workspace.
// Per pair i (all products 128-wide, fp32 accumulation in TMEM):
//   S^T = K Q^T ; dP^T = V dO^T                         (smem x smem)
//   phase A: P^T = 2^(S^T c + (L_i-corrected bias))      -> 16-bit, written over S^T
//   phase B: dS^T = P^T (dP^T - delta)                   -> 16-bit, over dP^T and to smem
//   dV += P^T dO ; dK += dS^T Q                          (TMEM x smem)
//   dQ_i = dS [K | 1]                                    (smem x smem, fresh accumulator)
// The tensor pipe and the compute warps overlap: while phase B(i) runs the pipe does
// dV(i) and S(i+1); while phase A(i+1) runs it does dK(i), dP(i+1), dQ(i) (D = 128, where the dQ
// accumulator has to share columns with S^T / dP^T: dK(i), dQ(i), drain, S(i+1), dP(i+1)).
// The two halves of the log-gate gradient, colsum(dS) per key and rowsum(dS) per query, are sums of the fp32
// dS values, as upstream's are (lines 1122, 1326).  With the fragment layout a thread's column sums (over the
// query index) are running sums of its four KV rows, joined across the four threads of a row once per launch;
// the row sum of a tile (over the KV index) is a sum over the thread's four rows followed by a transposing
// reduction across the eight threads that share a column pair (7 shuffles leave each thread with one query
// column's sum), done after dS has been handed to the tensor pipe and added to the fp32 workspace.  Both halves
// sum the same values, so they cancel in the reverse prefix sum as upstream's do; against upstream's own backward
// kernels on the same saved tensors the gate gradient then agrees to 1e-4.
// Measured on B2 T16384 H24 D64: 4.18 ms.  With one KV row per thread (tcgen05.ld 32x32b: 32 columns of one
// lane) the same sums took a 31-shuffle, 62-select reduction per warp and tile and the kernel 4.96 ms; that
// layout with the sums taken from 16 "ones" columns appended to K and Q (the dQ and dK products then deliver
// sums of the 16-bit dS values for free: FOX_BWD_FP32_SUMS=0) took 4.23 ms but left the gate gradient 2-4e-2
// off upstream's, up to 1.8 times the tolerance: the rounding of dS to 8 significant bits, summed over the
// (query, key) pairs that straddle a position.  Writing dS as fp16 for bf16 inputs, to keep the free sums at
// 11 significant bits, is not an option: a kind::f16 product whose A and B operands differ in format raises an
// illegal-instruction error on sm_100a.
#include <type_traits>

#include "fox_common.cuh"
#include "fox_host.h"

#ifndef FOX_BWD_FP32_SUMS
#define FOX_BWD_FP32_SUMS 1
#endif
// of a thread's 16 column pairs per tile, how many take the FMA-pipe exponential instead of the ex2 unit
// (only on tiles off the diagonal whose KV rows are all valid)
#ifndef FOX_BWD_POLY
#define FOX_BWD_POLY 0
#endif

namespace fox {

constexpr int kBwdBM = FOX_BWD_BLOCK_M;
constexpr int kBwdBN = FOX_BWD_BLOCK_N;
constexpr float kLog2eB = 1.4426950408889634f;

struct BwdParams {
  const float* lam;          // (B,H,N)
  const float* L;            // (B,H,M) log normaliser from the forward
  const float* delta;        // (B,H,M)
  const int64_t* seq_start;  // (B,) or nullptr
  const int64_t* end_index;  // (B,H,ceil(N/128)) or nullptr
  float* dq_accum;           // (B,H,M,D) fp32, zero-initialised
  float* dlam_row;           // (B,H,M) fp32, zero-initialised
  float* dlam_col;           // (B,H,N) fp32, fully written
  void* dk; int64_t dk_sb, dk_sh, dk_st;
  void* dv; int64_t dv_sb, dv_sh, dv_st;
  int* status;
  long long* trace;          // optional (debug builds of the kernel only): clock64 stamps of CTA (0,0,0)
  int H, M, N;
  float sm_scale, qk_scale;
};

enum BwdWaitSite {
  kBSiteKV = 31, kBSiteQFull = 32, kBSiteQEmpty = 33, kBSiteSFull = 34, kBSitePDone = 35, kBSiteDq = 36,
  kBSiteVec = 37, kBSiteDone = 38, kBSiteDqFree = 39, kBSiteDOFull = 40, kBSiteDOEmpty = 41, kBSiteDpFull = 42,
  kBSiteDsDone = 43, kBSiteDsmFree = 44, kBSiteColsum = 45, kBSiteStaged = 46, kBSiteStageFree = 47, kBSiteEpi = 48
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int D, bool kBf16, bool kTrace, int kCWG, bool kNoDQ>
__global__ void __launch_bounds__((4 * kCWG + 6) * 32, 1)
fox_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                    const __grid_constant__ CUtensorMap tmDV, const BwdParams p) {
  constexpr int kTileBytes = 128 * D * 2;
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  // kNoDQ: dK, dV and the key-side gate gradient only (dQ comes from fox_attn_bwd_dq_kernel): no dQ product, no
  // drain, no reductions, and at D = 128 no sharing of TMEM columns
  constexpr bool kAliasDQ = (D == 128) && !kNoDQ;  // dQ accumulator shares columns with S^T / dP^T
  constexpr bool kFp32Sums = FOX_BWD_FP32_SUMS != 0;            // gate-gradient sums of the fp32 dS values
  constexpr bool kColsumMMA = (D == 64) && !kNoDQ && !kFp32Sums;  // colsum(dS) from the dK product
  constexpr int STQ = 2;
  constexpr int STDO = (D == 64) ? 2 : 1;
  constexpr int kDsBufs = (D == 64) ? 2 : 1;
  constexpr int kStageSub = (D == 64) ? 2 : 1;  // 32-column fp32 sub-tiles of the dQ staging buffer
  // warp roles: kCWG compute warpgroups (each owns CW query columns of the tile), producer, issuer, 4 drain warps
  constexpr int CW = 128 / kCWG;
  constexpr int kTmaWarp = 4 * kCWG, kMmaWarp = 4 * kCWG + 1, kDrainWarp0 = 4 * kCWG + 2;
  constexpr uint32_t kTmemCols = 512;
  constexpr int kNdk = kColsumMMA ? D + 16 : D;
  constexpr int kNdq = kFp32Sums ? D : D + 16;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 256 + kNdk;
  constexpr uint32_t kColDQ = kAliasDQ ? 0 : kColDV + D;
  // With the sums off the tensor pipe (no "ones" columns) a second dQ accumulator fits at D = 64: the dQ product
  // of the next tile then runs while this tile's accumulator is still being drained and add-reduced into L2.
  constexpr int kDqBufs = (D == 64 && kFp32Sums && !kNoDQ) ? 2 : 1;
  static_assert(kAliasDQ || kNoDQ || kColDQ + kDqBufs * kNdq <= 512, "TMEM budget");

  // 1024-byte aligned by declaration: at D=128 the tiles use all but 3 KiB of the 227 KiB a CTA may
  // have, so there is no room for a manual alignment slack.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_dq_full[kDqBufs], bar_dq_free[kDqBufs];
  __shared__ uint64_t bar_kv, bar_s_full, bar_dp_full, bar_p_done, bar_ds_done, bar_done,
      bar_colsum;
  __shared__ uint64_t bar_q_full[STQ], bar_q_empty[STQ], bar_do_full[STDO], bar_do_empty[STDO],
      bar_staged, bar_stage_free, bar_epi[2];
  __shared__ __align__(16) float s_e[STQ][kBwdBM];      // per Q stage; read as float4
  __shared__ __align__(16) float s_delta[STQ][kBwdBM];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* smem = smem_raw;
  // The "ones" tile directly follows K (it is K's next 64-column block for the dQ product) and
  // lies above the Q stages (whose descriptors reach it through their leading-dimension offset).
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + STQ * kTileBytes;
  uint8_t* sK = sDO + STDO * kTileBytes;
  uint8_t* sOnes = sK + kTileBytes;
  uint8_t* sV = sOnes + 16384;
  uint8_t* sdS = sV + kTileBytes;                 // kDsBufs x [128 kv][128 q] (two 64-wide sub-tiles each)
  uint8_t* sStage = sdS + kDsBufs * 32768;        // kStageSub x [128 q][32 fp32], 128-byte swizzled, for the dQ reduction

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int M = p.M, N = p.N, P = N - M;
  const int64_t bh = static_cast<int64_t>(b) * p.H + h;
  const int seq0 = p.seq_start ? static_cast<int>(p.seq_start[b]) : 0;

  // ---- query-tile range of this KV tile (upstream lines 1003-1049) ----
  int lo = max(nb * kBwdBN - P, 0);
  lo = (lo / kBwdBM) * kBwdBM;
  int hi = M;
  if (p.end_index) {
    const int64_t e = p.end_index[bh * gridDim.x + nb];
    hi = static_cast<int>(e < static_cast<int64_t>(M) ? e : static_cast<int64_t>(M));
  }
  if (p.seq_start && !(nb * kBwdBN + kBwdBN >= seq0 - 1)) hi = lo;
  const int mb_lo = lo / kBwdBM;
  const int mb_hi = (hi + kBwdBM - 1) / kBwdBM;
  const int n_tiles = max(mb_hi - mb_lo, 0);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_kv, 1);
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_dp_full, 1);
    mbar_init(&bar_p_done, 128 * kCWG);
    mbar_init(&bar_ds_done, 128 * kCWG);
    for (int s = 0; s < kDqBufs; ++s) { mbar_init(&bar_dq_full[s], 1); mbar_init(&bar_dq_free[s], 128); }
    mbar_init(&bar_done, 1);
    mbar_init(&bar_colsum, 128 * kCWG);
    // q_full: the TMA transaction plus one arrival of the producer warp for the per-row vectors
    for (int s = 0; s < STQ; ++s) { mbar_init(&bar_q_full[s], 2); mbar_init(&bar_q_empty[s], 1); }
    for (int s = 0; s < STDO; ++s) { mbar_init(&bar_do_full[s], 1); mbar_init(&bar_do_empty[s], 1); }
    mbar_init(&bar_epi[0], 64 * kCWG);
    mbar_init(&bar_epi[1], 64 * kCWG);
    mbar_init(&bar_staged, 128);
    mbar_init(&bar_stage_free, 1);
    mbar_fence_init();
  }
  if (warp == kTmaWarp) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp < 4 && !kFp32Sums) {
    // "ones" sub-tile: 16-bit 1.0 in columns 0..15 of every row, zero elsewhere
    const uint32_t one2 = kBf16 ? 0x3F803F80u : 0x3C003C00u;
    const uint4 ones = make_uint4(one2, one2, one2, one2), zeros = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int cj = 0; cj < 8; ++cj)
      *reinterpret_cast<uint4*>(sOnes + tid * 128 + ((cj ^ (tid & 7)) << 4)) = cj < 2 ? ones : zeros;
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_slot;
  volatile int* abortp = &abort_flag;
  // debug time stamps: trace[(role * 64 + event) * 16 + tile] for the first 16 tiles of CTA (0,0,0)
  auto stamp = [&](int role, int event, int it) {
    if (kTrace && p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && it < 16)
      p.trace[(role * 8 + event) * 16 + it] = clock64();
  };

  if (warp == kTmaWarp) {
    // ===================== TMA producer (whole warp converged, one elected lane issues) =====================
    if (n_tiles > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmDO);
        mbar_expect_tx(&bar_kv, 2 * kTileBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
          tma_load_4d(sK + s * 16384, &tmK, &bar_kv, s * 64, nb * kBwdBN, h, b);
          tma_load_4d(sV + s * 16384, &tmV, &bar_kv, s * 64, nb * kBwdBN, h, b);
        }
      }
      __syncwarp();
      // Per-row vectors of a query tile (L_i, Lambda_i, delta_i: lane l holds rows rr*32 + l) are fetched two
      // tiles ahead into one of two register sets with loads that stay where they are written, and only
      // combined when they are staged: a global load here sees well over a thousand cycles of latency
      // while the reductions are in flight, and anything the producer waits for delays every copy behind it.
      // (prefixes relative to this KV tile's first key before the scaling by log2(e): see b_j below)
      const float lam_ref = p.lam[bh * N + min(nb * kBwdBN, N - 1)];
      float rawL[2][kBwdBM / 32], rawLam[2][kBwdBM / 32], rawD[2][kBwdBM / 32];
      auto fetch_vec = [&](int mb_, auto slot_c) {
        constexpr int slot = decltype(slot_c)::value;
#pragma unroll
        for (int rr = 0; rr < kBwdBM / 32; ++rr) {
          const int i = mb_ * kBwdBM + rr * 32 + lane;
          const bool in = i < M;
          const int ic = in ? i : 0;
          const float l_ = ldg_f32_here(p.L + bh * M + ic);
          const float a_ = ldg_f32_here(p.lam + bh * N + P + ic);
          const float d_ = ldg_f32_here(p.delta + bh * M + ic);
          rawL[slot][rr] = in ? l_ : -INFINITY;
          rawLam[slot][rr] = a_;
          rawD[slot][rr] = in ? d_ : 0.f;
        }
      };
      int issued_q = 0, issued_do = 0;
      auto tile = [&](int it, auto slot_c) -> bool {
        constexpr int slot = decltype(slot_c)::value;
        const int mb = mb_lo + it;
        const int st = it % STQ;
        if (!mbar_wait_warp(&bar_q_empty[st], ((it / STQ) & 1) ^ 1, abortp, p.status, kBSiteQEmpty, it)) return false;
        if (elect_one()) {
          mbar_expect_tx(&bar_q_full[st], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(sQ + st * kTileBytes + s * 16384, &tmQ, &bar_q_full[st], s * 64, mb * kBwdBM, h, b);
        }
        __syncwarp();
        issued_q = it + 1;
        const int sd = it % STDO;
        if (!mbar_wait_warp(&bar_do_empty[sd], ((it / STDO) & 1) ^ 1, abortp, p.status, kBSiteDOEmpty, it)) return false;
        if (elect_one()) {
          mbar_expect_tx(&bar_do_full[sd], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s)
            tma_load_4d(sDO + sd * kTileBytes + s * 16384, &tmDO, &bar_do_full[sd], s * 64, mb * kBwdBM, h, b);
        }
        __syncwarp();
        issued_do = it + 1;
        // e_i = (Lambda_i - L_i) log2 e (-inf for an empty or out-of-range row) and delta_i go into the Q
        // stage's vectors.  Consumers reach them through s_full, which the MMA warp commits only after it
        // has seen q_full.
#pragma unroll
        for (int rr = 0; rr < kBwdBM / 32; ++rr) {
          const float Li = rawL[slot][rr];
          s_e[st][rr * 32 + lane] = (Li == -INFINITY) ? -INFINITY : ((rawLam[slot][rr] - lam_ref) - Li) * kLog2eB;
          s_delta[st][rr * 32 + lane] = -rawD[slot][rr];   // (phase B adds it)
        }
        __syncwarp();
        if (elect_one()) mbar_arrive(&bar_q_full[st]);
        __syncwarp();
        if (it + 2 < n_tiles) fetch_vec(mb + 2, slot_c);
        return true;
      };
      fetch_vec(mb_lo, std::integral_constant<int, 0>{});
      if (n_tiles > 1) fetch_vec(mb_lo + 1, std::integral_constant<int, 1>{});
      for (int it = 0; it < n_tiles; it += 2) {
        if (!tile(it, std::integral_constant<int, 0>{})) break;
        if (it + 1 < n_tiles && !tile(it + 1, std::integral_constant<int, 1>{})) break;
      }
      if (*abortp && lane == 0) {
        // error path only: let the copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_kv, 0) && clock64() - t0 < 200000000LL) {
        }
        for (int it = max(issued_q - STQ, 0); it < issued_q; ++it)
          while (!mbar_try_wait(&bar_q_full[it % STQ], (it / STQ) & 1) && clock64() - t0 < 200000000LL) {
          }
        for (int it = max(issued_do - STDO, 0); it < issued_do; ++it)
          while (!mbar_try_wait(&bar_do_full[it % STDO], (it / STDO) & 1) && clock64() - t0 < 200000000LL) {
          }
      }
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer (whole warp converged, one elected lane issues) =====================
    if (n_tiles > 0) {
      constexpr uint32_t idS = umma_idesc(kFmt, 128, 128, 0, 0);
      constexpr uint32_t idDV = umma_idesc(kFmt, 128, D, 0, 1);
      constexpr uint32_t idDK = umma_idesc(kFmt, 128, kNdk, 0, 1);
      constexpr uint32_t idDQ = umma_idesc(kFmt, 128, kNdq, 1, 1);
      // Operand descriptors are built once; inside the loops only the start-address field moves
      // (the issuing thread must stay far ahead of the tensor pipe, so its instruction count matters).
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), ones0 = smem_u32(sOnes);
      const uint64_t dK_k = umma_desc_kmajor(smem_u32(sK));            // S^T : A = K
      const uint64_t dV_k = umma_desc_kmajor(smem_u32(sV));            // dP^T: A = V
      const uint64_t dK_mn = umma_desc_mnmajor(smem_u32(sK), 16384);   // dQ  : B = [K | 1]
      const uint64_t dQ_k = umma_desc_kmajor(q_base);                  // S^T : B = Q (stage 0)
      const uint64_t dDO_k = umma_desc_kmajor(do_base);                // dP^T: B = dO (stage 0)
      const uint64_t dDO_mn = umma_desc_mnmajor(do_base, 16384);       // dV  : B = dO (stage 0)
      const uint64_t dDS_mn = umma_desc_mnmajor(smem_u32(sdS), 16384); // dQ  : A = dS (buffer 0)
      // dK: B = [Q | 1]; the ones tile is reached through the leading offset, which depends on the stage
      uint64_t dQ_mn[STQ];
#pragma unroll
      for (int s_ = 0; s_ < STQ; ++s_)
        dQ_mn[s_] = umma_desc_mnmajor(q_base + s_ * kTileBytes, kColsumMMA ? (ones0 - (q_base + s_ * kTileBytes)) : 16384u);
      auto issue_S = [&](int it) -> bool {
        const int st = it % STQ;
        if (!mbar_wait_warp(&bar_q_full[st], (it / STQ) & 1, abortp, p.status, kBSiteQFull, it)) return false;
        tc_fence_after();
        const uint64_t bq = umma_desc_advance(dQ_k, st * kTileBytes);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            mma_ss_raw(tbase + kColS, umma_desc_advance(dK_k, off), umma_desc_advance(bq, off), idS, kk > 0);
          }
          tc_commit_raw(&bar_s_full);
        }
        __syncwarp();
        return true;
      };
      auto issue_dP = [&](int it) -> bool {
        const int st = it % STDO;
        if (!mbar_wait_warp(&bar_do_full[st], (it / STDO) & 1, abortp, p.status, kBSiteDOFull, it)) return false;
        tc_fence_after();
        const uint64_t bdo = umma_desc_advance(dDO_k, st * kTileBytes);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            mma_ss_raw(tbase + kColDP, umma_desc_advance(dV_k, off), umma_desc_advance(bdo, off), idS, kk > 0);
          }
          tc_commit_raw(&bar_dp_full);
        }
        __syncwarp();
        return true;
      };
      bool ok = mbar_wait_warp(&bar_kv, 0, abortp, p.status, kBSiteKV);
      ok = ok && issue_S(0) && issue_dP(0);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const uint32_t acc = it > 0 ? 1u : 0u;
        const uint64_t bdo_mn = umma_desc_advance(dDO_mn, (it % STDO) * kTileBytes);
        const uint64_t bq_mn = dQ_mn[it % STQ];
        const uint64_t ads_mn = umma_desc_advance(dDS_mn, (it % kDsBufs) * 32768);
        // ---- dV += P^T dO (P^T in TMEM: query columns [0,64) at S columns 0.., [64,128) at 64..) ----
        stamp(0, 0, it);
        ok = mbar_wait_warp(&bar_p_done, it & 1, abortp, p.status, kBSitePDone, it);
        if (!ok) break;
        stamp(0, 1, it);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts_raw(tbase + kColDV, tbase + kColS + ((kk * 16) / CW) * CW + ((kk * 16) % CW) / 2,
                       umma_desc_advance(bdo_mn, kk * 2048), idDV, acc | (kk > 0));
          tc_commit_raw(&bar_do_empty[it % STDO]);
        }
        __syncwarp();
        if (!kAliasDQ && it + 1 < n_tiles) {
          ok = issue_S(it + 1);  // overwrites P^T(it): ordered behind dV(it) in the tensor pipe
          if (!ok) break;
          stamp(0, 7, it);
        }
        // ---- dK += dS^T [Q | 1] ----
        stamp(0, 2, it);
        ok = mbar_wait_warp(&bar_ds_done, it & 1, abortp, p.status, kBSiteDsDone, it);
        if (!ok) break;
        stamp(0, 3, it);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts_raw(tbase + kColDK, tbase + kColDP + ((kk * 16) / CW) * CW + ((kk * 16) % CW) / 2,
                       umma_desc_advance(bq_mn, kk * 2048), idDK, acc | (kk > 0));
          tc_commit_raw(&bar_q_empty[it % STQ]);  // dK is the last reader of this Q stage
        }
        __syncwarp();
        if (!kAliasDQ && it + 1 < n_tiles) {
          // dP^T(it+1) overwrites dS^T(it), whose only reader in TMEM is dK(it): it goes ahead of dQ(it), so that
          // a slow drain of the previous dQ tile (the wait below) does not hold up the next tile's phase B
          stamp(0, 5, it);
          ok = issue_dP(it + 1);
          if (!ok) break;
          stamp(0, 6, it);
        }
        // ---- dQ_tile = dS [K | 1] ----
        if (!kNoDQ && it > 0) {
          // (accumulator it % kDqBufs was last used by tile it - kDqBufs)
          if (it >= kDqBufs)
            ok = mbar_wait_warp(&bar_dq_free[it % kDqBufs], ((it - kDqBufs) / kDqBufs) & 1, abortp, p.status,
                                kBSiteDqFree, it);
          if (!ok) break;
          tc_fence_after();
        }
        if (!kNoDQ && elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ss_raw(tbase + kColDQ + (it % kDqBufs) * kNdq, umma_desc_advance(ads_mn, kk * 2048), umma_desc_advance(dK_mn, kk * 2048),
                       idDQ, kk > 0);
          tc_commit_raw(&bar_dq_full[it % kDqBufs]);
        }
        __syncwarp();
        stamp(0, 4, it);
        if (it + 1 < n_tiles) {
          if (kAliasDQ) {
            // the dQ tile sits on the S^T / dP^T columns: wait until it has been drained
            ok = mbar_wait_warp(&bar_dq_free[0], it & 1, abortp, p.status, kBSiteDqFree, it);
            if (!ok) break;
            tc_fence_after();
            ok = issue_S(it + 1);
            if (!ok) break;
          }
          if (kAliasDQ) {
            stamp(0, 5, it);
            ok = issue_dP(it + 1);  // overwrites dS^T(it): ordered behind dK(it)
            if (!ok) break;
            stamp(0, 6, it);
          }
        }
      }
      if (ok) tc_commit(&bar_done);
    }
  } else if (warp >= kDrainWarp0) {
    // ===================== dQ drain + per-row vectors =====================
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // query row inside the tile == TMEM lane
    const uint32_t tDQ0 = tbase + (static_cast<uint32_t>(quarter * 32) << 16) + kColDQ;
    bool ok = true;
    for (int it = 0; it < (kNoDQ ? 0 : n_tiles); ++it) {
      if (warp == kDrainWarp0) stamp(1, 0, it);
      const uint32_t tDQ = tDQ0 + (it % kDqBufs) * kNdq;
      ok = mbar_wait_warp(&bar_dq_full[it % kDqBufs], (it / kDqBufs) & 1, abortp, p.status, kBSiteDq, it);
      if (!ok) break;
      if (warp == kDrainWarp0) stamp(1, 1, it);
      tc_fence_after();
      const int i = (mb_lo + it) * kBwdBM + r;
      // The dQ tile goes TMEM -> registers -> swizzled shared memory -> one TMA add-reduction per
      // 32-column sub-tile into the fp32 workspace (the TMA unit issues the L2 reductions; rows past M
      // are clipped by the tensor map).  The accumulator is released as soon as it has been read.
      uint32_t rs[16];
      if (!kFp32Sums) tmem_ld16(tDQ + D, rs);  // rowsum(dS) sits in the column after the dQ columns
#pragma unroll
      for (int round = 0; round < D / (32 * kStageSub); ++round) {
        const int n_round = it * (D / (32 * kStageSub)) + round;
        if (n_round > 0) {
          ok = mbar_wait_warp(&bar_stage_free, (n_round - 1) & 1, abortp, p.status, kBSiteStageFree, it);
          if (!ok) break;
        }
#pragma unroll
        for (int sub = 0; sub < kStageSub; ++sub) {
          uint32_t v[32];
          tmem_ld32(tDQ + (round * kStageSub + sub) * 32, v);
          tmem_ld_wait();
          uint8_t* srow = sStage + sub * 16384 + r * 128;
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            *reinterpret_cast<uint4*>(srow + ((q4 ^ (r & 7)) << 4)) =
                make_uint4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
        }
        if (round == D / (32 * kStageSub) - 1) {
          tc_fence_before();
          mbar_arrive(&bar_dq_free[it % kDqBufs]);
        }
        fence_proxy_async_smem();
        mbar_arrive(&bar_staged);
        if (warp == kDrainWarp0) {
          ok = mbar_wait_warp(&bar_staged, n_round & 1, abortp, p.status, kBSiteStaged, it);
          if (!ok) break;
          if (elect_one()) {
#pragma unroll
            for (int sub = 0; sub < kStageSub; ++sub)
              tma_reduce_add_4d(&tmDQ, sStage + sub * 16384, (round * kStageSub + sub) * 32, (mb_lo + it) * kBwdBM,
                                h, b);
            tma_store_commit();
            tma_store_wait_read<0>();
            mbar_arrive(&bar_stage_free);
          }
          __syncwarp();
        }
      }
      if (!ok) break;
      if (warp == kDrainWarp0) stamp(1, 2, it);
      if (!kFp32Sums && i < M) atomicAdd(p.dlam_row + bh * M + i, __uint_as_float(rs[0]));
    }
    if (warp == kDrainWarp0) tma_store_wait_all<0>();
  } else {
    // ===================== compute warps =====================
    // A warp reads its 32 KV rows x 32 query columns of S^T / dP^T as matrix fragments (two 16-lane loads):
    // a thread holds four KV rows (r0 + 8 m) x eight query columns (pairs 8 k + q2, + 1).  Row sums of dS over the
    // KV index then need three shuffle steps over 8 values instead of five over 32, the column sums stay in
    // registers for the whole launch, and the per-query vectors are read as four 8-byte pairs.
    static_assert(CW == 32, "the fragment mapping below is written for four compute warpgroups");
    const int g = warp >> 2;               // which 32-column slice of the query tile
    const int quarter = warp & 3;          // which 32 KV rows (TMEM lanes) of the tile
    const int q2 = (lane & 3) * 2;         // this thread's column pair inside every 8-column group
    const int r0 = quarter * 32 + (lane >> 2);
    const int r = tid & 127;               // epilogue: KV row inside the tile == TMEM lane
    const int j = nb * kBwdBN + r;
    const bool j_ok = (j < N) && (j >= seq0);
    const float* lam = p.lam + bh * N;
    // Lambda_i - Lambda_j is formed from prefixes relative to the tile's first key: scaling a prefix of -1e4
    // by log2(e) first would cost an absolute 2e-3 per logit.  An invalid KV row gets b_j = +inf, i.e.
    // probability 0 everywhere.
    const float lam_ref = lam[min(nb * kBwdBN, N - 1)];
    float2 negb2[4];
    int jp[4];                             // KV index minus the causal offset, relative to this thread's first column
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int jm = nb * kBwdBN + r0 + 8 * m;
      const bool okm = (jm < N) && (jm >= seq0);
      const float nb_j = okm ? -(lam[min(jm, N - 1)] - lam_ref) * kLog2eB : -INFINITY;
      negb2[m] = make_float2(nb_j, nb_j);
      jp[m] = jm - P - g * 32 - q2;
    }
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tbase + lane_base + kColS + g * 32, tDP = tbase + lane_base + kColDP + g * 32;
    // stmatrix: this thread addresses row (lane & 7) of the 8x8 block of column group (lane >> 3)
    const uint32_t ds_addr0 = smem_u32(sdS) + ((g * 32) >> 6) * 16384 + (quarter * 32 + (lane & 7)) * 128 +
                              ((((((g * 32) & 63) >> 3) + (lane >> 3)) ^ (lane & 7)) << 4);
    float2 colacc[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) colacc[m] = make_float2(0.f, 0.f);
    bool ok = true;
    const float2 scale2 = make_float2(p.qk_scale, p.qk_scale);

    auto tile = [&](auto diag_tag, auto poly_tag, int it) -> bool {
      constexpr bool kDiag = decltype(diag_tag)::value;
      constexpr bool kPoly = decltype(poly_tag)::value;
      const int mb = mb_lo + it;
      const int st = it % STQ;
      if (warp < 8) stamp(6 + warp, 4, it);
      bool good = mbar_wait(&bar_s_full, it & 1, abortp, p.status, kBSiteSFull, it);
      if (warp < 8) stamp(6 + warp, 6, it);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      tc_fence_after();
      if (warp < 8) stamp(6 + warp, 0, it);
      float2 pf[2][4][2];   // [16-lane half][column group][row + 8]
      const uint32_t ds_addr = ds_addr0 + (it % kDsBufs) * 32768;
      float2 rs[4];         // sums over this thread's four KV rows, per query-column pair
      float2 ev[4], nd[4];  // e_i and -delta_i of this thread's four column pairs
      {
        const float2* e2 = reinterpret_cast<const float2*>(&s_e[st][g * 32 + q2]);
        const float2* d2 = reinterpret_cast<const float2*>(&s_delta[st][g * 32 + q2]);
#pragma unroll
        for (int k = 0; k < 4; ++k) { ev[k] = e2[4 * k]; nd[k] = d2[4 * k]; }
      }
      // phase A, one column group of one 16-lane half: probabilities (fp32 kept in pf, 16-bit pairs into pk)
      auto a_k = [&](int half, int k, const uint32_t* sreg, uint32_t* pk) {
#pragma unroll
        for (int h8 = 0; h8 < 2; ++h8) {
          const int m = half * 2 + h8;
          // packed two-wide fp32 arithmetic: x = s c + (e_i - b_j)
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * k + 2 * h8]),
                                                  __uint_as_float(sreg[4 * k + 2 * h8 + 1])),
                                      scale2, __fadd2_rn(ev[k], negb2[m]));
          float2 pe;
          if (kPoly && (((half * 8 + 2 * k + h8) * FOX_BWD_POLY) % 16) < FOX_BWD_POLY) pe = poly_exp2_x2(x);
          else pe = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          if constexpr (kDiag) {
            // query column (8 k + e past this thread's first) below the first one this KV row is attended from
            const int c_min = jp[m] - mb * kBwdBM;
            pe.x = (8 * k >= c_min) ? pe.x : 0.f;
            pe.y = (8 * k + 1 >= c_min) ? pe.y : 0.f;
          }
          pf[half][k][h8] = pe;
          pk[2 * k + h8] = pack2<kBf16>(pe.x, pe.y);
        }
      };
      // phase B, the same unit: dS (16-bit pairs into dsk) and the two sums
      auto b_k = [&](int half, int k, const uint32_t* dpreg, uint32_t* dsk) {
#pragma unroll
        for (int h8 = 0; h8 < 2; ++h8) {
          const int m = half * 2 + h8;
          const float2 ds = __fmul2_rn(pf[half][k][h8],
                                       __fadd2_rn(make_float2(__uint_as_float(dpreg[4 * k + 2 * h8]),
                                                              __uint_as_float(dpreg[4 * k + 2 * h8 + 1])),
                                                  nd[k]));
          const uint32_t d16 = pack2<kBf16>(ds.x, ds.y);
          dsk[2 * k + h8] = d16;
          if constexpr (kNoDQ || kFp32Sums) {
            // fp32 values on both sides (with kNoDQ the row sums come from another kernel's recomputed dS, which
            // agrees to fp32 rounding; the two kernels' 16-bit roundings differ on a few percent of the elements)
            colacc[m] = __fadd2_rn(colacc[m], ds);
            if constexpr (kFp32Sums && !kNoDQ) rs[k] = (m == 0) ? ds : __fadd2_rn(rs[k], ds);
          } else if (!kColsumMMA) {
            colacc[m] = __fadd2_rn(colacc[m], unpack2<kBf16>(d16));
          }
        }
      };
      auto store_ds = [&](int half, const uint32_t* dsk) {
        tmem_st_16x128b_x4(tDP + (static_cast<uint32_t>(half * 16) << 16), dsk);
        if constexpr (!kNoDQ) {   // (dS in shared memory only feeds the dQ product)
#pragma unroll
          for (int h8 = 0; h8 < 2; ++h8)
            stmatrix_x4(ds_addr + (half * 2 + h8) * 1024, dsk[h8], dsk[2 + h8], dsk[4 + h8], dsk[6 + h8]);
        }
      };
      uint32_t sregs[2][16], dpregs[2][16], pk[8], dsk[8];
      // ---------------- phase A: probabilities ----------------
      tmem_ld_16x256b_x4(tS, sregs[0]);
      tmem_ld_wait();
      tmem_ld_16x256b_x4(tS + (16u << 16), sregs[1]);   // in flight under the first half's arithmetic
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half == 1) tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 4; ++k) a_k(half, k, sregs[half], pk);
        // inside this warpgroup's own (already loaded) S columns
        tmem_st_16x128b_x4(tS + (static_cast<uint32_t>(half * 16) << 16), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_p_done);
      if (warp < 8) stamp(6 + warp, 1, it);

      // ---------------- phase B: dS ----------------
      if (warp < 8) stamp(6 + warp, 7, it);
      good = mbar_wait(&bar_dp_full, it & 1, abortp, p.status, kBSiteDpFull, it);
      // dP(it) was issued behind dQ(it - kDsBufs) and a commit covers everything issued before it, so the
      // dS buffer about to be overwritten is no longer being read.
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      tc_fence_after();
      if (warp < 8) stamp(6 + warp, 2, it);
      tmem_ld_16x256b_x4(tDP, dpregs[0]);
      tmem_ld_wait();
      tmem_ld_16x256b_x4(tDP + (16u << 16), dpregs[1]);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half == 1) tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 4; ++k) b_k(half, k, dpregs[half], dsk);
        store_ds(half, dsk);
      }
      tmem_st_wait();
      if (!kNoDQ) fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_ds_done);
      if (warp < 8) stamp(6 + warp, 3, it);
      if constexpr (kFp32Sums && !kNoDQ) {
        // rowsum(dS) over this warp's 32 KV rows, under the products that now read dS: the eight threads that
        // share a column pair differ in lane bits 2..4; at the step with lane distance `off` a thread keeps the
        // half of its values whose index has that bit as its own lane number does and receives the partner's
        // sums of them, so it ends with the sum of one column
        float v[8] = {rs[0].x, rs[0].y, rs[1].x, rs[1].y, rs[2].x, rs[2].y, rs[3].x, rs[3].y};
#pragma unroll
        for (int step = 0; step < 3; ++step) {
          const int off = 16 >> step, n = 4 >> step;
          const bool upper = (lane & off) != 0;
#pragma unroll
          for (int c = 0; c < n; ++c) {
            const float send = upper ? v[c] : v[c + n];
            const float keep = upper ? v[c + n] : v[c];
            v[c] = keep + __shfl_xor_sync(0xffffffffu, send, off);
          }
        }
        const int c8 = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
        const int i = mb * kBwdBM + g * 32 + 8 * (c8 >> 1) + q2 + (c8 & 1);
        if (i < M) atomicAdd(p.dlam_row + bh * M + i, v[0]);
      }
      if (warp < 8) stamp(6 + warp, 5, it);
      return true;
    };

    // the polynomial bottoms out at 2^-125 instead of 0: only where every KV row of the tile is a valid one
    const bool poly_ok = (nb * kBwdBN >= seq0) && (nb * kBwdBN + kBwdBN <= N);
    for (int it = 0; it < n_tiles; ++it) {
      // (only the tiles on the diagonal mask by position)
      const bool diag = (nb * kBwdBN + kBwdBN - 1 - P - (mb_lo + it) * kBwdBM) > 0;
      ok = diag ? tile(std::true_type{}, std::false_type{}, it)
                : (poly_ok ? tile(std::false_type{}, std::integral_constant<bool, (FOX_BWD_POLY > 0)>{}, it)
                           : tile(std::false_type{}, std::false_type{}, it));
      if (!ok) break;
    }

    // ---- epilogue: warpgroup 0 writes dK (and the key-side gate gradient), warpgroup 1 writes dV ----
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_done, 0, abortp, p.status, kBSiteDone);
      ok = __all_sync(0xffffffffu, ok);
    }
    float colsum = 0.f;
    if (!kColsumMMA && ok) {
      // per-thread partial column sums -> the four threads of a row -> one array per query-column slice (the
      // per-row vector buffers are dead by now) -> warpgroup 0, whose thread r owns KV row r from here on
      float* part = g < 2 ? &s_e[g][0] : &s_delta[g - 2][0];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        float c = colacc[m].x + colacc[m].y;
        c += __shfl_xor_sync(0xffffffffu, c, 1);
        c += __shfl_xor_sync(0xffffffffu, c, 2);
        if ((lane & 3) == m) part[r0 + 8 * m] = c;
      }
      mbar_arrive(&bar_colsum);
      if (g == 0) {
        ok = mbar_wait(&bar_colsum, 0, abortp, p.status, kBSiteColsum);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) colsum = (s_e[0][r] + s_e[1][r]) + (s_delta[0][r] + s_delta[1][r]);
      }
    }
    if (ok) {
      // warpgroups [0, kCWG/2) hold dK, the rest dV, each a D / (kCWG/2) wide column slice.  With pruning on, a
      // CTA lives for a few tiles and this epilogue weighs: the 16-bit tiles then go through shared memory (the
      // two Q stages are idle: every product has retired) and leave as TMA stores, which write whole lines and
      // clip the rows past N (a thread storing its own row 16 bytes at a time keeps the CTA ~7 us here).
      // Without pruning the direct stores measured 2 % faster for the whole kernel and are kept.
      tc_fence_after();
      constexpr int kPer = kCWG / 2;
      constexpr int kCols = D / kPer;
      const int which = g / kPer, part_c = (g % kPer) * kCols;
      const bool keep = j_ok && n_tiles > 0;
      const bool via_tma = p.end_index != nullptr;
      const uint32_t tcol = tbase + lane_base + (which == 0 ? kColDK : kColDV) + part_c;
      const float sc = which == 0 ? p.sm_scale : 1.f;
      uint16_t* orow = (which == 0
          ? reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_sb + h * p.dk_sh + static_cast<int64_t>(j) * p.dk_st
          : reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_sb + h * p.dv_sh + static_cast<int64_t>(j) * p.dv_st) + part_c;
      uint8_t* stile = sQ + which * kTileBytes;
#pragma unroll
      for (int c = 0; c < kCols; c += 32) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld32(tcol + c, v);
          tmem_ld_wait();
        }
        const int col = part_c + c;
        uint8_t* srow = stile + (col >> 6) * 16384 + r * 128;
#pragma unroll
        for (int q8 = 0; q8 < 32; q8 += 8) {
          uint4 w = make_uint4(0, 0, 0, 0);
          if (keep) {
            w.x = pack2<kBf16>(__uint_as_float(v[q8 + 0]) * sc, __uint_as_float(v[q8 + 1]) * sc);
            w.y = pack2<kBf16>(__uint_as_float(v[q8 + 2]) * sc, __uint_as_float(v[q8 + 3]) * sc);
            w.z = pack2<kBf16>(__uint_as_float(v[q8 + 4]) * sc, __uint_as_float(v[q8 + 5]) * sc);
            w.w = pack2<kBf16>(__uint_as_float(v[q8 + 6]) * sc, __uint_as_float(v[q8 + 7]) * sc);
          }
          if (via_tma) *reinterpret_cast<uint4*>(srow + (((((col & 63) + q8) >> 3) ^ (r & 7)) << 4)) = w;
          else if (j < N) *reinterpret_cast<uint4*>(orow + c + q8) = w;
        }
      }
      if (via_tma) {
        fence_proxy_async_smem();
        mbar_arrive(&bar_epi[which]);
      }
      if (via_tma && g % kPer == 0 && (warp & 3) == 0) {
        // (a bounded wait like every other one: a warp that gave up elsewhere never arrives)
        if (mbar_wait_warp(&bar_epi[which], 0, abortp, p.status, kBSiteEpi) && elect_one()) {
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub)
            tma_store_4d(which == 0 ? &tmDK : &tmDV, stile + sub * 16384, sub * 64, nb * kBwdBN, h, b);
          tma_store_commit();
          tma_store_wait_read<0>();   // the tile must stay in shared memory until it has been read
        }
        __syncwarp();
      }
      if (g == 0) {
        if (kColsumMMA && n_tiles > 0) {
          uint32_t cs[16];
          tmem_ld16(tbase + lane_base + kColDK + D, cs);
          tmem_ld_wait();
          colsum = __uint_as_float(cs[0]);
        }
        if (j < N) p.dlam_col[bh * N + j] = keep ? -colsum : 0.f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tbase, kTmemCols);
}

#ifdef FOX_DEBUG
// Debug builds (-DFOX_DEBUG) only: when set, the next backward launches record clock64 stamps of CTA (0,0,0).
static long long* g_bwd_trace = nullptr;
#endif

template <int D, bool kBf16>
static int launch_bwd(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N,
                      const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o,
                      const BwdParams& prm) {
  CUtensorMap tmQ, tmK, tmV, tmDO;
  Tensor4 tq{q->ptr, B, H, M, D, q->sb, q->sh, q->st};
  Tensor4 tk{k->ptr, B, H, N, D, k->sb, k->sh, k->st};
  Tensor4 tv{v->ptr, B, H, N, D, v->sb, v->sh, v->st};
  Tensor4 tdo{d_o->ptr, B, H, M, D, d_o->sb, d_o->sh, d_o->st};
  if (!tma_compatible(tq, 2) || !tma_compatible(tk, 2) || !tma_compatible(tv, 2) || !tma_compatible(tdo, 2))
    return FOX_ERR_ALIGNMENT;
  int rc;
  if ((rc = cached_tmap_4d(&tmQ, tq, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmK, tk, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmV, tv, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmDO, tdo, 2, false, kBf16, 64, 128, true))) return rc;
  CUtensorMap tmDK, tmDV;
  Tensor4 tdk{prm.dk, B, H, N, D, prm.dk_sb, prm.dk_sh, prm.dk_st};
  Tensor4 tdv{prm.dv, B, H, N, D, prm.dv_sb, prm.dv_sh, prm.dv_st};
  if (!tma_compatible(tdk, 2) || !tma_compatible(tdv, 2)) return FOX_ERR_ALIGNMENT;
  if ((rc = cached_tmap_4d(&tmDK, tdk, 2, false, kBf16, 64, 128, true))) return rc;
  if ((rc = cached_tmap_4d(&tmDV, tdv, 2, false, kBf16, 64, 128, true))) return rc;
  CUtensorMap tmDQ;
  Tensor4 tdq{prm.dq_accum, B, H, M, D, H * M * D, M * D, D};
  if (prm.dq_accum == nullptr) tmDQ = tmQ;  // unused by the kernel without a dQ product
  else if ((rc = cached_tmap_4d(&tmDQ, tdq, 4, true, false, 32, 128, true))) return rc;
  constexpr int kStQ = 2, kStDO = (D == 64) ? 2 : 1, kDsBufs = (D == 64) ? 2 : 1;
  constexpr int kStageSub = (D == 64) ? 2 : 1;
  constexpr int smem = (2 + kStQ + kStDO) * 128 * D * 2 + kDsBufs * 32768 + 16384 + kStageSub * 16384;
  static_assert(smem + 3072 <= 232448, "shared memory budget (tiles + static barriers/vectors rounded to 1 KiB)");
  constexpr int kCWG = 4;  // compute warpgroups per CTA (2 was measured no faster at D=64 and slower at D=128)
#ifdef FOX_DEBUG
  // debug builds also carry the traced instances and the form without a dQ product (the key side before
  // fox_attn_bwd_kv_kernel replaced it)
  const bool tracing = prm.trace != nullptr;
  const bool nodq = prm.dq_accum == nullptr;
  auto kern = tracing ? (nodq ? fox_attn_bwd_kernel<D, kBf16, true, kCWG, true> : fox_attn_bwd_kernel<D, kBf16, true, kCWG, false>)
                      : (nodq ? fox_attn_bwd_kernel<D, kBf16, false, kCWG, true> : fox_attn_bwd_kernel<D, kBf16, false, kCWG, false>);
#else
  constexpr bool tracing = false, nodq = false;
  if (prm.dq_accum == nullptr) return FOX_ERR_BAD_ARG;   // key-side-only calls go to fox_attn_bwd_kv_kernel
  auto kern = fox_attn_bwd_kernel<D, kBf16, false, kCWG, false>;
#endif
  const int threads = (4 * kCWG + 6) * 32;
  static bool configured[4][64] = {};
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  const int slot = tracing ? (nodq ? 3 : 1) : (nodq ? 2 : 0);
  if (!configured[slot][device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[slot][device] = true;
  }
  dim3 grid((unsigned)((N + kBwdBN - 1) / kBwdBN), (unsigned)H, (unsigned)B);
  kern<<<grid, threads, smem, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, tmDK, tmDV, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

}  // namespace fox

namespace fox {
// fox_attn_bwd_kv.cu: the key side with P^T and dS^T both written in phase B
int launch_bwd_kv(int device, cudaStream_t stream, bool bf16, int D, int64_t B, int64_t H, int64_t M, int64_t N,
                       const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o,
                       const float* log_lambda, const float* L, const float* delta, const int64_t* seq_start,
                       const int64_t* end_index, float sm_scale, float* dlam_col, const fox_tensor4* dk,
                       const fox_tensor4* dv, int32_t* status);
#ifdef FOX_DEBUG
static int g_kv_variant = 1;   // 0: the general kernel without its dQ product; 1: the key-side kernel
#endif
}  // namespace fox

#ifdef FOX_DEBUG
// Debug builds only: which kernel serves a key-side-only call (dq_accum_zeroed == NULL), and the trace buffer.
extern "C" void fox_debug_set_kv_variant(int v) { fox::g_kv_variant = v; }
extern "C" void fox_debug_set_bwd_trace(void* device_buffer) { fox::g_bwd_trace = static_cast<long long*>(device_buffer); }
#endif

extern "C" int fox_attn_bwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                            int64_t D, const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                            const fox_tensor4* d_o, const float* log_lambda, const float* L, const float* delta,
                            const int64_t* seq_start, const int64_t* end_index, float sm_scale,
                            float* dq_accum_zeroed, float* dlam_row_zeroed, float* dlam_col, const fox_tensor4* dk,
                            const fox_tensor4* dv, int32_t* status) {
  using namespace fox;
  if (!q || !k || !v || !d_o || !dk || !dv || !q->ptr || !k->ptr || !v->ptr || !d_o->ptr || !dk->ptr || !dv->ptr ||
      !log_lambda || !L || !delta || ((dq_accum_zeroed == nullptr) != (dlam_row_zeroed == nullptr)) || !dlam_col || !status)
    return FOX_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || M <= 0 || N <= 0 || M > N || H > 65535 || B > 65535) return FOX_ERR_BAD_ARG;
  if (N > 2147483647LL) return FOX_ERR_TOO_LARGE;   // row indices are 32-bit inside the kernels (M <= N)
  if (D != 64 && D != 128) return FOX_ERR_HEAD_DIM;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  const fox_tensor4* outs[2] = {dk, dv};
  for (int i = 0; i < 2; ++i)
    if (reinterpret_cast<uintptr_t>(outs[i]->ptr) % 16 || (outs[i]->sb * 2) % 16 || (outs[i]->sh * 2) % 16 ||
        (outs[i]->st * 2) % 16)
      return FOX_ERR_ALIGNMENT;
  if (reinterpret_cast<uintptr_t>(dq_accum_zeroed) % 16) return FOX_ERR_ALIGNMENT;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  BwdParams prm;
  prm.lam = log_lambda; prm.L = L; prm.delta = delta;
  prm.seq_start = seq_start; prm.end_index = end_index;
  prm.dq_accum = dq_accum_zeroed; prm.dlam_row = dlam_row_zeroed; prm.dlam_col = dlam_col;
  prm.dk = dk->ptr; prm.dk_sb = dk->sb; prm.dk_sh = dk->sh; prm.dk_st = dk->st;
  prm.dv = dv->ptr; prm.dv_sb = dv->sb; prm.dv_sh = dv->sh; prm.dv_st = dv->st;
  prm.status = status;
#ifdef FOX_DEBUG
  prm.trace = g_bwd_trace;
#else
  prm.trace = nullptr;
#endif
  prm.H = (int)H; prm.M = (int)M; prm.N = (int)N;
  prm.sm_scale = sm_scale;
  prm.qk_scale = sm_scale * 1.4426950408889634f;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = dtype == FOX_DTYPE_BF16;
#ifdef FOX_DEBUG
  const bool key_side_kernel = dq_accum_zeroed == nullptr && g_kv_variant == 1 && g_bwd_trace == nullptr;
#else
  const bool key_side_kernel = dq_accum_zeroed == nullptr;
#endif
  if (key_side_kernel)
    return launch_bwd_kv(device, st, bf, (int)D, B, H, M, N, q, k, v, d_o, log_lambda, L, delta, seq_start, end_index,
                         sm_scale, dlam_col, dk, dv, status);
  if (D == 64)
    return bf ? launch_bwd<64, true>(device, st, B, H, M, N, q, k, v, d_o, prm)
              : launch_bwd<64, false>(device, st, B, H, M, N, q, k, v, d_o, prm);
  return bf ? launch_bwd<128, true>(device, st, B, H, M, N, q, k, v, d_o, prm)
            : launch_bwd<128, false>(device, st, B, H, M, N, q, k, v, d_o, prm);
}
