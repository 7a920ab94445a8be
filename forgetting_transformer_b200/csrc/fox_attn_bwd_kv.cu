// Forgetting Attention backward, key side: dK, dV and the key-side log-gate gradient.
//
// Stands in for upstream's Triton `_bwd_kv_kernel`
// (src/forgetting_transformer/ops/forgetting_attention.py:956-1147).  Used together with the query-side kernel
// (fox_attn_bwd_dq.cu); the general kernel of fox_attn_bwd.cu without its dQ product does the same job.  There
// the 16-bit P^T is written over S^T, so S^T(i+1) has to wait for dV(i), which waits for the whole of phase A(i):
// phase A(i) -> dV(i) -> S^T(i+1) -> phase A(i+1) is one serial chain per tile.  Here both 16-bit operands, P^T and
// dS^T, are written in phase B into the dP^T columns a warpgroup has itself just read (32 fp32 columns hold its
// 16 + 16 packed ones), so S^T(i+1) is issued as soon as S^T(i) has been read and runs under phase B(i) and the
// dV / dK products.
//
// One CTA = one (batch, head, 128-row KV tile), one CTA per SM; K and V resident in shared memory:
//   warps 0-15 : four elementwise warpgroups, thread = KV row (TMEM lane) x 32 of the tile's 128 query columns
//                phase A: p^T = 2^(s^T c + e_i - b_j), kept in registers; S^T is free once it has been read
//                phase B: dS^T = p^T (dP^T - delta_i); P^T and dS^T -> 16 bit over its own dP^T columns;
//                         colsum(dS) in fp32
//   warp 16    : TMA producer (K, V once; Q, dO tiles in rings of two; stages e_i = (Lambda_i - L_i) log2e, delta_i)
//   warp 17    : tcgen05.mma issuer:
//                wait S read(i): S^T(i+1) = K Q(i+1)^T | wait dS(i): dV += P^T(i) dO(i), dK += dS^T(i) Q(i),
//                dP^T(i+1) = V dO(i+1)^T
// TMEM (512 columns): S^T [0,128), dP^T [128,256), dK [256,384), dV [384,512).
// Query tiles are walked upwards from the diagonal to end_index (lines 1003-1049).
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int kKvBN = 128, kKvBM = 128;
constexpr float kKvLog2e = 1.4426950408889634f;

struct KvParams {
  const float* lam;          // (B,H,N)
  const float* L;            // (B,H,M)
  const float* delta;        // (B,H,M)
  const int64_t* seq_start;  // (B,) or nullptr
  const int64_t* end_index;  // (B,H,ceil(N/128)) or nullptr
  float* dlam_col;           // (B,H,N), fully written
  void* dk; int64_t dk_sb, dk_sh, dk_st;
  void* dv; int64_t dv_sb, dv_sh, dv_st;
  int* status;
  int H, M, N;
  float sm_scale, qk_scale;
};

#ifdef FOX_KV_TRACE
__device__ long long g_kv_trace[24 * 8 * 16];
#define KVSTAMP(role, ev, it) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (it) >= 32 && (it) < 48) g_kv_trace[((role) * 8 + (ev)) * 16 + (it) - 32] = clock64(); } while (0)
extern "C" int fox_debug_read_kv_trace(long long* host) { return cudaMemcpyFromSymbol(host, g_kv_trace, sizeof(g_kv_trace)); }
// CTA timeline: nanosecond stamps of up to 8192 CTAs (entry, after set-up, first S^T, last tile, products done,
// stores done, exit) and the SM they ran on
__device__ unsigned long long g_kv_cta[8192 * 8];
__device__ __forceinline__ unsigned long long kv_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define KVCTA(ev) do { const unsigned cta_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); if (cta_ < 8192) g_kv_cta[cta_ * 8 + (ev)] = kv_now_ns(); } while (0)
extern "C" int fox_debug_read_kv_cta(unsigned long long* host) { return cudaMemcpyFromSymbol(host, g_kv_cta, sizeof(g_kv_cta)); }
#else
#define KVSTAMP(role, ev, it)
#define KVCTA(ev)
#endif

enum KvWaitSite { kKvSiteQ = 71, kKvSiteDO = 72, kKvSiteQE = 73, kKvSiteDOE = 74, kKvSiteS = 75, kKvSiteDP = 76,
                  kKvSiteP = 77, kKvSiteDS = 78, kKvSiteDone = 79, kKvSiteVec = 80, kKvSiteCol = 81, kKvSiteKV = 82, kKvSiteEpi = 83 };

template <int D, bool kBf16>
__global__ void __launch_bounds__(576, 1)
fox_attn_bwd_kv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                       const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV, const KvParams p) {
  static_assert(D == 64 || D == 128, "head dim");
  constexpr int BM = kKvBM;                      // query rows per tile
  constexpr int kWG = 4, CW = BM / kWG;          // 32 query columns of every tile per warpgroup
  constexpr int kSt = 2;                         // Q and dO stages
  constexpr int kVec = 4;                        // ring of per-row vectors
  constexpr int kTileBytes = BM * D * 2;         // 32 KB
  constexpr int kSubBytes = BM * 128;            // one [128 rows][64 x 16 bit] sub-tile
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 384;
  constexpr uint32_t kTmemCols = 512;
  constexpr int kTmaWarp = 4 * kWG, kMmaWarp = 4 * kWG + 1;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full[kSt], bar_q_empty[kSt], bar_do_full[kSt], bar_do_empty[kSt], bar_vec[kVec], bar_s_full,
      bar_dp_full, bar_s_read, bar_ds_full, bar_done, bar_kv, bar_colsum, bar_epi[2];
  __shared__ __align__(16) float s_e[kVec][BM];
  __shared__ __align__(16) float s_delta[kVec][BM];
  __shared__ float s_part[kWG - 1][128];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* sQ = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sDO = sQ + kSt * kTileBytes;
  uint8_t* sK = sDO + kSt * kTileBytes;
  uint8_t* sV = sK + kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    KVCTA(0);
#ifdef FOX_KV_TRACE
    unsigned smid_;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid_));
    { const unsigned cta_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); if (cta_ < 8192) g_kv_cta[cta_ * 8 + 7] = smid_; }
#endif
  }
  const int nb = static_cast<int>(blockIdx.x);   // (KV tile 0 sees every query row: heavy tiles first)
  const int h = blockIdx.y, b = blockIdx.z;
  const int M = p.M, N = p.N, P = N - M;
  const int64_t bh = static_cast<int64_t>(b) * p.H + h;
  const int seq0 = p.seq_start ? static_cast<int>(p.seq_start[b]) : 0;
  const int j0 = nb * kKvBN;

  // ---- query-tile range of this KV tile (upstream lines 1003-1049) ----
  int lo = max(j0 - P, 0);
  lo = (lo / BM) * BM;
  int hi = M;
  if (p.end_index) {
    const int64_t e = p.end_index[bh * gridDim.x + nb];
    hi = static_cast<int>(e < static_cast<int64_t>(M) ? e : static_cast<int64_t>(M));
  }
  if (p.seq_start && !(j0 + kKvBN >= seq0 - 1)) hi = lo;
  const int hb_lo = lo / BM;
  const int hb_hi = (hi + BM - 1) / BM;
  const int n_tiles = max(hb_hi - hb_lo, 0);

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < kSt; ++i) {
      mbar_init(&bar_q_full[i], 1);
      mbar_init(&bar_q_empty[i], 1);
      mbar_init(&bar_do_full[i], 1);
      mbar_init(&bar_do_empty[i], 1);
    }
    for (int i = 0; i < kVec; ++i) mbar_init(&bar_vec[i], 1);
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_dp_full, 1);
    mbar_init(&bar_s_read, 128 * kWG);
    mbar_init(&bar_ds_full, 128 * kWG);
    mbar_init(&bar_done, 1);
    mbar_init(&bar_kv, 1);
    mbar_init(&bar_colsum, 128 * (kWG - 1));
    mbar_init(&bar_epi[0], 256);
    mbar_init(&bar_epi[1], 256);
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
  if (tid == 0) KVCTA(1);

  if (warp == kTmaWarp) {
    // ===================== TMA producer =====================
    if (n_tiles > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_expect_tx(&bar_kv, 2 * kTileBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
          tma_load_4d(sK + s * kSubBytes, &tmK, &bar_kv, s * 64, j0, h, b);
          tma_load_4d(sV + s * kSubBytes, &tmV, &bar_kv, s * 64, j0, h, b);
        }
      }
      __syncwarp();
      const float* lam = p.lam + bh * N + P;
      const float* Lp = p.L + bh * M;
      const float* dl = p.delta + bh * M;
      // prefixes relative to this KV tile's first key before the scaling by log2(e), as for negb below
      const float lam_ref = p.lam[bh * N + min(j0, N - 1)];
      float ev[4], dv_[4];   // lane l holds query rows 4l .. 4l+3 of a tile
      auto fetch_vec = [&](int it) {
        const int i0 = (hb_lo + it) * BM + 4 * lane;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + e;
          float Li = -INFINITY, la = 0.f, de = 0.f;
          if (i < M) {
            Li = ldg_f32_here(Lp + i);
            la = ldg_f32_here(lam + i);
            de = ldg_f32_here(dl + i);
          }
          ev[e] = (Li == -INFINITY) ? -INFINITY : ((la - lam_ref) - Li) * kKvLog2e;
          dv_[e] = de;
        }
      };
      auto stage_vec = [&](int it) {
        const int slot = it % kVec;
        *reinterpret_cast<float4*>(&s_e[slot][4 * lane]) = make_float4(ev[0], ev[1], ev[2], ev[3]);
        *reinterpret_cast<float4*>(&s_delta[slot][4 * lane]) = make_float4(dv_[0], dv_[1], dv_[2], dv_[3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_vec[slot]);
        __syncwarp();
      };
      fetch_vec(0);
      int issued = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int i0 = (hb_lo + it) * BM;
        const int st = it % kSt;
        const uint32_t ph = ((it / kSt) & 1) ^ 1;
        if (!mbar_wait_warp(&bar_q_empty[st], ph, abortp, p.status, kKvSiteQE, it)) break;
        if (elect_one()) {
          mbar_expect_tx(&bar_q_full[st], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s) tma_load_4d(sQ + st * kTileBytes + s * kSubBytes, &tmQ, &bar_q_full[st], s * 64, i0, h, b);
        }
        __syncwarp();
        if (!mbar_wait_warp(&bar_do_empty[st], ph, abortp, p.status, kKvSiteDOE, it)) {
          issued = 2 * it + 1;
          break;
        }
        if (elect_one()) {
          mbar_expect_tx(&bar_do_full[st], kTileBytes);
#pragma unroll
          for (int s = 0; s < kSub; ++s) tma_load_4d(sDO + st * kTileBytes + s * kSubBytes, &tmDO, &bar_do_full[st], s * 64, i0, h, b);
        }
        __syncwarp();
        issued = 2 * it + 2;
        // (slot it % 4 last held tile it-4; the Q stage just re-used was freed by dK(it-2), behind dS(it-2))
        stage_vec(it);
        if (it + 1 < n_tiles) fetch_vec(it + 1);
      }
      if (*abortp && lane == 0) {
        // error path only: let the copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_kv, 0) && clock64() - t0 < 200000000LL) {
        }
        for (int c = max(issued - 2 * kSt, 0); c < issued; ++c) {
          const int it = c >> 1;
          uint64_t* bar = (c & 1) ? &bar_do_full[it % kSt] : &bar_q_full[it % kSt];
          while (!mbar_try_wait(bar, (it / kSt) & 1) && clock64() - t0 < 200000000LL) {
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    if (n_tiles > 0) {
      constexpr uint32_t idS = umma_idesc(kFmt, 128, BM, 0, 0);    // S^T, dP^T: N = 128 query rows, B K-major
      constexpr uint32_t idKV = umma_idesc(kFmt, 128, D, 0, 1);    // dV, dK: N = D, B MN-major
      const uint64_t dKk = umma_desc_kmajor(smem_u32(sK));
      const uint64_t dVk = umma_desc_kmajor(smem_u32(sV));
      const uint64_t dQk = umma_desc_kmajor(smem_u32(sQ));
      const uint64_t dDOk = umma_desc_kmajor(smem_u32(sDO));
      const uint64_t dQmn = umma_desc_mnmajor(smem_u32(sQ), kSubBytes);
      const uint64_t dDOmn = umma_desc_mnmajor(smem_u32(sDO), kSubBytes);
      auto issue_s = [&](int t) {
        if (elect_one()) {
          const uint64_t dq_ = umma_desc_advance(dQk, (t % kSt) * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kSubBytes + (kk & 3) * 32;
            mma_ss_raw(tbase + kColS, umma_desc_advance(dKk, off), umma_desc_advance(dq_, off), idS, kk > 0);
          }
          tc_commit_raw(&bar_s_full);
        }
        __syncwarp();
      };
      auto issue_dp = [&](int t) {
        if (elect_one()) {
          const uint64_t do_ = umma_desc_advance(dDOk, (t % kSt) * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kSubBytes + (kk & 3) * 32;
            mma_ss_raw(tbase + kColDP, umma_desc_advance(dVk, off), umma_desc_advance(do_, off), idS, kk > 0);
          }
          tc_commit_raw(&bar_dp_full);
        }
        __syncwarp();
      };
      bool ok = mbar_wait_warp(&bar_kv, 0, abortp, p.status, kKvSiteKV);
      if (ok) ok = mbar_wait_warp(&bar_q_full[0], 0, abortp, p.status, kKvSiteQ, 0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = mbar_wait_warp(&bar_do_full[0], 0, abortp, p.status, kKvSiteDO, 0);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(0);
      }
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int st = it % kSt;
        KVSTAMP(17, 0, it);
        // S^T(it) has been read into registers: S^T(it+1) may overwrite it
        ok = mbar_wait_warp(&bar_s_read, it & 1, abortp, p.status, kKvSiteP, it);
        if (!ok) break;
        KVSTAMP(17, 1, it);
        if (it + 1 < n_tiles) {
          ok = mbar_wait_warp(&bar_q_full[(it + 1) % kSt], ((it + 1) / kSt) & 1, abortp, p.status, kKvSiteQ, it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        KVSTAMP(17, 2, it);
        ok = mbar_wait_warp(&bar_ds_full, it & 1, abortp, p.status, kKvSiteDS, it);
        if (!ok) break;
        KVSTAMP(17, 3, it);
        tc_fence_after();
        if (elect_one()) {
          // warpgroup g's 32 dP^T columns now hold its 16-bit P^T (first 16) and dS^T (last 16);
          // product step kk covers query columns [16 kk, 16 kk + 16): warpgroup kk / 2, half kk % 2
          const uint64_t do_ = umma_desc_advance(dDOmn, st * kTileBytes);
          const uint64_t dq_ = umma_desc_advance(dQmn, st * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk)
            mma_ts_raw(tbase + kColDV, tbase + kColDP + (kk >> 1) * CW + (kk & 1) * 8, umma_desc_advance(do_, kk * 2048), idKV,
                       (it > 0 || kk > 0) ? 1u : 0u);
          tc_commit_raw(&bar_do_empty[st]);
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk)
            mma_ts_raw(tbase + kColDK, tbase + kColDP + (kk >> 1) * CW + 16 + (kk & 1) * 8, umma_desc_advance(dq_, kk * 2048), idKV,
                       (it > 0 || kk > 0) ? 1u : 0u);
          tc_commit_raw(&bar_q_empty[st]);
        }
        __syncwarp();
        if (it + 1 < n_tiles) {
          ok = mbar_wait_warp(&bar_do_full[(it + 1) % kSt], ((it + 1) / kSt) & 1, abortp, p.status, kKvSiteDO, it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_dp(it + 1);   // overwrites P^T(it), dS^T(it): ordered behind dV(it), dK(it) in the tensor pipe
        }
        KVSTAMP(17, 4, it);
      }
      if (ok) tc_commit(&bar_done);
    }
  } else {
    // ===================== elementwise / epilogue =====================
    const int g = warp >> 2;
    const int r = tid & 127;
    const int j = j0 + r;
    const bool j_ok = j < N && j >= seq0;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // Lambda_i - Lambda_j from prefixes relative to the tile's first key: scaling a prefix of -1e4 by log2(e)
    // first would cost an absolute 2e-3 per logit
    const float negb = j_ok ? (p.lam[bh * N + min(j0, N - 1)] - p.lam[bh * N + j]) * kKvLog2e : -INFINITY;
    const uint32_t tS = tbase + lane_base + kColS + g * CW, tDP = tbase + lane_base + kColDP + g * CW;
    const float2 scale2 = make_float2(p.qk_scale, p.qk_scale);
    const float2 negb2 = make_float2(negb, negb);
    float2 colsum2 = make_float2(0.f, 0.f);
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int i0 = (hb_lo + it) * BM;
      const int slot = it % kVec;
      // ---------------- phase A: p^T into registers ----------------
      KVSTAMP(warp, 0, it);
      ok = mbar_wait(&bar_vec[slot], (it / kVec) & 1, abortp, p.status, kKvSiteVec, it);
      ok = mbar_wait(&bar_s_full, it & 1, abortp, p.status, kKvSiteS, it) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      KVSTAMP(warp, 1, it);
      if (tid == 0 && it == 0) KVCTA(2);
      tc_fence_after();
      uint32_t sreg[32], pk[16];
      float2 pf[16];
      tmem_ld32(tS, sreg);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bar_s_read);          // S^T(it) is in registers: the issuer may start S^T(it+1)
      // causal: query column c is seen by KV row j iff j <= P + i0 + c
      const bool need_mask = j0 + kKvBN - 1 > P + i0;
      const int c_lo = j - P - i0;
      const float4* e4 = reinterpret_cast<const float4*>(&s_e[slot][g * CW]);
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 ev = e4[c4];
        float2 x01 = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4]), __uint_as_float(sreg[4 * c4 + 1])), scale2,
                                __fadd2_rn(make_float2(ev.x, ev.y), negb2));
        float2 x23 = __ffma2_rn(make_float2(__uint_as_float(sreg[4 * c4 + 2]), __uint_as_float(sreg[4 * c4 + 3])), scale2,
                                __fadd2_rn(make_float2(ev.z, ev.w), negb2));
        if (need_mask) {
          const int cc = g * CW + 4 * c4;
          x01.x = (cc >= c_lo) ? x01.x : -INFINITY;
          x01.y = (cc + 1 >= c_lo) ? x01.y : -INFINITY;
          x23.x = (cc + 2 >= c_lo) ? x23.x : -INFINITY;
          x23.y = (cc + 3 >= c_lo) ? x23.y : -INFINITY;
        }
        pf[2 * c4] = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
        pf[2 * c4 + 1] = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
      }
      KVSTAMP(warp, 2, it);
      // ---------------- phase B: P^T and dS^T, 16 bit, over this warpgroup's own dP^T columns ----------------
      ok = mbar_wait(&bar_dp_full, it & 1, abortp, p.status, kKvSiteDP, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      KVSTAMP(warp, 3, it);
      tc_fence_after();
      tmem_ld32(tDP, sreg);
      tmem_ld_wait();
#pragma unroll
      for (int c2 = 0; c2 < 16; ++c2) pk[c2] = pack2<kBf16>(pf[c2].x, pf[c2].y);
      tmem_st16(tDP, pk);
      const float4* d4 = reinterpret_cast<const float4*>(&s_delta[slot][g * CW]);
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 dl = d4[c4];
        const float2 ds01 = __fmul2_rn(pf[2 * c4], make_float2(__uint_as_float(sreg[4 * c4]) - dl.x, __uint_as_float(sreg[4 * c4 + 1]) - dl.y));
        const float2 ds23 = __fmul2_rn(pf[2 * c4 + 1], make_float2(__uint_as_float(sreg[4 * c4 + 2]) - dl.z, __uint_as_float(sreg[4 * c4 + 3]) - dl.w));
        pk[2 * c4] = pack2<kBf16>(ds01.x, ds01.y);
        pk[2 * c4 + 1] = pack2<kBf16>(ds23.x, ds23.y);
        colsum2 = __fadd2_rn(colsum2, __fadd2_rn(ds01, ds23));   // fp32 values, as the query-side kernel's row sums
      }
      tmem_st16(tDP + 16, pk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_ds_full);
      KVSTAMP(warp, 4, it);
    }
    // ---- epilogue: dK * sm_scale, dV -> 16-bit -> global; -colsum(dS) ----
    if (tid == 0) KVCTA(3);
    float colsum = colsum2.x + colsum2.y;
    if (g > 0) {
      s_part[g - 1][r] = colsum;
      mbar_arrive(&bar_colsum);
    } else {
      ok = mbar_wait(&bar_colsum, 0, abortp, p.status, kKvSiteCol) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) colsum += (s_part[0][r] + s_part[1][r]) + s_part[2][r];
    }
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_done, 0, abortp, p.status, kKvSiteDone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (tid == 0) KVCTA(4);
    if (ok) {
      tc_fence_after();
      // warpgroups 0, 1 hold the halves of dK, 2 and 3 those of dV.  The 16-bit tiles go through shared memory
      // (the Q stages are idle: every product has retired) and leave as TMA stores, which write whole lines and
      // clip the rows past N; a thread storing its own row 16 bytes at a time kept the CTA ~7 us in this epilogue.
      constexpr int kHalf = D / 2;   // columns of dK or dV per warpgroup
      const int which = g >> 1, part_c = (g & 1) * kHalf;
      const bool keep = j_ok && n_tiles > 0;
      const uint32_t tcol = tbase + lane_base + (which == 0 ? kColDK : kColDV) + part_c;
      const float sc = which == 0 ? p.sm_scale : 1.f;
      uint8_t* stile = sQ + which * kTileBytes;
#pragma unroll
      for (int c = 0; c < kHalf; c += 32) {
        uint32_t t0[32];
        if (n_tiles > 0) {
          tmem_ld32(tcol + c, t0);
          tmem_ld_wait();
        }
        const int col = part_c + c;
        uint8_t* srow = stile + (col >> 6) * kSubBytes + r * 128;
#pragma unroll
        for (int q8 = 0; q8 < 32; q8 += 8) {
          uint4 w = make_uint4(0, 0, 0, 0);
          if (keep) {
            w.x = pack2<kBf16>(__uint_as_float(t0[q8 + 0]) * sc, __uint_as_float(t0[q8 + 1]) * sc);
            w.y = pack2<kBf16>(__uint_as_float(t0[q8 + 2]) * sc, __uint_as_float(t0[q8 + 3]) * sc);
            w.z = pack2<kBf16>(__uint_as_float(t0[q8 + 4]) * sc, __uint_as_float(t0[q8 + 5]) * sc);
            w.w = pack2<kBf16>(__uint_as_float(t0[q8 + 6]) * sc, __uint_as_float(t0[q8 + 7]) * sc);
          }
          *reinterpret_cast<uint4*>(srow + (((((col & 63) + q8) >> 3) ^ (r & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&bar_epi[which]);
      if ((g & 1) == 0 && (warp & 3) == 0) {
        // (a bounded wait like every other one: a warp that gave up elsewhere never arrives)
        if (mbar_wait_warp(&bar_epi[which], 0, abortp, p.status, kKvSiteEpi) && elect_one()) {
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub)
            tma_store_4d(which == 0 ? &tmDK : &tmDV, stile + sub * kSubBytes, sub * 64, j0, h, b);
          tma_store_commit();
          tma_store_wait_read<0>();   // the tile must stay in shared memory until it has been read
        }
        __syncwarp();
      }
      if (g == 0 && j < N) p.dlam_col[bh * N + j] = keep ? -colsum : 0.f;
    }
    if (tid == 0) KVCTA(5);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) tmem_dealloc(tbase, kTmemCols);
  if (tid == 0) KVCTA(6);
}

template <int D, bool kBf16>
static int launch_kv(int device, cudaStream_t stream, int64_t B, int64_t H, int64_t M, int64_t N, const fox_tensor4* q,
                     const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o, const KvParams& prm) {
  CUtensorMap tmQ, tmK, tmV, tmDO;
  Tensor4 tq{q->ptr, B, H, M, D, q->sb, q->sh, q->st};
  Tensor4 tk{k->ptr, B, H, N, D, k->sb, k->sh, k->st};
  Tensor4 tv{v->ptr, B, H, N, D, v->sb, v->sh, v->st};
  Tensor4 tdo{d_o->ptr, B, H, M, D, d_o->sb, d_o->sh, d_o->st};
  if (!tma_compatible(tq, 2) || !tma_compatible(tk, 2) || !tma_compatible(tv, 2) || !tma_compatible(tdo, 2))
    return FOX_ERR_ALIGNMENT;
  int rc;
  if ((rc = cached_tmap_4d(&tmQ, tq, 2, false, kBf16, 64, kKvBM, true))) return rc;
  if ((rc = cached_tmap_4d(&tmDO, tdo, 2, false, kBf16, 64, kKvBM, true))) return rc;
  if ((rc = cached_tmap_4d(&tmK, tk, 2, false, kBf16, 64, kKvBN, true))) return rc;
  if ((rc = cached_tmap_4d(&tmV, tv, 2, false, kBf16, 64, kKvBN, true))) return rc;
  CUtensorMap tmDK, tmDV;
  Tensor4 tdk{prm.dk, B, H, N, D, prm.dk_sb, prm.dk_sh, prm.dk_st};
  Tensor4 tdv{prm.dv, B, H, N, D, prm.dv_sb, prm.dv_sh, prm.dv_st};
  if (!tma_compatible(tdk, 2) || !tma_compatible(tdv, 2)) return FOX_ERR_ALIGNMENT;
  if ((rc = cached_tmap_4d(&tmDK, tdk, 2, false, kBf16, 64, kKvBN, true))) return rc;
  if ((rc = cached_tmap_4d(&tmDV, tdv, 2, false, kBf16, 64, kKvBN, true))) return rc;
  constexpr int smem = (2 * 2 + 2) * 128 * D * 2 + 1024;   // Q, dO in two stages each, K, V
  auto kern = fox_attn_bwd_kv_kernel<D, kBf16>;
  static bool configured[64] = {};
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[device] = true;
  }
  dim3 grid((unsigned)((N + kKvBN - 1) / kKvBN), (unsigned)H, (unsigned)B);
  kern<<<grid, 576, smem, stream>>>(tmQ, tmK, tmV, tmDO, tmDK, tmDV, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

// Key side (dk, dv, dlam_col); arguments as fox_attn_bwd's, already validated there.
int launch_bwd_kv(int device, cudaStream_t stream, bool bf16, int D, int64_t B, int64_t H, int64_t M, int64_t N,
                       const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v, const fox_tensor4* d_o,
                       const float* log_lambda, const float* L, const float* delta, const int64_t* seq_start,
                       const int64_t* end_index, float sm_scale, float* dlam_col, const fox_tensor4* dk,
                       const fox_tensor4* dv, int32_t* status) {
  KvParams prm;
  prm.lam = log_lambda; prm.L = L; prm.delta = delta; prm.seq_start = seq_start; prm.end_index = end_index;
  prm.dlam_col = dlam_col;
  prm.dk = dk->ptr; prm.dk_sb = dk->sb; prm.dk_sh = dk->sh; prm.dk_st = dk->st;
  prm.dv = dv->ptr; prm.dv_sb = dv->sb; prm.dv_sh = dv->sh; prm.dv_st = dv->st;
  prm.status = status;
  prm.H = (int)H; prm.M = (int)M; prm.N = (int)N;
  prm.sm_scale = sm_scale;
  prm.qk_scale = sm_scale * kKvLog2e;
  if (D == 64)
    return bf16 ? launch_kv<64, true>(device, stream, B, H, M, N, q, k, v, d_o, prm)
                : launch_kv<64, false>(device, stream, B, H, M, N, q, k, v, d_o, prm);
  return bf16 ? launch_kv<128, true>(device, stream, B, H, M, N, q, k, v, d_o, prm)
              : launch_kv<128, false>(device, stream, B, H, M, N, q, k, v, d_o, prm);
}

}  // namespace fox
