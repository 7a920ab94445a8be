// Forgetting Attention backward for sm_100a: one pass over the (query tile, KV
// tile) pairs with five tcgen05 matrix products per pair and a single exp2.
//
// Stands in for upstream's Triton `_bwd_kv_kernel` and `_bwd_q_kernel`
// (src/forgetting_transformer/ops/forgetting_attention.py:956-1143, 1156-1344),
// which recompute S and dP twice (seven products per pair).
//
// One CTA = one (batch, head, 128-row KV tile); it keeps K and V resident and
// streams the query tiles from the causal diagonal downwards.
//   warps 0-3 : thread t owns KV row t (TMEM lane t of S^T, dP^T, dK, dV) and,
//               when draining dQ, query row t of the current tile
//   warp 4    : TMA producer,  warp 5 : tcgen05.mma issuer
// Per pair:  S^T = K Q^T,  dP^T = V dO^T            (smem x smem -> TMEM)
//            P^T = 2^(S^T scale + bias - L)          (registers, written over S^T as 16-bit)
//            dS^T = P^T (dP^T - delta)               (registers -> swizzled smem, 16-bit)
//            dV += P^T dO   (TMEM x smem),  dK += dS^T Q   (smem x smem)
//            dQ_tile = dS K | dS 1                   (smem x smem, fresh accumulator)
// dQ tiles are added into an fp32 workspace with vector reductions; the extra 16
// "ones" columns appended to K make the same product deliver rowsum(dS), i.e. the
// query-side part of the log-gate gradient, built from exactly the rounded dS
// values whose column sums form the key-side part (so the two cancel the way
// they do upstream when the reverse prefix sum is taken).
#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int kBwdBM = FOX_BWD_BLOCK_M;
constexpr int kBwdBN = FOX_BWD_BLOCK_N;
constexpr int kBwdThreads = 192;
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
  int H, M, N;
  float sm_scale, qk_scale;
};

enum BwdWaitSite {
  kBSiteKV = 31, kBSiteQFull = 32, kBSiteQEmpty = 33, kBSiteSFull = 34, kBSitePds = 35, kBSiteDq = 36,
  kBSiteVec = 37, kBSiteDone = 38, kBSiteDrained = 39, kBSiteDrain = 40
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int D, bool kBf16, int STAGES>
__global__ void __launch_bounds__(kBwdThreads, 1)
fox_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const BwdParams p) {
  constexpr int kTileBytes = 128 * D * 2;
  constexpr int kSub = D / 64;
  constexpr uint32_t kFmt = kBf16 ? 1u : 0u;
  constexpr bool kAliasDQ = (D == 128);      // dQ accumulator shares columns with S^T / dP^T
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 256 + D;
  constexpr uint32_t kColDQ = kAliasDQ ? 0 : 256 + 2 * D;
  constexpr int kNdq = D + 16;               // dQ columns + rowsum columns

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_kv, bar_s_full, bar_pds, bar_dq, bar_done, bar_drained;
  __shared__ uint64_t bar_q_full[STAGES], bar_q_empty[STAGES], bar_vec[2];
  __shared__ float s_e[2][kBwdBM], s_delta[2][kBwdBM];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                         // kSub sub-tiles, then the "ones" sub-tile
  uint8_t* sOnes = sK + kTileBytes;
  uint8_t* sV = sOnes + 16384;
  uint8_t* sdS = sV + kTileBytes;             // [128 kv][128 q] as two 64-wide sub-tiles
  uint8_t* sQ = sdS + 32768;
  uint8_t* sDO = sQ + STAGES * kTileBytes;

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
    mbar_init(&bar_pds, 128);
    mbar_init(&bar_dq, 1);
    mbar_init(&bar_done, 1);
    mbar_init(&bar_drained, 128);
    mbar_init(&bar_vec[0], 128);
    mbar_init(&bar_vec[1], 128);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_q_full[s], 1);
      mbar_init(&bar_q_empty[s], 1);
    }
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp < 4) {
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

  if (warp == 4) {
    // ===================== TMA producer =====================
    if (lane == 0 && n_tiles > 0) {
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
      int issued = 0;
      for (int it = 0; it < n_tiles; ++it) {
        const int mb = mb_lo + it;
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&bar_q_empty[st], ph ^ 1, abortp, p.status, kBSiteQEmpty, it)) break;
        mbar_expect_tx(&bar_q_full[st], 2 * kTileBytes);
#pragma unroll
        for (int s = 0; s < kSub; ++s) {
          tma_load_4d(sQ + st * kTileBytes + s * 16384, &tmQ, &bar_q_full[st], s * 64, mb * kBwdBM, h, b);
          tma_load_4d(sDO + st * kTileBytes + s * 16384, &tmDO, &bar_q_full[st], s * 64, mb * kBwdBM, h, b);
        }
        issued = it + 1;
      }
      if (*abortp) {
        // error path only: let the copies already in flight land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bar_kv, 0) && clock64() - t0 < 200000000LL) {
        }
        for (int it = max(issued - STAGES, 0); it < issued; ++it) {
          const int st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          while (!mbar_try_wait(&bar_q_full[st], ph) && clock64() - t0 < 200000000LL) {
          }
        }
      }
    }
  } else if (warp == 5) {
    // ===================== MMA issuer =====================
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idS = umma_idesc(kFmt, 128, 128, 0, 0);
      constexpr uint32_t idKV = umma_idesc(kFmt, 128, D, 0, 1);
      constexpr uint32_t idDQ = umma_idesc(kFmt, 128, kNdq, 1, 1);
      const uint32_t k0 = smem_u32(sK), v0 = smem_u32(sV), ds0 = smem_u32(sdS);
      bool ok = mbar_wait(&bar_kv, 0, abortp, p.status, kBSiteKV);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        ok = mbar_wait(&bar_q_full[st], ph, abortp, p.status, kBSiteQFull, it);
        if (!ok) break;
        if (kAliasDQ && it > 0) {
          ok = mbar_wait(&bar_drained, (it - 1) & 1, abortp, p.status, kBSiteDrained, it);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t q0 = smem_u32(sQ + st * kTileBytes), do0 = smem_u32(sDO + st * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_ss(tbase + kColS, umma_desc_kmajor(k0 + off), umma_desc_kmajor(q0 + off), idS, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_ss(tbase + kColDP, umma_desc_kmajor(v0 + off), umma_desc_kmajor(do0 + off), idS, kk > 0);
        }
        tc_commit(&bar_s_full);
        ok = mbar_wait(&bar_pds, it & 1, abortp, p.status, kBSitePds, it);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)   // dV += P^T dO
          mma_ts(tbase + kColDV, tbase + kColS + kk * 8, umma_desc_mnmajor(do0 + kk * 2048, 16384), idKV,
                 acc | (kk > 0));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) { // dK += dS^T Q
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_ss(tbase + kColDK, umma_desc_kmajor(ds0 + off), umma_desc_mnmajor(q0 + kk * 2048, 16384), idKV,
                 acc | (kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)   // dQ_tile = dS [K | 1]
          mma_ss(tbase + kColDQ, umma_desc_mnmajor(ds0 + kk * 2048, 16384),
                 umma_desc_mnmajor(k0 + kk * 2048, 16384), idDQ, kk > 0);
        tc_commit(&bar_dq);
        tc_commit(&bar_q_empty[st]);
      }
      if (ok) tc_commit(&bar_done);
    }
  } else {
    // ===================== compute warps =====================
    const int j = nb * kBwdBN + tid;  // KV row owned by this thread
    const bool j_ok = (j < N) && (j >= seq0);
    const float* lam = p.lam + bh * N;
    const float b_j = (j < N) ? lam[j] * kLog2eB : 0.f;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tS = tbase + lane_base + kColS, tDP = tbase + lane_base + kColDP;
    const uint32_t tDQ = tbase + lane_base + kColDQ;
    float colsum = 0.f;
    bool ok = true;

    float e_next = -INFINITY, delta_next = 0.f;
    if (n_tiles > 0) {
      const int i = mb_lo * kBwdBM + tid;
      if (i < M) {
        const float Li = p.L[bh * M + i];
        e_next = (Li == -INFINITY) ? -INFINITY : (lam[P + i] - Li) * kLog2eB;
        delta_next = p.delta[bh * M + i];
      }
    }
    for (int it = 0; it < n_tiles; ++it) {
      const int mb = mb_lo + it;
      s_e[it & 1][tid] = e_next;
      s_delta[it & 1][tid] = delta_next;
      mbar_arrive(&bar_vec[it & 1]);
      if (it + 1 < n_tiles) {
        const int i = (mb + 1) * kBwdBM + tid;
        e_next = -INFINITY;
        delta_next = 0.f;
        if (i < M) {
          const float Li = p.L[bh * M + i];
          e_next = (Li == -INFINITY) ? -INFINITY : (lam[P + i] - Li) * kLog2eB;
          delta_next = p.delta[bh * M + i];
        }
      }
      ok = mbar_wait(&bar_vec[it & 1], (it >> 1) & 1, abortp, p.status, kBSiteVec, it);
      ok = mbar_wait(&bar_s_full, it & 1, abortp, p.status, kBSiteSFull, it) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // first query column of this tile this KV row may attend from (causal)
      const int c_min = j_ok ? max(j - P - mb * kBwdBM, 0) : kBwdBM;
      const float4* e4 = reinterpret_cast<const float4*>(s_e[it & 1]);
      const float4* d4 = reinterpret_cast<const float4*>(s_delta[it & 1]);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t sreg[32], dpreg[32], pk[16], dsk[16];
        tmem_ld32(tS + ch * 32, sreg);
        tmem_ld32(tDP + ch * 32, dpreg);
        tmem_ld_wait();
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 ev = e4[ch * 8 + c4];
          const float4 dv = d4[ch * 8 + c4];
          const float es[4] = {ev.x, ev.y, ev.z, ev.w};
          const float dl[4] = {dv.x, dv.y, dv.z, dv.w};
          float pv[4], dsv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = ch * 32 + c4 * 4 + e;
            float x = fmaf(__uint_as_float(sreg[c4 * 4 + e]), p.qk_scale, es[e]) - b_j;
            float pe = fast_exp2(x);
            pe = (c >= c_min) ? pe : 0.f;
            pv[e] = pe;
            dsv[e] = pe * (__uint_as_float(dpreg[c4 * 4 + e]) - dl[e]);
          }
          pk[c4 * 2] = pack2<kBf16>(pv[0], pv[1]);
          pk[c4 * 2 + 1] = pack2<kBf16>(pv[2], pv[3]);
          const uint32_t d01 = pack2<kBf16>(dsv[0], dsv[1]), d23 = pack2<kBf16>(dsv[2], dsv[3]);
          dsk[c4 * 2] = d01;
          dsk[c4 * 2 + 1] = d23;
          const float2 r01 = unpack2<kBf16>(d01), r23 = unpack2<kBf16>(d23);
          colsum += (r01.x + r01.y) + (r23.x + r23.y);
        }
        tmem_st16(tS + ch * 16, pk);  // columns [16 ch, 16 ch + 16) <- 32 probabilities; S chunk already in registers
        // dS^T row `tid`, columns [32 ch, 32 ch + 32): four 16-byte chunks of sub-tile ch/2
        uint8_t* drow = sdS + (ch >> 1) * 16384 + tid * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int cj = (ch & 1) * 4 + q4;
          *reinterpret_cast<uint4*>(drow + ((cj ^ (tid & 7)) << 4)) =
              make_uint4(dsk[q4 * 4], dsk[q4 * 4 + 1], dsk[q4 * 4 + 2], dsk[q4 * 4 + 3]);
        }
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_pds);

      // ---- drain dQ tile: thread t now owns query row mb*128 + t ----
      ok = mbar_wait(&bar_dq, it & 1, abortp, p.status, kBSiteDq, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        const int i = mb * kBwdBM + tid;
        float* dst = p.dq_accum + (bh * M + i) * D;
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t r[32];
          tmem_ld32(tDQ + c, r);
          tmem_ld_wait();
          if (i < M) {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              red_add_v4(dst + c + q4 * 4, __uint_as_float(r[q4 * 4]), __uint_as_float(r[q4 * 4 + 1]),
                         __uint_as_float(r[q4 * 4 + 2]), __uint_as_float(r[q4 * 4 + 3]));
          }
        }
        uint32_t rs[16];
        tmem_ld16(tDQ + D, rs);
        tmem_ld_wait();
        if (i < M) atomicAdd(p.dlam_row + bh * M + i, __uint_as_float(rs[0]));
      }
      if (kAliasDQ) {
        tc_fence_before();
        mbar_arrive(&bar_drained);
      }
    }

    // ---- epilogue: dK, dV, key-side log-gate gradient ----
    if (n_tiles > 0 && ok) {
      ok = mbar_wait(&bar_done, 0, abortp, p.status, kBSiteDone);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const bool keep = j_ok && n_tiles > 0;
      uint16_t* dkrow = reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_sb + h * p.dk_sh + static_cast<int64_t>(j) * p.dk_st;
      uint16_t* dvrow = reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_sb + h * p.dv_sh + static_cast<int64_t>(j) * p.dv_st;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t tcol = tbase + lane_base + (which == 0 ? kColDK : kColDV);
        const float sc = which == 0 ? p.sm_scale : 1.f;
        uint16_t* orow = which == 0 ? dkrow : dvrow;
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t r[32];
          if (n_tiles > 0) {
            tmem_ld32(tcol + c, r);
            tmem_ld_wait();
          }
          if (j < N) {
#pragma unroll
            for (int q8 = 0; q8 < 32; q8 += 8) {
              uint4 w = make_uint4(0, 0, 0, 0);
              if (keep) {
                w.x = pack2<kBf16>(__uint_as_float(r[q8 + 0]) * sc, __uint_as_float(r[q8 + 1]) * sc);
                w.y = pack2<kBf16>(__uint_as_float(r[q8 + 2]) * sc, __uint_as_float(r[q8 + 3]) * sc);
                w.z = pack2<kBf16>(__uint_as_float(r[q8 + 4]) * sc, __uint_as_float(r[q8 + 5]) * sc);
                w.w = pack2<kBf16>(__uint_as_float(r[q8 + 6]) * sc, __uint_as_float(r[q8 + 7]) * sc);
              }
              *reinterpret_cast<uint4*>(orow + c + q8) = w;
            }
          }
        }
      }
      if (j < N) p.dlam_col[bh * N + j] = keep ? -colsum : 0.f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tbase, kTmemCols);
}

template <int D, bool kBf16, int STAGES>
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
  constexpr int smem = (2 + 2 * STAGES) * 128 * D * 2 + 16384 + 32768 + 1024;
  auto kern = fox_attn_bwd_kernel<D, kBf16, STAGES>;
  static bool configured[64] = {};
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  if (!configured[device]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FOX_ERR_LAUNCH;
    configured[device] = true;
  }
  dim3 grid((unsigned)((N + kBwdBN - 1) / kBwdBN), (unsigned)H, (unsigned)B);
  kern<<<grid, kBwdThreads, smem, stream>>>(tmQ, tmK, tmV, tmDO, prm);
  return cudaGetLastError() == cudaSuccess ? FOX_OK : FOX_ERR_LAUNCH;
}

}  // namespace fox

extern "C" int fox_attn_bwd(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                            int64_t D, const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                            const fox_tensor4* d_o, const float* log_lambda, const float* L, const float* delta,
                            const int64_t* seq_start, const int64_t* end_index, float sm_scale,
                            float* dq_accum_zeroed, float* dlam_row_zeroed, float* dlam_col, const fox_tensor4* dk,
                            const fox_tensor4* dv, int32_t* status) {
  using namespace fox;
  if (!q || !k || !v || !d_o || !dk || !dv || !q->ptr || !k->ptr || !v->ptr || !d_o->ptr || !dk->ptr || !dv->ptr ||
      !log_lambda || !L || !delta || !dq_accum_zeroed || !dlam_row_zeroed || !dlam_col || !status)
    return FOX_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || M <= 0 || N <= 0 || M > N || H > 65535 || B > 65535) return FOX_ERR_BAD_ARG;
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
  prm.H = (int)H; prm.M = (int)M; prm.N = (int)N;
  prm.sm_scale = sm_scale;
  prm.qk_scale = sm_scale * 1.4426950408889634f;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = dtype == FOX_DTYPE_BF16;
  if (D == 64)
    return bf ? launch_bwd<64, true, 2>(device, st, B, H, M, N, q, k, v, d_o, prm)
              : launch_bwd<64, false, 2>(device, st, B, H, M, N, q, k, v, d_o, prm);
  return bf ? launch_bwd<128, true, 1>(device, st, B, H, M, N, q, k, v, d_o, prm)
            : launch_bwd<128, false, 1>(device, st, B, H, M, N, q, k, v, d_o, prm);
}
