// Device-side building blocks shared by the sm_100a kernels of this library:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM alloc/ld/st, commit)
// wrappers, UMMA descriptor builders and the bounded-wait / abort protocol.
//
// Every spin-wait in this library is bounded.  A waiter that runs out of its
// budget records (site, block) in a global error word, raises a CTA-wide
// abort flag in shared memory and returns false; every other waiter polls the
// abort flag and bails out as well, so a protocol bug ends as an error code
// read by the host, never as a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fox {

// ---------------------------------------------------------------- error word
// layout of the int32[4] status buffer the attention kernels write to:
//   [0] first failing wait site (0 = ok), [1] blockIdx.x of the failing CTA,
//   [2] thread index, [3] free-form detail (tile index).
constexpr int kStatusWords = 4;


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  // make barrier initialisation visible to the async proxy (TMA, tcgen05.commit)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory; `status` in global.
// The fast path is a two-instruction loop around mbarrier.try_wait with a suspend-time hint:
// a waiting warp is parked by the hardware instead of burning issue slots that the compute
// warps on the same scheduler need.  kWaitTries x kWaitHintNs (~2 s) bounds the wait.
constexpr uint32_t kWaitHintNs = 500000u;
constexpr uint32_t kWaitTries = 4000u;
constexpr uint32_t kWaitTriesBackoff = 20000000u;  // x (>= 32 ns sleep + poll) ~ 2 s
template <bool kBackoff = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int site, int detail = 0) {
  // fast path: the phase has usually completed already; one plain try_wait costs ~15 cycles
  if (mbar_try_wait(bar, parity)) return true;
  uint32_t ok;
  const uint32_t addr = smem_u32(bar);
  if (kBackoff) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .u32 n;\n\tmov.u32 n, 0;\n"
        "FOX_WAITB_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra FOX_WAITB_DONE;\n\t"
        "nanosleep.u32 20;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra FOX_WAITB_LOOP;\n"
        "FOX_WAITB_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(*abort_flag ? 1u : kWaitTriesBackoff)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .u32 n;\n\tmov.u32 n, 0;\n"
        "FOX_WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "@p bra FOX_WAIT_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %4;\n\t"
        "@q bra FOX_WAIT_LOOP;\n"
        "FOX_WAIT_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(kWaitHintNs), "r"(*abort_flag ? 1u : kWaitTries)
        : "memory");
  }
  if (ok) return true;
  // ran out of budget (or another waiter already did): record the first failing site and give up
  if (!*abort_flag) {
    *abort_flag = 1;
    if (atomicCAS(&status[0], 0, site) == 0) {
      status[1] = static_cast<int>(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
      status[2] = static_cast<int>(threadIdx.x);
      status[3] = detail;
    }
  }
  return false;
}

// Warp-collective form: every lane waits, the outcome is made uniform so the warp stays converged.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int site, int detail = 0) {
  const bool ok = mbar_wait<false>(bar, parity, abort_flag, status, site, detail);
  return __all_sync(0xffffffffu, ok);
}

// ----------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}
// 4-D tiled load, coordinates innermost first.  c0 * elem_size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tm, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 4-D tiled store from shared memory (bulk-group completion).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* tm, const void* smem_src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(tm)),
      "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 4-D tiled fp32 add-reduction from shared memory into global memory.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* tm, const void* smem_src, int c0,
                                                  int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::
          "l"(reinterpret_cast<uint64_t>(tm)),
      "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA / UMMA)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------- tcgen05
// One lane of a fully converged warp.  tcgen05.mma / commit / TMA take their operands from
// uniform registers: issued from a converged warp (every lane computes the same operands, one
// elected lane executes) they issue back to back; issued from a diverged `lane == 0` branch
// each instruction costs ~170 cycles (measured), several times the tensor pipe's own rate.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred px;\n\telect.sync _|px, 0xffffffff;\n\tselp.u32 %0, 1, 0, px;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Raw forms: to be executed by ONE lane, inside an `if (elect_one())` block of a converged warp
// whose operands were computed by all lanes (so they live in uniform registers).
__device__ __forceinline__ void tc_commit_raw(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mma_ss_raw(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_raw(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The three wrappers below must be called by ALL lanes of a converged warp; one lane executes.
// arrive (count 1) on `bar` once every tcgen05.mma issued so far by this warp retired
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  const uint32_t addr = smem_u32(bar);
  if (elect_one())
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(addr) : "memory");
  __syncwarp();
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  if (elect_one())
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  __syncwarp();
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  if (elect_one())
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  __syncwarp();
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 bit, 32 consecutive columns: thread t of the warp gets lane
// (base_lane + t), registers r[0..31] = columns col..col+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Matrix-fragment shapes: the warp touches 16 lanes (base lane of taddr: the warp's own quarter, +0 or +16).
// 16 lanes x 256 bit, four times (32 columns): thread t gets, for each 8-column group k,
//   r[4k + 0], r[4k + 1] = lane (t / 4),     columns 8k + 2 (t % 4), + 1
//   r[4k + 2], r[4k + 3] = lane (t / 4) + 8, the same two columns
// (the accumulator fragment of an m16n8 product).
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 128 bit, four times (16 columns): r[2k + 0] = lane (t / 4), column 4k + (t % 4);
// r[2k + 1] = lane (t / 4) + 8, the same column -- the fragment above with each column pair packed into 32 bits.
__device__ __forceinline__ void tmem_st_16x128b_x4(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
// Four 8x8 matrices of 16-bit elements to shared memory: matrix m's row (t % 8) is written at the address
// given by thread 8 m + (t % 8) (16 contiguous bytes); register m of thread t holds that matrix's row t / 4,
// columns 2 (t % 4), + 1.
__device__ __forceinline__ void stmatrix_x4(uint32_t smem_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(smem_addr), "r"(a),
               "r"(b), "r"(c), "r"(d)
               : "memory");
}

// ------------------------------------------------------------ UMMA descriptors
// Shared-memory tiles are [rows][64 x 16-bit] = 128-byte rows, 8-row groups of
// 1024 bytes, 128-byte swizzle (16-byte chunk index XOR (row & 7)); tile bases
// are 1024-byte aligned.  This is both what TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B and the canonical UMMA SWIZZLE_128B layout.
constexpr uint32_t kSwizzleRowBytes = 128;
constexpr uint32_t kSwizzleGroupBytes = 1024;  // 8 rows

// byte offset of 16-bit element (row, col) inside one [rows][64] swizzled tile
__device__ __forceinline__ uint32_t swz128_offset(uint32_t row, uint32_t col) {
  const uint32_t chunk = (col >> 3) ^ (row & 7);
  return row * kSwizzleRowBytes + (chunk << 4) + ((col & 7) << 1);
}

// Descriptor of an operand whose reduction (K) dimension is the contiguous one
// ("K-major"): rows = M or N index.  `addr` may be advanced by 32 bytes per
// 16-element K step inside a 64-element tile.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);              // start address
  d |= static_cast<uint64_t>(1) << 16;                                 // LBO (unused with swizzle)
  d |= static_cast<uint64_t>(kSwizzleGroupBytes >> 4) << 32;           // SBO: next 8-row group
  d |= static_cast<uint64_t>(1) << 46;                                 // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                                 // SWIZZLE_128B
  return d;
}
// Descriptor of an operand whose M/N dimension is the contiguous one
// ("MN-major"): rows = K index.  `lbo_bytes` is the distance between
// successive 64-element tiles along M/N; one 16-row K step is 2048 bytes.
__device__ __forceinline__ uint64_t umma_desc_mnmajor(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;         // LBO: next 64-wide tile along M/N
  d |= static_cast<uint64_t>(kSwizzleGroupBytes >> 4) << 32;           // SBO: next 8 K rows
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Advance a descriptor's start address by `bytes` (a multiple of 16; the tile stays below the
// 256 KiB the 14-bit field can address, so the add never carries into the next field).
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t desc, uint32_t bytes) {
  return desc + static_cast<uint64_t>(bytes >> 4);
}
// kind::f16 instruction descriptor, fp32 accumulate.  fmt: 0 = fp16, 1 = bf16.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t fmt, uint32_t m, uint32_t n, uint32_t a_mn_major,
                                                  uint32_t b_mn_major) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// ------------------------------------------------------------------- helpers
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (kBf16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}
// 2^x for two values on the FMA pipe (no ex2 unit): x = n + f with n = round(x), f in [-0.5, 0.5];
// 2^f by a cubic (relative error 7.5e-5, below 16-bit rounding), 2^n by adding n to the exponent
// field.  x is clamped to >= -125 (result 2^-125 instead of a denormal or zero); x must stay below 2^22.
__device__ __forceinline__ float2 poly_exp2_x2(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);  // 1.5 * 2^23: the sum's low mantissa bits hold n
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 xr = __fadd2_rn(x, magic);
  const float2 n = __fadd2_rn(xr, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(make_float2(0.0551716685f, 0.0551716685f), f, make_float2(0.24261114f, 0.24261114f));
  p = __ffma2_rn(p, f, make_float2(0.693260968f, 0.693260968f));
  p = __ffma2_rn(p, f, make_float2(0.999928057f, 0.999928057f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(xr.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(xr.y) << 23));
  return r;
}

// Read-only global load that stays where it is written: the compiler may sink a plain load down to its
// first use, which puts the whole memory latency in front of that use; a volatile asm is not moved.
__device__ __forceinline__ float ldg_f32_here(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace fox
