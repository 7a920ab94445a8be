// Backward attention for callers that must not allocate device memory.
//
// The regular backward entry point (fox_attn_bwd) reduces dQ and the query-side
// log-gate gradient into two zero-initialised fp32 scratch arrays that its caller
// allocates.  Some hosts cannot do that at call time: a serving process or a
// framework that gave the whole GPU to its own arena at start-up has nothing
// left for cudaMalloc to hand out, and cudaMalloc / cudaFree also serialise the
// device, which a latency-critical thread may not be allowed to do.  For them
// this file keeps the scratch in a fixed array that is part of the loaded
// library image, and exposes one entry point that uses it.
//
// Consequences of a single fixed array, all of which the caller has to know:
//  * a GPU holds the array's kScratchFloats * 4 bytes (64 MiB) from the moment the
//    CUDA runtime loads this file's module on it until the process exits.  With the
//    runtime's default lazy module loading that moment is the FIRST CALL of this
//    entry point on the device (the address look-up below), and that first call
//    therefore does obtain device memory and may serialise the device once: make
//    it at start-up, on every device that will use the entry point, BEFORE the
//    host's arena takes the rest of the GPU, with any small valid problem.  With
//    CUDA_MODULE_LOADING=EAGER in the environment the array is placed when the
//    library's first CUDA call initialises the device, and every GPU that uses
//    the library holds it whether or not this entry point is ever called.  If the
//    device has no room for the array any more, the call returns
//    FOX_ERR_NO_MEMORY;
//  * B*H*M*(D+1) must not exceed kScratchFloats, larger problems are refused
//    with FOX_ERR_TOO_LARGE (use fox_attn_bwd with your own scratch);
//  * all calls on one device share the array and it keeps whatever the last call
//    left in it: the part a call needs is cleared on the caller's stream first,
//    and two calls whose work overlaps on the GPU (different streams, or graphs
//    replayed concurrently) race on it -- serialise them;
//  * the first call on each device looks the array's device address up
//    (cudaGetSymbolAddress, with that device current); make that first call
//    outside any stream capture.
//
// In host code `fox_scratch` is only a handle for the runtime, not a device
// address, so it is never passed to a kernel directly: the looked-up pointer is.
#include <mutex>

#include "fox_common.cuh"
#include "fox_host.h"

namespace fox {

constexpr int64_t kScratchFloats = int64_t(1) << 24;  // 16 Mi floats = 64 MiB per device

static __device__ __align__(256) float fox_scratch[kScratchFloats];

// device address of fox_scratch per CUDA ordinal, looked up on first use
static float* g_scratch_ptr[64] = {};
static std::mutex g_scratch_mu;

static int scratch_for_device(int device, float** out) {
  if (device < 0 || device >= 64) return FOX_ERR_DEVICE;
  std::lock_guard<std::mutex> g(g_scratch_mu);
  if (!g_scratch_ptr[device]) {
    if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
    void* p = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&p, fox_scratch);
    if (err == cudaErrorMemoryAllocation) {   // loading the module found no room for the array
      (void)cudaGetLastError();
      return FOX_ERR_NO_MEMORY;
    }
    if (err != cudaSuccess || !p) return FOX_ERR_DEVICE;
    g_scratch_ptr[device] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[device];
  return FOX_OK;
}

}  // namespace fox

extern "C" int64_t fox_noalloc_scratch_floats(void) { return fox::kScratchFloats; }

extern "C" int fox_attn_bwd_noalloc(int device, void* stream, int dtype, int64_t B, int64_t H, int64_t M, int64_t N,
                                    int64_t D, const fox_tensor4* q, const fox_tensor4* k, const fox_tensor4* v,
                                    const fox_tensor4* d_o, const float* log_lambda, const float* L,
                                    const float* delta, const int64_t* seq_start, const int64_t* end_index,
                                    float sm_scale, const fox_tensor4* dq, const fox_tensor4* dk,
                                    const fox_tensor4* dv, float* dlam_col, float* dlog_fgate, int32_t* status) {
  using namespace fox;
  if (B <= 0 || H <= 0 || M <= 0 || N <= 0 || M > N || !dq || !dq->ptr || !dlam_col || !dlog_fgate || !status)
    return FOX_ERR_BAD_ARG;
  // the same range checks fox_attn_bwd makes, before any product of the sizes is formed or anything is queued
  if (B > 65535 || H > 65535) return FOX_ERR_BAD_ARG;
  if (D != 64 && D != 128) return FOX_ERR_HEAD_DIM;
  if (dtype != FOX_DTYPE_BF16 && dtype != FOX_DTYPE_FP16) return FOX_ERR_BAD_ARG;
  if (N > 2147483647LL) return FOX_ERR_TOO_LARGE;
  if (M > kScratchFloats) return FOX_ERR_TOO_LARGE;   // (keeps B*H*M*(D+1) below 2^63)
  const int64_t rows = B * H * M;
  const int64_t need = rows * (D + 1);
  if (need > kScratchFloats) return FOX_ERR_TOO_LARGE;  // B*H*M*(D+1) floats do not fit the fixed array
  float* scratch = nullptr;
  int rc = scratch_for_device(device, &scratch);
  if (rc != FOX_OK) return rc;
  if (cudaSetDevice(device) != cudaSuccess) return FOX_ERR_DEVICE;
  float* dq_accum = scratch;              // (B,H,M,D)
  float* dlam_row = scratch + rows * D;   // (B,H,M)
  // the array still holds the previous call's sums: both halves are reduced into, so clear them
  if (cudaMemsetAsync(scratch, 0, sizeof(float) * static_cast<size_t>(need), static_cast<cudaStream_t>(stream)) !=
      cudaSuccess)
    return FOX_ERR_LAUNCH;
  rc = fox_attn_bwd(device, stream, dtype, B, H, M, N, D, q, k, v, d_o, log_lambda, L, delta, seq_start, end_index,
                    sm_scale, dq_accum, dlam_row, dlam_col, dk, dv, status);
  if (rc != FOX_OK) return rc;
  rc = fox_dq_convert(device, stream, dtype, B, H, M, D, dq_accum, sm_scale, dq);
  if (rc != FOX_OK) return rc;
  return fox_revcumsum(device, stream, B, H, M, N, dlam_col, dlam_row, nullptr, dlog_fgate, nullptr);
}
