/*
 * fox_b200.h -- C ABI of the B200 (sm_100a) Forgetting Attention library.
 *
 * The upstream project (zhixuan-lin/forgetting-transformer) is pure Python: its
 * operator boundary is the Python function
 *   forgetting_transformer.forgetting_attention(q, k, v, log_fgate, *, head_first,
 *       seq_start, sm_scale, adaptive_threshold)
 * (src/forgetting_transformer/ops/forgetting_attention.py:403-455) and the Triton
 * launches underneath it.  Each entry point below replaces one of those launches
 * (or the ATen call next to it) and cites the lines it stands in for.
 *
 * Conventions
 *  - every pointer is a device pointer unless stated otherwise; nothing here
 *    allocates device memory, synchronises the device or prints;
 *  - q/k/v-like tensors are logical (B, H, T, D) arrays of 16-bit floats with a
 *    unit stride on D and arbitrary element strides (sb, sh, st) on the rest,
 *    described by a fox_tensor4; base pointers and byte strides must be
 *    multiples of 16 (the Python host copies a view that is not);
 *  - (B, H, T) fp32 vectors (log_fgate, log_lambda, L, delta, dlog_lambda) are
 *    contiguous;
 *  - `dtype` is FOX_DTYPE_BF16 or FOX_DTYPE_FP16;
 *  - `stream` is a cudaStream_t passed as void*; `device` is the CUDA ordinal
 *    the buffers live on (made current for the duration of the call);
 *  - the return value is FOX_OK (0) or a negative FOX_ERR_* code.
 */
#ifndef FOX_B200_H_
#define FOX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FOX_OK 0
#define FOX_ERR_BAD_ARG (-1)      /* null pointer, negative size, M > N ...            */
#define FOX_ERR_HEAD_DIM (-2)     /* head dim not supported by the kernel              */
#define FOX_ERR_ALIGNMENT (-3)    /* base pointer / stride not 16-byte aligned         */
#define FOX_ERR_DRIVER (-4)       /* cuTensorMapEncodeTiled entry point unavailable    */
#define FOX_ERR_TENSORMAP (-5)    /* tensor-map encoding rejected the view             */
#define FOX_ERR_LAUNCH (-6)       /* cudaGetLastError() after the launch               */
#define FOX_ERR_DEVICE (-7)       /* cudaSetDevice failed / not an sm_100 device       */
#define FOX_ERR_TOO_LARGE (-8)    /* size beyond a documented maximum                  */
#define FOX_ERR_THRESHOLD (-9)    /* reserved                                          */

#define FOX_DTYPE_FP16 0
#define FOX_DTYPE_BF16 1

typedef struct fox_tensor4 {
  void* ptr;
  int64_t sb, sh, st; /* element strides of the B, H and T axes; D has stride 1 */
} fox_tensor4;

/* Block geometry of the attention kernels.  Adaptive Computation Pruning works on
 * whole blocks, so the index arrays below are defined relative to these sizes
 * (they play the role of get_fwd_config / get_bwd_kv_config / get_bwd_q_config,
 * forgetting_attention.py:460-493, 838-890). */
#define FOX_FWD_BLOCK_M 128
#define FOX_FWD_BLOCK_N 128
#define FOX_BWD_BLOCK_M 128
#define FOX_BWD_BLOCK_N 128

/* Library / build information: returns a static string. */
const char* fox_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FOX_B200_H_ */
