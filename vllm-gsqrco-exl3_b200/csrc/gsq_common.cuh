// Shared device/host helpers of the gsq kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gsq.h"
#include "../../include/gsq_debug.h"

#define GSQ_WARP 32
#define GSQ_QK_K 256

namespace gsq {

// thread-local record of the last failing CUDA call (read through gsq_last_cuda_error)
int record_cuda_error(cudaError_t e);
#define GSQ_CUDA_TRY(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return gsq::record_cuda_error(_e); \
  } while (0)

// activation tiles of the prefill GEMMs: besides GSQ_Q8_LAYOUT_D4 / _DS4, the quants as fp16 with fp32 d (gsq_gemm3.cu)
constexpr int Q8_TILES_H16 = 2;
// the products d * q themselves as fp16, scaled by a power of two per token: the rounded product alone (16 KB per unit)
// or with the rounding's remainder as a second fp16 plane (2 x 16 KB per unit); see gemm3_acc_kernel
constexpr int Q8_TILES_F16S = 3, Q8_TILES_F16S2 = 4;
// Q8_TILES_F16S with d and the sum of x kept as halves (Q4_K's q8_1 form) and, behind the units, the scaled sums as a
// tensor-core operand of their own: one 8 KB unit per token block and superblock
constexpr int Q8_TILES_F16SD = 5;

struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
  bool ready;
};
// cached facts about the current device (filled by gsq_device_init)
int device_info(DeviceInfo* out);

__host__ __device__ constexpr int block_bytes(int t) {
  return t == GSQ_TYPE_Q4_K     ? 144
         : t == GSQ_TYPE_Q6_K   ? 210
         : t == GSQ_TYPE_IQ3_S  ? 110
         : t == GSQ_TYPE_IQ4_XS ? 136
         : t == GSQ_TYPE_Q2_K   ? 84
         : t == GSQ_TYPE_IQ2_XXS ? 66
         : t == GSQ_TYPE_IQ2_XS ? 74
         : t == GSQ_TYPE_IQ3_XXS ? 98
         : t == GSQ_TYPE_IQ2_S  ? 82
         : t == GSQ_TYPE_IQ1_M  ? 56
                                : 0;
}

__device__ __forceinline__ float h2f(uint32_t bits16) {
  return __half2float(__ushort_as_half((unsigned short)(bits16 & 0xFFFFu)));
}

__device__ __forceinline__ int dp4a(int a, int b, int c) { return __dp4a(a, b, c); }

// streaming loads: weights are read once, keep them out of L1
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u16(const void* p) {
  unsigned short v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u8(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void store_out_dyn(void* y, int y_dtype, int64_t idx, float v) {
  if (y_dtype == GSQ_F32) {
    ((float*)y)[idx] = v;
  } else if (y_dtype == GSQ_F16) {
    ((__half*)y)[idx] = __float2half_rn(v);
  } else {
    ((__nv_bfloat16*)y)[idx] = __float2bfloat16_rn(v);
  }
}

}  // namespace gsq
