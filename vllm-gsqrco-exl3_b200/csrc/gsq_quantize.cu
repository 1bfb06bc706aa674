// q8_1 activation quantisers for fp32 / fp16 / bf16 X (sm_100a).
//
// Same arithmetic, bit for bit, as the reference's quantize_q8_1_x and quantize_mmq_q8_1_x
// (plugin/vllm_gguf_plugin/csrc/lcpp_shim.cu:274-294, 298-355), which are built with
// --use_fast_math (plugin/setup.py:42): divisions are the approximate div.approx.ftz / rcp.approx.ftz
// forms, written out explicitly here so this file needs no global fast-math flag. The launch shape
// differs: each thread owns 8 consecutive values (one 128-bit load of 16-bit X), 4 threads share a
// 32-value block. The block sum is formed in the same order as the reference's 16,8,4,2,1
// xor-shuffle tree over one value per lane (common.cuh:468-475): lane offsets 16 and 8 become
// thread offsets 2 and 1, offsets 4,2,1 become a tree inside the thread.
#include "gsq_common.cuh"

namespace gsq {

__device__ __forceinline__ float div_approx(float a, float b) {
  float r;
  asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float rcp_approx(float a) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// 8 consecutive values of row `row` starting at column c (c % 8 == 0). VEC: 16-byte aligned rows.
// Loads go to L2 (ld.global.cg): launched as a programmatic dependent, this kernel can be resident while the
// kernel that writes X still runs, so X is not read-only for its lifetime and the non-coherent path is not valid.
template <typename T, bool VEC>
__device__ __forceinline__ void load8(const T* __restrict__ x, int64_t off, float (&v)[8]) {
  if constexpr (VEC && sizeof(T) == 2) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x + off));
    const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = to_f32<T>(p[e]);
  } else if constexpr (VEC && sizeof(T) == 4) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(x + off));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(x + off + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = to_f32<T>(__ldcg(x + off + e));
  }
}

__device__ __forceinline__ uint32_t pack4(float a, float b, float c, float d) {
  // float -> int8 as the C conversion in the reference (round toward zero of an already rounded value)
  const int ia = (int)a, ib = (int)b, ic = (int)c, id = (int)d;
  return (uint32_t)(ia & 0xFF) | ((uint32_t)(ib & 0xFF) << 8) | ((uint32_t)(ic & 0xFF) << 16) | ((uint32_t)(id & 0xFF) << 24);
}

// This thread's 8 consecutive values (piece `piece` of the 32-value block its 4 adjacent lanes share) -> block_q8_1 at
// `b`. All 32 lanes of the warp must call it (shuffles); dead lanes pass zeros and live = false.
__device__ __forceinline__ void q8_1_store8(const float (&v)[8], bool live, uint8_t* b, int piece) {
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  float s[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) s[e] = v[e] + __shfl_xor_sync(0xFFFFFFFFu, v[e], 2);  // lane offset 16
#pragma unroll
  for (int e = 0; e < 8; ++e) s[e] = s[e] + __shfl_xor_sync(0xFFFFFFFFu, s[e], 1);  // lane offset 8
  const float s0 = s[0] + s[4], s1 = s[1] + s[5], s2 = s[2] + s[6], s3 = s[3] + s[7];  // offset 4
  const float sum = (s0 + s2) + (s1 + s3);                                              // offsets 2, 1
  if (!live) return;
  const float d = div_approx(amax, 127.0f);
  float q[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) q[e] = amax == 0.0f ? 0.0f : roundf(div_approx(v[e], d));
  uint32_t* q32 = reinterpret_cast<uint32_t*>(b + 4 + piece * 8);  // the quants follow the (d, sum) pair
  q32[0] = pack4(q[0], q[1], q[2], q[3]);
  q32[1] = pack4(q[4], q[5], q[6], q[7]);
  if (piece == 0) {
    *reinterpret_cast<__half2*>(b) = __floats2half2_rn(d, sum);
  }
}

// MMVQ layout: block_q8_1 = half d, half sum, 32 x int8 (36 bytes).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                           int64_t m, int64_t k, int64_t stride) {
  // a product kernel launched behind this one with programmatic stream serialisation may start its prologue now;
  // it waits for this grid to finish before it reads `out`
  asm volatile("griddepcontrol.launch_dependents;");
  // this kernel is itself launched with programmatic stream serialisation: it may be scheduled while the kernel
  // before it drains, and waits here until that one has finished and its writes (X, perhaps) are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 values
  const int64_t per_row = k >> 3;
  // whole warps stay together: k % 32 == 0 makes per_row a multiple of 4, so a 4-thread group never
  // straddles the end of the work
  const bool live = t < m * per_row;
  const int64_t row = live ? t / per_row : 0;
  const int64_t c8 = live ? t - row * per_row : 0;
  float v[8];
  if (live) {
    load8<T, VEC>(x, row * stride + c8 * 8, v);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.0f;
  }
  q8_1_store8(v, live, out + (row * (k >> 5) + (c8 >> 2)) * 36, (int)(c8 & 3));
}

// 128-value blocks: 16 scale bytes + 128 x int8, block (kb, row) at (kb * m + row) * 144.
template <typename T, bool VEC, int LAYOUT>
__global__ void __launch_bounds__(256) quantize_q8_1_mmq_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                               int64_t m, int64_t k, int64_t stride) {
  asm volatile("griddepcontrol.launch_dependents;");
  // this kernel is itself launched with programmatic stream serialisation: it may be scheduled while the kernel
  // before it drains, and waits here until that one has finished and its writes (X, perhaps) are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t per_row = k >> 3;
  const bool live = t < m * per_row;
  const int64_t row = live ? t / per_row : 0;
  const int64_t c8 = live ? t - row * per_row : 0;
  float v[8];
  if (live) {
    load8<T, VEC>(x, row * stride + c8 * 8, v);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.0f;
  }
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  float sum = 0.0f;
  if constexpr (LAYOUT == GSQ_Q8_LAYOUT_DS4) {
    // the reference sums 4 values per thread, then lane offsets 4, 2, 1 over 8 threads
    float pa = ((v[0] + v[1]) + v[2]) + v[3];
    float pb = ((v[4] + v[5]) + v[6]) + v[7];
    pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 2);
    pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 2);
    pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 1);
    pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 1);
    sum = pa + pb;
  }
  if (!live) return;
  const float d_inv = div_approx(127.0f, amax);
  float q[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) q[e] = roundf(v[e] * d_inv);
  const float d = rcp_approx(d_inv);
  const int64_t kb = c8 >> 4;             // 128-value block along k
  const int iqs = (int)(c8 & 15) * 8;     // value offset inside the block
  uint8_t* b = out + (kb * m + row) * 144;
  *reinterpret_cast<uint2*>(b + 16 + iqs) = make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
  if ((iqs & 31) == 0) {
    if constexpr (LAYOUT == GSQ_Q8_LAYOUT_DS4) {
      reinterpret_cast<__half2*>(b)[iqs >> 5] = __floats2half2_rn(d, sum);
    } else {
      reinterpret_cast<float*>(b)[iqs >> 5] = d;
    }
  }
}

// Per token (one warp each) the power of two that brings its largest magnitude over all of k to [2^13, 2^14), stored as
// its reciprocal; tokens past m get 0, a token of zeros 1. For the scaled-product units below.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) row_scale_kernel(const T* __restrict__ x, float* __restrict__ inv_scale, int64_t m,
                                                       int64_t mpad, int64_t k, int64_t stride) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= mpad) return;
  if (row >= m) {
    if (lane == 0) inv_scale[row] = 0.0f;
    return;
  }
  float amax = 0.0f;
  for (int64_t c = 8 * lane; c < k; c += 256) {
    float v[8];
    load8<T, VEC>(x, row * stride + c, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if (lane == 0) {
    float inv = 1.0f;
    if (amax > 0.0f && amax <= 3.0e38f) {
      int e;
      frexpf(amax, &e);                        // amax = f * 2^e, f in [0.5, 1)
      const int up = min(max(14 - e, -100), 100);
      inv = ldexpf(1.0f, -up);
    }
    inv_scale[row] = inv;
  }
}

// Activation units of the prefill GEMMs (gsq_gemm2.cu, gsq_gemm3.cu): the same quantisation as
// quantize_q8_1_mmq_kernel (32-value blocks, d = 1 / (127 / amax), D4 or DS4 scales), written in the shared-memory layout
// of the tensor-core operand so that one bulk copy brings a unit into place. A unit is one 32-value slice of a block
// of 256 tokens, [token block][superblock][slice][unit]:
//   int8 operands:  [32 token groups][2 K chunks of 16][8 tokens][16 bytes] quants       (8192 bytes)
//                   [256 tokens] float d                                                 (1024 bytes)
//                   [256 tokens] float(half(sum x))   (DS4 only)                         (1024 bytes)
//   fp16 operands (LAYOUT = Q8_TILES_H16): the same quants as fp16 numbers
//                   [32 token groups][4 K chunks of 8][8 tokens][8 fp16] quants          (16384 bytes)
//                   [256 tokens] float d                                                 (1024 bytes)
//   scaled products (LAYOUT = Q8_TILES_F16S / _F16S2): in the fp16 operand order, hi = fp16(d * q * 2^e[token]) (16384
//                   bytes) and, for _F16S2, lo = fp16(d * q * 2^e - hi) (16384 more); after the last unit one float
//                   per token of the padded range, 2^-e[token] (row_scale_kernel: 2^e brings the token's largest
//                   magnitude to [2^13, 2^14), so no product overflows fp16 and hi + lo carries 22 bits of each)
//   ... with sums (LAYOUT = Q8_TILES_F16SD, for Q4_K): d and sum x rounded to halves as the reference's DS4 blocks
//                   keep them; between the last unit and the per-token floats one 8 KB unit per token block and
//                   superblock, [32 token groups][2 K chunks of 8][8 tokens][8 fp16], for the 8 slices:
//                   chunk 0 = half(sum x) * 2^(e - 4) (exact, below 2^15: the minimum term's activations);
//                   chunk 1 = (sum of the slice's exact products - sum of the rounded ones) * 2^-4, what the rounding
//                   took from the slice in total. Q4_K's quants are all of one sign (0..15), so the roundings would
//                   add up along a slice as 8 sc * (sum of the errors); the kernel adds that amount back.
// Tokens past m (up to the end of the last block) are written as zeros. One CUDA block = 64 tokens x one slice:
// warp w holds token group w of the 64, lane = (token % 8) * 4 + 8-value piece, so a warp writes whole core matrices.
template <typename T, bool VEC, int LAYOUT>
__global__ void __launch_bounds__(256) quantize_q8_1_tiles_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                                 int64_t m, int64_t k, int64_t stride) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr bool SD = LAYOUT == Q8_TILES_F16SD;
  constexpr bool DS = LAYOUT == GSQ_Q8_LAYOUT_DS4 || SD, H16 = LAYOUT == Q8_TILES_H16;
  constexpr bool F16S = LAYOUT == Q8_TILES_F16S || LAYOUT == Q8_TILES_F16S2 || SD, LO = LAYOUT == Q8_TILES_F16S2;
  constexpr int UB = F16S ? (LO ? 32768 : 16384) : H16 ? 16384 + 1024 : 8192 + (DS ? 2048 : 1024);
  const int slice = blockIdx.x;              // 32-value slice along k
  const int64_t tt = blockIdx.y;             // token tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = 8 * warp + (lane >> 2), piece = lane & 3;
  const int64_t row = tt * 64 + r;
  const bool live = row < m;
  float v[8];
  if (live) {
    load8<T, VEC>(x, row * stride + (int64_t)slice * 32 + piece * 8, v);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.0f;
  }
  float amax = 0.0f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  float sum = 0.0f;
  if constexpr (DS) {
    float pa = ((v[0] + v[1]) + v[2]) + v[3];
    float pb = ((v[4] + v[5]) + v[6]) + v[7];
    pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 2);
    pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 2);
    pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 1);
    pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 1);
    sum = pa + pb;
  }
  const float d_inv = div_approx(127.0f, amax);
  float q[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) q[e] = live && amax > 0.0f ? roundf(v[e] * d_inv) : 0.0f;   // (a block of zeros: 0 * inf)
  float d = live ? rcp_approx(d_inv) : 0.0f;
  const int sb = slice >> 3, s = slice & 7;
  const int rb = (int)(tt & 3) * 64 + r;   // token within its block of 256
  uint8_t* unit = out + (((tt >> 2) * (k >> 8) + sb) * 8 + s) * UB;
  if constexpr (F16S) {
    uint8_t* behind = out + (int64_t)gridDim.y / 4 * (k >> 8) * 8 * UB;     // what follows the last unit
    const float* inv_scale = reinterpret_cast<const float*>(behind + (SD ? (int64_t)gridDim.y / 4 * (k >> 8) * 8192 : 0));
    const float up = live ? 1.0f / inv_scale[row] : 0.0f;         // 2^e, a power of two: the products below are exact
    float sum_half = 0.0f;
    if constexpr (SD) {
      const float2 dsum = __half22float2(__floats2half2_rn(d, sum));   // the reference keeps half2(d, sum)
      d = dsum.x;
      sum_half = dsum.y;
    }
    const float ds = d * up;
    uint8_t* dst = unit + (rb >> 3) * 512 + piece * 128 + (rb & 7) * 16;
    __half2 hi[4], lo[4];
    float lost = 0.0f;   // exact products minus rounded ones, this lane's 8 values
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p0 = ds * q[2 * e], p1 = ds * q[2 * e + 1];
      hi[e] = __floats2half2_rn(p0, p1);
      const float2 back = __half22float2(hi[e]);
      lo[e] = __floats2half2_rn(p0 - back.x, p1 - back.y);
      lost += (p0 - back.x) + (p1 - back.y);
    }
    if constexpr (SD) {
      lost += __shfl_xor_sync(0xFFFFFFFFu, lost, 2);
      lost += __shfl_xor_sync(0xFFFFFFFFu, lost, 1);
      if (piece == 0) {
        uint8_t* su = behind + ((tt >> 2) * (k >> 8) + sb) * 8192 + (rb >> 3) * 256 + (rb & 7) * 16;
        reinterpret_cast<__half*>(su)[s] = __float2half_rn(sum_half * up * 0.0625f);
        reinterpret_cast<__half*>(su + 128)[s] = __float2half_rn(lost * 0.0625f);
      }
    }
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(hi);
    if constexpr (LO) *reinterpret_cast<uint4*>(dst + 16384) = *reinterpret_cast<const uint4*>(lo);
    return;
  }
  if constexpr (H16) {
    // the lane's 8 values are one 16-byte row of a core matrix (integers up to 127 in magnitude: exact in fp16)
    uint8_t* dst = unit + (rb >> 3) * 512 + piece * 128 + (rb & 7) * 16;
    __half2 h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(q[2 * e], q[2 * e + 1]);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
    if (piece == 0) reinterpret_cast<float*>(unit + 16384)[rb] = d;
    return;
  }
  uint8_t* dst = unit + (rb >> 3) * 256 + (piece >> 1) * 128 + (rb & 7) * 16 + (piece & 1) * 8;
  *reinterpret_cast<uint2*>(dst) = make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
  if (piece == 0) {
    float* sc = reinterpret_cast<float*>(unit + 8192);
    if constexpr (DS) {
      const float2 ds = __half22float2(__floats2half2_rn(d, sum));   // the reference keeps half2(d, sum)
      sc[rb] = live ? ds.x : 0.0f;
      sc[256 + rb] = live ? ds.y : 0.0f;
    } else {
      sc[rb] = d;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The two element-wise steps that stand in front of a quantised linear in a decoder layer, fused with its q8_1
// quantiser (block_q8_1 layout), so that the step costs one launch and the normalised / activated values never make
// a round trip through memory on their way to the quantiser. The arithmetic between the steps is the unfused one:
// every intermediate is rounded to X's type where the separate kernels would have stored it, and the quantiser part
// is q8_1_store8 above, so the q8_1 bytes equal quantising the (optional) y_out of the same call bit for bit.

template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) store_out<T>(p + e, v[e]);
}

// RMSNorm (optionally with the residual add in front of it) -> q8_1. One CTA per row:
//   z = T(x + residual)          (residual updated in place; z = x without one)
//   var = sum z^2 / k            (fp32: each thread adds its items in order, lanes by the 16-8-4-2-1 xor tree, the
//                                 eight warps' sums in warp order)
//   y = T(T(z * rsqrt(var + eps)) * gamma)
// which is vLLM's rms_norm / fused_add_rms_norm arithmetic (csrc/layernorm_kernels.cu: the scaled value is converted
// to the tensor's type before the multiplication by the weight), then quantised.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_q8_1_kernel(const T* __restrict__ x, int64_t stride, T* __restrict__ residual,
                                                          const T* __restrict__ gamma, float eps, uint8_t* __restrict__ out,
                                                          T* __restrict__ y_out, int64_t k) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float zrow[];          // the row after the residual add, as fp32
  __shared__ float wsum[8];
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, per_row = (int)(k >> 3);
  float ss = 0.0f;
  for (int it = tid; it < per_row; it += 256) {
    float v[8];
    load8<T, false>(x, row * stride + (int64_t)it * 8, v);
    if (residual) {
      float r[8];
      load8<T, false>(residual, row * k + (int64_t)it * 8, r);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = round_to<T>(v[e] + r[e]);
      store8<T>(residual + row * k + (int64_t)it * 8, v);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      zrow[it * 8 + e] = v[e];
      ss = fmaf(v[e], v[e], ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((tid & 31) == 0) wsum[tid >> 5] = ss;
  __syncthreads();
  float tot = wsum[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) tot += wsum[w];
  const float rs = rsqrtf(tot / (float)k + eps);
  // whole warps pass q8_1_store8 together: the loop bound is rounded up to the warp
  for (int it0 = 0; it0 < per_row; it0 += 256) {
    const int it = it0 + tid;
    const bool live = it < per_row;
    float v[8];
    if (live) {
      float g[8];
      load8<T, false>(gamma, (int64_t)it * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = round_to<T>(round_to<T>(zrow[it * 8 + e] * rs) * g[e]);
      if (y_out) store8<T>(y_out + row * k + (int64_t)it * 8, v);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.0f;
    }
    q8_1_store8(v, live, out + (row * (k >> 5) + (it >> 2)) * 36, it & 3);
  }
}

// SwiGLU -> q8_1: gate_up [m, 2 * inter] (gate = the first `inter` columns, up = the rest), as vLLM's silu_and_mul
// (csrc/activation_kernels.cu): y = T(g / (1 + exp(-g))) * u in T arithmetic, then quantised over the `inter` columns.
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_q8_1_kernel(const T* __restrict__ gu, int64_t stride, uint8_t* __restrict__ out,
                                                           T* __restrict__ y_out, int64_t m, int64_t inter) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 values
  const int64_t per_row = inter >> 3;
  const bool live = t < m * per_row;
  const int64_t row = live ? t / per_row : 0;
  const int64_t c8 = live ? t - row * per_row : 0;
  float v[8];
  if (live) {
    float g[8], u[8];
    load8<T, false>(gu, row * stride + c8 * 8, g);
    load8<T, false>(gu, row * stride + inter + c8 * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = round_to<T>(round_to<T>(g[e] / (1.0f + expf(-g[e]))) * u[e]);
    if (y_out) store8<T>(y_out + row * inter + c8 * 8, v);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.0f;
  }
  q8_1_store8(v, live, out + (row * (inter >> 5) + (c8 >> 2)) * 36, (int)(c8 & 3));
}

// launch with programmatic stream serialisation (see griddepcontrol.wait in the kernels)
template <typename... KArgs, typename... Args>
static int launch_pdl(void (*kern)(KArgs...), unsigned grid, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, args...));
  return GSQ_OK;
}

template <typename T>
static int launch_q8_1(const void* x, int64_t m, int64_t k, int64_t stride, void* out, cudaStream_t st) {
  const int64_t threads = m * (k >> 3);
  if (threads == 0) return GSQ_OK;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  const bool vec = ((uintptr_t)x % 16 == 0) && ((stride * (int64_t)sizeof(T)) % 16 == 0);
  return vec ? launch_pdl(quantize_q8_1_kernel<T, true>, grid, st, (const T*)x, (uint8_t*)out, m, k, stride)
             : launch_pdl(quantize_q8_1_kernel<T, false>, grid, st, (const T*)x, (uint8_t*)out, m, k, stride);
}

template <typename T, int LAYOUT>
static int launch_q8_1_mmq(const void* x, int64_t m, int64_t k, int64_t stride, void* out, cudaStream_t st) {
  const int64_t threads = m * (k >> 3);
  if (threads == 0) return GSQ_OK;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  const bool vec = ((uintptr_t)x % 16 == 0) && ((stride * (int64_t)sizeof(T)) % 16 == 0);
  return vec ? launch_pdl(quantize_q8_1_mmq_kernel<T, true, LAYOUT>, grid, st, (const T*)x, (uint8_t*)out, m, k, stride)
             : launch_pdl(quantize_q8_1_mmq_kernel<T, false, LAYOUT>, grid, st, (const T*)x, (uint8_t*)out, m, k, stride);
}

template <typename T, int LAYOUT>
static int launch_q8_1_tiles(const void* x, int64_t m, int64_t k, int64_t stride, void* out, cudaStream_t st) {
  if (m == 0) return GSQ_OK;
  const bool vec = ((uintptr_t)x % 16 == 0) && ((stride * (int64_t)sizeof(T)) % 16 == 0);
  if constexpr (LAYOUT == Q8_TILES_F16S || LAYOUT == Q8_TILES_F16S2 || LAYOUT == Q8_TILES_F16SD) {
    // first the per-token scales, behind the last unit (and the units of sums)
    const int64_t mpad = (m + 255) / 256 * 256;
    float* inv_scale = reinterpret_cast<float*>((uint8_t*)out + mpad / 256 * (k >> 8) *
                                                                    (8 * (LAYOUT == Q8_TILES_F16S2 ? 32768 : 16384) +
                                                                     (LAYOUT == Q8_TILES_F16SD ? 8192 : 0)));
    const unsigned grid = (unsigned)(mpad / 8);
    const int rc = vec ? launch_pdl(row_scale_kernel<T, true>, grid, st, (const T*)x, inv_scale, m, mpad, k, stride)
                       : launch_pdl(row_scale_kernel<T, false>, grid, st, (const T*)x, inv_scale, m, mpad, k, stride);
    if (rc != GSQ_OK) return rc;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(k >> 5), (unsigned)((m + 255) / 256 * 4));   // whole blocks of 256 tokens
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (vec) {
    GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_1_tiles_kernel<T, true, LAYOUT>, (const T*)x, (uint8_t*)out, m, k, stride));
  } else {
    GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_1_tiles_kernel<T, false, LAYOUT>, (const T*)x, (uint8_t*)out, m, k, stride));
  }
  return GSQ_OK;
}

// x [m, k] -> activation tiles for the prefill GEMM (see quantize_q8_1_tiles_kernel); k % 256 == 0.
int quantize_tiles_host(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride, int layout, void* out, void* stream) {
  if (m < 0 || k <= 0 || k % 256 != 0 || (m > 0 && (!x || !out)) || (m + 255) / 256 * 4 > 65535) return GSQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
#define GSQ_TILES_CASE(T)                                                                                  \
  return layout == Q8_TILES_H16      ? launch_q8_1_tiles<T, Q8_TILES_H16>(x, m, k, stride, out, st)     \
         : layout == Q8_TILES_F16S   ? launch_q8_1_tiles<T, Q8_TILES_F16S>(x, m, k, stride, out, st)    \
         : layout == Q8_TILES_F16S2  ? launch_q8_1_tiles<T, Q8_TILES_F16S2>(x, m, k, stride, out, st)   \
         : layout == Q8_TILES_F16SD  ? launch_q8_1_tiles<T, Q8_TILES_F16SD>(x, m, k, stride, out, st)   \
         : layout == GSQ_Q8_LAYOUT_D4 ? launch_q8_1_tiles<T, GSQ_Q8_LAYOUT_D4>(x, m, k, stride, out, st) \
                                      : launch_q8_1_tiles<T, GSQ_Q8_LAYOUT_DS4>(x, m, k, stride, out, st)
  switch (x_dtype) {
    case GSQ_F32: GSQ_TILES_CASE(float);
    case GSQ_F16: GSQ_TILES_CASE(__half);
    case GSQ_BF16: GSQ_TILES_CASE(__nv_bfloat16);
    default: return GSQ_ERR_UNSUPPORTED;
  }
#undef GSQ_TILES_CASE
}

}  // namespace gsq

extern "C" int gsq_quantize_q8_1(const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* out,
                                 void* stream) {
  if (m < 0 || k <= 0 || k % 32 != 0 || (m > 0 && (!x || !out))) return GSQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case GSQ_F32: return gsq::launch_q8_1<float>(x, m, k, x_row_stride, out, st);
    case GSQ_F16: return gsq::launch_q8_1<__half>(x, m, k, x_row_stride, out, st);
    case GSQ_BF16: return gsq::launch_q8_1<__nv_bfloat16>(x, m, k, x_row_stride, out, st);
    default: return GSQ_ERR_UNSUPPORTED;
  }
}

extern "C" int gsq_quantize_q8_1_mmq(const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride,
                                     int layout, void* out, void* stream) {
  if (m < 0 || k <= 0 || k % 128 != 0 || (m > 0 && (!x || !out))) return GSQ_ERR_UNSUPPORTED;
  if (layout != GSQ_Q8_LAYOUT_D4 && layout != GSQ_Q8_LAYOUT_DS4) return GSQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
#define GSQ_MMQ_CASE(T)                                                                                   \
  return layout == GSQ_Q8_LAYOUT_D4 ? gsq::launch_q8_1_mmq<T, GSQ_Q8_LAYOUT_D4>(x, m, k, x_row_stride, out, st) \
                                    : gsq::launch_q8_1_mmq<T, GSQ_Q8_LAYOUT_DS4>(x, m, k, x_row_stride, out, st)
  switch (x_dtype) {
    case GSQ_F32: GSQ_MMQ_CASE(float);
    case GSQ_F16: GSQ_MMQ_CASE(__half);
    case GSQ_BF16: GSQ_MMQ_CASE(__nv_bfloat16);
    default: return GSQ_ERR_UNSUPPORTED;
  }
#undef GSQ_MMQ_CASE
}

namespace gsq {

template <typename T>
static int launch_rmsnorm_q8_1(const void* x, int64_t m, int64_t k, int64_t stride, void* residual, const void* gamma, float eps,
                               void* out, void* y_out, cudaStream_t st) {
  static bool configured[64];
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GSQ_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(rmsnorm_q8_1_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)m);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = (size_t)k * 4;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rmsnorm_q8_1_kernel<T>, (const T*)x, stride, (T*)residual, (const T*)gamma, eps,
                                  (uint8_t*)out, (T*)y_out, k));
  return GSQ_OK;
}

}  // namespace gsq

extern "C" int gsq_rmsnorm_quantize_q8_1(const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride,
                                         void* residual, const void* gamma, float eps, void* out_q8, void* y_out,
                                         void* stream) {
  if (m == 0) return GSQ_OK;
  if (m < 0 || m > 65535 || k <= 0 || k % 32 != 0 || k > 40960 || !x || !gamma || !out_q8) return GSQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case GSQ_F32: return gsq::launch_rmsnorm_q8_1<float>(x, m, k, x_row_stride, residual, gamma, eps, out_q8, y_out, st);
    case GSQ_F16: return gsq::launch_rmsnorm_q8_1<__half>(x, m, k, x_row_stride, residual, gamma, eps, out_q8, y_out, st);
    case GSQ_BF16: return gsq::launch_rmsnorm_q8_1<__nv_bfloat16>(x, m, k, x_row_stride, residual, gamma, eps, out_q8, y_out, st);
    default: return GSQ_ERR_UNSUPPORTED;
  }
}

extern "C" int gsq_silu_mul_quantize_q8_1(const void* gate_up, int x_dtype, int64_t m, int64_t inter, int64_t row_stride,
                                          void* out_q8, void* y_out, void* stream) {
  if (m == 0) return GSQ_OK;
  if (m < 0 || inter <= 0 || inter % 32 != 0 || !gate_up || !out_q8) return GSQ_ERR_UNSUPPORTED;
  const int64_t threads = m * (inter >> 3);
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case GSQ_F32:
      return gsq::launch_pdl(gsq::silu_mul_q8_1_kernel<float>, grid, st, (const float*)gate_up, row_stride, (uint8_t*)out_q8,
                             (float*)y_out, m, inter);
    case GSQ_F16:
      return gsq::launch_pdl(gsq::silu_mul_q8_1_kernel<__half>, grid, st, (const __half*)gate_up, row_stride, (uint8_t*)out_q8,
                             (__half*)y_out, m, inter);
    case GSQ_BF16:
      return gsq::launch_pdl(gsq::silu_mul_q8_1_kernel<__nv_bfloat16>, grid, st, (const __nv_bfloat16*)gate_up, row_stride,
                             (uint8_t*)out_q8, (__nv_bfloat16*)y_out, m, inter);
    default: return GSQ_ERR_UNSUPPORTED;
  }
}
