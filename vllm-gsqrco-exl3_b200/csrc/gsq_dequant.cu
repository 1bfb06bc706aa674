// Row gather + dequantisation of GGUF weights (sm_100a): the quantised embedding look-up.
//
// Replaces, for the ten types of the model file, the reference's torch.index_select + _C_gguf::ggml_dequantize pair
// (plugin/vllm_gguf_plugin/quantization/vocal_embeds.py:79-98; the op: csrc/gguf/gguf_kernel.cu:87-103 over the stock
// dequantize kernels of csrc/gguf/dequantize.cuh) with one kernel that reads the selected rows' blocks and writes
// their values in the requested type: no gathered copy of the quantised rows.
//
// Arithmetic: the fp32 operation order of llama.cpp's C dequantiser / gguf-py, which the reference pins bit for bit on
// 84 real rows (tests/cpu/test_dequant_fixtures.py:54-64) -- d * sub-scale rounded to fp32, then times the integer
// value (and, for Q4_K / Q2_K, minus the separately rounded dmin * m): results equal those fixtures bit for bit in
// fp32; fp16 / bf16 outputs are that value rounded once. (The stock CUDA kernels do part of this in half precision
// for the K-quants, so they differ from the fixtures in the last places; this kernel does not.)
// Multiplications and the subtraction are written with the non-contracting intrinsics: a fused multiply-add would
// round differently.
//
// One CTA per output row, 8 threads per superblock (one 32-value slice each).
#include "gsq_common.cuh"
#include "gsq_f1_codec.cuh"
#include "gsq_tables.h"

namespace gsq {

enum { DQ_Q4K = 10, DQ_Q6K = 11, DQ_IQ3S = 12, DQ_IQ4XS = 13 };   // beside the F1_* kinds of gsq_f1_codec.cuh

static __device__ const uint32_t g_dq_iq3s_grid[512] = GSQ_IQ3S_GRID_INIT;
static __constant__ int8_t c_dq_iq4nl[16] = GSQ_IQ4NL_VALUES_INIT;

__host__ __device__ constexpr int dq_block_bytes(int kind) {
  return kind == DQ_Q4K ? 144 : kind == DQ_Q6K ? 210 : kind == DQ_IQ3S ? 110 : kind == DQ_IQ4XS ? 136 : f1_block_bytes(kind);
}

__device__ __forceinline__ uint32_t ldb(const uint8_t* p) { return __ldg(p); }

// the 32 values of slice s of the superblock at b
template <int KIND>
__device__ __forceinline__ void dequant_slice(const uint8_t* b, int s, float (&o)[32]) {
  if constexpr (KIND == DQ_IQ3S) {
    const float d = h2f(ldb(b) | (ldb(b + 1) << 8));
    const uint32_t qh = ldb(b + 66 + s);
    const uint32_t ls = (ldb(b + 106 + (s >> 1)) >> (4 * (s & 1))) & 0xFu;
    const float db = __fmul_rn(d, (float)(1 + 2 * (int)ls));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t gv = g_dq_iq3s_grid[ldb(b + 2 + 8 * s + j) | (((qh >> j) & 1u) << 8)];
      const uint32_t sg = ldb(b + 74 + 4 * s + (j >> 1)) >> (4 * (j & 1));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mag = (float)((gv >> (8 * e)) & 0xFFu);
        o[4 * j + e] = __fmul_rn(db, ((sg >> e) & 1u) ? -mag : mag);
      }
    }
  } else if constexpr (KIND == DQ_IQ4XS) {
    const float d = h2f(ldb(b) | (ldb(b + 1) << 8));
    const uint32_t sh = ldb(b + 2) | (ldb(b + 3) << 8);
    const uint32_t lsb = ((ldb(b + 4 + (s >> 1)) >> (4 * (s & 1))) & 0xFu) | (((sh >> (2 * s)) & 3u) << 4);
    const float dl = __fmul_rn(d, (float)((int)lsb - 32));
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t q = ldb(b + 8 + 16 * s + i);
      o[i] = __fmul_rn(dl, (float)c_dq_iq4nl[q & 0xFu]);
      o[16 + i] = __fmul_rn(dl, (float)c_dq_iq4nl[q >> 4]);
    }
  } else if constexpr (KIND == DQ_Q4K) {
    const float d = h2f(ldb(b) | (ldb(b + 1) << 8)), dmin = h2f(ldb(b + 2) | (ldb(b + 3) << 8));
    uint32_t sc, mn;   // six-bit scale and min of sub-block s (12 packed bytes at b + 4)
    if (s < 4) {
      sc = ldb(b + 4 + s) & 63u;
      mn = ldb(b + 8 + s) & 63u;
    } else {
      sc = (ldb(b + 8 + s) & 0xFu) | ((ldb(b + s) >> 6) << 4);
      mn = (ldb(b + 8 + s) >> 4) | ((ldb(b + 4 + s) >> 6) << 4);
    }
    const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)mn);
    const int j = s >> 1, hi = s & 1;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint32_t q = ldb(b + 16 + 32 * j + i);
      o[i] = __fsub_rn(__fmul_rn(dl, (float)(hi ? q >> 4 : q & 0xFu)), ml);
    }
  } else if constexpr (KIND == DQ_Q6K) {
    const float d = h2f(ldb(b + 208) | (ldb(b + 209) << 8));
    const int n = s >> 2, qt = s & 3;      // 128-value half, quarter of it
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      const uint32_t lo = ldb(b + 64 * n + 32 * (qt & 1) + l), hb = ldb(b + 128 + 32 * n + l);
      const int q = (int)(((qt & 2) ? lo >> 4 : lo & 0xFu) | (((hb >> (2 * qt)) & 3u) << 4)) - 32;
      const int scv = (int)(int8_t)ldb(b + 192 + 8 * n + 2 * qt + (l >> 4));
      o[l] = __fmul_rn(__fmul_rn(d, (float)scv), (float)q);
    }
  } else {
    // the low-bit types: raw words and integer decode shared with the dp4a kernel
    Raw<KIND> raw;
    raw.fetch(b, s);
    Slice<KIND> sl;
    sl.decode(raw, s);
    float w[32];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
#pragma unroll
      for (int c = 0; c < 4; ++c) w[4 * e + c] = (float)(int)(int8_t)((uint32_t)sl.wv[e] >> (8 * c));
    }
    if constexpr (KIND == F1_IQ2XXS || KIND == F1_IQ3XXS) {
      const float db = __fmul_rn(__fmul_rn(sl.d, 0.5f + (float)sl.p0), KIND == F1_IQ3XXS ? 0.5f : 0.25f);
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = __fmul_rn(db, w[i]);
    } else if constexpr (KIND == F1_IQ2XS || KIND == F1_IQ2S) {
      const float db0 = __fmul_rn(__fmul_rn(sl.d, 0.5f + (float)sl.p0), 0.25f);
      const float db1 = __fmul_rn(__fmul_rn(sl.d, 0.5f + (float)sl.p1), 0.25f);
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = __fmul_rn(i < 16 ? db0 : db1, w[i]);
    } else if constexpr (KIND == F1_Q2K) {
      const float dl0 = __fmul_rn(sl.d, (float)sl.p0), dl1 = __fmul_rn(sl.d, (float)sl.p1);
      const float ml0 = __fmul_rn(sl.dmin, (float)sl.p2), ml1 = __fmul_rn(sl.dmin, (float)sl.p3);
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = __fsub_rn(__fmul_rn(i < 16 ? dl0 : dl1, w[i]), i < 16 ? ml0 : ml1);
    } else {  // IQ1_M: the slice keeps codebook value + 1 (0..2) and the sign of each group's delta; p0, p1 = 2 sc + 1
      const float dl0 = __fmul_rn(sl.d, (float)sl.p0), dl1 = __fmul_rn(sl.d, (float)sl.p1);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float gd = (w[i] - 1.0f) + (((sl.p2 >> (i >> 3)) & 1) ? -0.125f : 0.125f);   // exact
        o[i] = __fmul_rn(i < 16 ? dl0 : dl1, gd);
      }
    }
  }
}

// 32 consecutive values as 16-byte stores (dst 16-byte aligned)
template <typename T>
__device__ __forceinline__ void store32(T* dst, const float (&o)[32]);
template <>
__device__ __forceinline__ void store32<float>(float* dst, const float (&o)[32]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
}
template <>
__device__ __forceinline__ void store32<__half>(__half* dst, const float (&o)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(o[8 * i + 2 * e], o[8 * i + 2 * e + 1]);
    reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(h);
  }
}
template <>
__device__ __forceinline__ void store32<__nv_bfloat16>(__nv_bfloat16* dst, const float (&o)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(o[8 * i + 2 * e], o[8 * i + 2 * e + 1]);
    reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(h);
  }
}

template <int KIND, typename T>
__global__ void __launch_bounds__(256) dequant_rows_kernel(const uint8_t* __restrict__ w, int64_t row_bytes, int64_t w_rows,
                                                          const int64_t* __restrict__ ids, int nsb, T* __restrict__ out,
                                                          int64_t ldo, int* __restrict__ bad_id, bool vec) {
  const int64_t orow = blockIdx.x;
  int64_t src = ids ? ids[orow] : orow;
  if (src < 0 || src >= w_rows) {          // an index outside the table: flagged, the row is written as zeros
    if (threadIdx.x == 0) atomicExch(bad_id, 1);
    src = -1;
  }
  for (int it = threadIdx.x; it < nsb * 8; it += 256) {
    const int sb = it >> 3, s = it & 7;
    float o[32];
    if (src >= 0) {
      dequant_slice<KIND>(w + src * row_bytes + (int64_t)sb * dq_block_bytes(KIND), s, o);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0.0f;
    }
    T* dst = out + orow * ldo + (int64_t)sb * 256 + s * 32;
    if (vec) {
      store32<T>(dst, o);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) store_out<T>(dst + i, o[i]);
    }
  }
}

__device__ int g_dequant_bad_id = 0;

template <int KIND>
static int launch_dequant(const void* w, int64_t row_bytes, int64_t w_rows, const int64_t* ids, int64_t n, int64_t k, void* out,
                          int out_dtype, int64_t ldo, cudaStream_t st) {
  int* bad = nullptr;
  GSQ_CUDA_TRY(cudaGetSymbolAddress((void**)&bad, g_dequant_bad_id));
  const int nsb = (int)(k >> 8);
  const unsigned grid = (unsigned)n;
  const bool vec = (uintptr_t)out % 16 == 0 && (ldo * (out_dtype == GSQ_F32 ? 4 : 2)) % 16 == 0;
  switch (out_dtype) {
    case GSQ_F32:
      dequant_rows_kernel<KIND, float><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, w_rows, ids, nsb, (float*)out, ldo, bad, vec);
      break;
    case GSQ_F16:
      dequant_rows_kernel<KIND, __half><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, w_rows, ids, nsb, (__half*)out, ldo, bad, vec);
      break;
    case GSQ_BF16:
      dequant_rows_kernel<KIND, __nv_bfloat16><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, w_rows, ids, nsb,
                                                                    (__nv_bfloat16*)out, ldo, bad, vec);
      break;
    default: return GSQ_ERR_UNSUPPORTED;
  }
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}

}  // namespace gsq

extern "C" int gsq_dequantize_rows(const void* w, int64_t row_bytes, int64_t w_rows, int ggml_type, const int64_t* ids,
                                   int64_t n, int64_t k, void* out, int out_dtype, int64_t out_row_stride, void* stream) {
  using namespace gsq;
  if (n == 0) return GSQ_OK;
  if (n < 0 || n > INT32_MAX || w_rows <= 0 || k <= 0 || k % 256 != 0 || !w || !out || out_row_stride < k) return GSQ_ERR_UNSUPPORTED;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs) return GSQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
#define GSQ_DQ(K) return launch_dequant<K>(w, row_bytes, w_rows, ids, n, k, out, out_dtype, out_row_stride, st)
  switch (ggml_type) {
    case GSQ_TYPE_Q4_K: GSQ_DQ(DQ_Q4K);
    case GSQ_TYPE_Q6_K: GSQ_DQ(DQ_Q6K);
    case GSQ_TYPE_IQ3_S: GSQ_DQ(DQ_IQ3S);
    case GSQ_TYPE_IQ4_XS: GSQ_DQ(DQ_IQ4XS);
    case GSQ_TYPE_Q2_K: GSQ_DQ(F1_Q2K);
    case GSQ_TYPE_IQ2_XXS: GSQ_DQ(F1_IQ2XXS);
    case GSQ_TYPE_IQ2_XS: GSQ_DQ(F1_IQ2XS);
    case GSQ_TYPE_IQ2_S: GSQ_DQ(F1_IQ2S);
    case GSQ_TYPE_IQ3_XXS: GSQ_DQ(F1_IQ3XXS);
    case GSQ_TYPE_IQ1_M: GSQ_DQ(F1_IQ1M);
    default: return GSQ_ERR_UNSUPPORTED;
  }
#undef GSQ_DQ
}

extern "C" int gsq_dequantize_bad_index_flag(int* flag) {
  if (!flag) return GSQ_ERR_UNSUPPORTED;
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(flag, gsq::g_dequant_bad_id, sizeof(int)));
  return GSQ_OK;
}
