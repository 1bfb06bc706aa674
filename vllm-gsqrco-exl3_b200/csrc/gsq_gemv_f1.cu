// dp4a product for the low-bit GGUF types a model file mixes with the four main ones: Q2_K, IQ2_XXS, IQ2_XS, IQ2_S,
// IQ3_XXS, IQ1_M, read in GGUF order (no repack), 1..8 activation rows per launch (sm_100a).
//
// Replaces, for these types, the reference's route through the stock MMVQ kernel (lcpp_mul_mat_vec_q:
// plugin/vllm_gguf_plugin/csrc/lcpp_shim.cu:573-624 -> csrc/lcpp/ggml/src/ggml-cuda/mmvq.cu) with the per-type dot
// products of ggml-cuda/vecdotq.cuh: 367-393 + 868-889 (Q2_K), 1048-1078 (IQ2_XXS), 1083-1119 (IQ2_XS), 1124-1167
// (IQ2_S), 1172-1206 (IQ3_XXS), 1286-1329 (IQ1_M). The arithmetic per 32-value block is the reference's: an exact
// integer dot product of the signed codebook bytes with the q8_1 quants, the integer sub-scale applied with the same
// truncating divisions, then one fp32 product with d_w * d_x.
//
// Work split: a warp owns 4 weight rows (2 at one or two activation rows); per step its 32 lanes cover 4 superblocks x 8 slices of 32 values, each lane
// decoding its slice of the 4 rows once and dotting it with every activation row (the 36-byte q8_1 blocks come through
// L1: every warp of the SM reads the same ones). Blocks of these types are only 2-byte aligned (66, 74, 82, 98 bytes),
// so weights come in as halfwords. Codebooks are device tables read through the cache hierarchy.
#include "gsq_common.cuh"
#include "gsq_tables_f1.h"

namespace gsq {

enum { F1_Q2K = 0, F1_IQ2XXS = 1, F1_IQ2XS = 2, F1_IQ2S = 3, F1_IQ3XXS = 4, F1_IQ1M = 5 };

__device__ const uint64_t g_iq2xxs_grid[256] = GSQ_IQ2XXS_GRID_INIT;
__device__ const uint64_t g_iq2xs_grid[512] = GSQ_IQ2XS_GRID_INIT;
__device__ const uint64_t g_iq2s_grid[1024] = GSQ_IQ2S_GRID_INIT;
__device__ const uint32_t g_iq3xxs_grid[256] = GSQ_IQ3XXS_GRID_INIT;
__device__ const uint32_t g_iq1_grid[2048] = GSQ_IQ1_GRID_INIT;
__device__ const uint8_t g_ksigns[128] = GSQ_KSIGNS_INIT;

struct F1Args {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;
  int k;
  const uint8_t* xq8;   // [m][k / 32] blocks of 36 bytes
  void* y;
  int y_dtype;
  int64_t ldy;
  int* dump;            // debug: integer group sums [m0 + m][nrows][k / g]
  int dump_m0;
};

__host__ __device__ constexpr int f1_block_bytes(int kind) {
  return kind == F1_Q2K ? 84 : kind == F1_IQ2XXS ? 66 : kind == F1_IQ2XS ? 74 : kind == F1_IQ2S ? 82 : kind == F1_IQ3XXS ? 98 : 56;
}
// values per integer sub-scale (what the debug dump is grouped by)
__host__ __device__ constexpr int f1_group(int kind) { return (kind == F1_IQ2XXS || kind == F1_IQ3XXS) ? 32 : 16; }

__device__ __forceinline__ uint32_t ld32_h(const uint8_t* p) {   // 32 bits from a 2-byte aligned address
  return ldg_stream_u16(p) | (ldg_stream_u16(p + 2) << 16);
}
// the 4 low bits of `bits` say which bytes of g to negate (no byte of these codebooks is zero, so ~g + 1 per byte
// never carries)
__device__ __forceinline__ int apply_signs4(uint32_t g, uint32_t bits) {
  const uint32_t ones = ((bits & 0xFu) * 0x00204081u) & 0x01010101u;
  return (int)((g ^ (ones * 0xFFu)) + ones);
}
// C integer division by a power of two (truncation toward zero)
__device__ __forceinline__ int tdiv(int a, int sh) { return (a + ((a >> 31) & ((1 << sh) - 1))) >> sh; }

// The raw words of one lane's slice of one row, as loaded (fetch), before any table look-up: fetched one step ahead
// of their use so that the load latency is behind the arithmetic of the step before.
template <int KIND>
struct Raw {
  uint32_t r[KIND == F1_Q2K ? 10 : KIND == F1_IQ2S ? 5 : 4];

  __device__ __forceinline__ void fetch(const uint8_t* b, int s) {
    if (KIND == F1_IQ2XXS) {
      r[0] = ldg_stream_u16(b);
      r[1] = ld32_h(b + 2 + 8 * s);
      r[2] = ld32_h(b + 6 + 8 * s);
    } else if (KIND == F1_IQ2XS) {
      r[0] = ldg_stream_u16(b);
      r[1] = ld32_h(b + 2 + 8 * s);
      r[2] = ld32_h(b + 6 + 8 * s);
      r[3] = ldg_stream_u8(b + 66 + s);
    } else if (KIND == F1_IQ2S) {
      r[0] = ldg_stream_u16(b);
      r[1] = ld32_h(b + 2 + 4 * s);
      r[2] = ld32_h(b + 34 + 4 * s);
      r[3] = ldg_stream_u8(b + 66 + s);
      r[4] = ldg_stream_u8(b + 74 + s);
    } else if (KIND == F1_IQ3XXS) {
      r[0] = ldg_stream_u16(b);
      r[1] = ld32_h(b + 2 + 8 * s);
      r[2] = ld32_h(b + 6 + 8 * s);
      r[3] = ld32_h(b + 66 + 4 * s);
    } else if (KIND == F1_Q2K) {
      const int h = s >> 2;
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = ldg_stream_u32(b + 16 + 32 * h + 4 * e);
      r[8] = ldg_stream_u16(b + 2 * s);
      r[9] = ldg_stream_u32(b + 80);
    } else {  // IQ1_M
      r[0] = ldg_stream_u32(b + 4 * s);
      r[1] = ldg_stream_u16(b + 32 + 2 * s);
      const uint2 sa = ldg_stream_v2(b + 48);
      r[2] = sa.x;
      r[3] = sa.y;
    }
  }
};

// One lane's slice of one row: the 8 int8x4 words of its 32 values and what scales them.
template <int KIND>
struct Slice {
  int wv[8];
  int p0, p1, p2, p3;   // per kind: sub-scales (and mins)
  float d, dmin;

  __device__ __forceinline__ void decode(const Raw<KIND>& w, int s) {
    if (KIND == F1_IQ2XXS) {
      d = h2f(w.r[0]);
      const uint32_t q = w.r[1], aux = w.r[2];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint64_t gv = g_iq2xxs_grid[(q >> (8 * g)) & 0xFFu];
        const uint32_t sg = g_ksigns[(aux >> (7 * g)) & 0x7Fu];
        wv[2 * g] = apply_signs4((uint32_t)gv, sg);
        wv[2 * g + 1] = apply_signs4((uint32_t)(gv >> 32), sg >> 4);
      }
      p0 = (int)(aux >> 28);
    } else if (KIND == F1_IQ2XS) {
      d = h2f(w.r[0]);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t q = (w.r[1 + (g >> 1)] >> (16 * (g & 1))) & 0xFFFFu;
        const uint64_t gv = g_iq2xs_grid[q & 511u];
        const uint32_t sg = g_ksigns[q >> 9];
        wv[2 * g] = apply_signs4((uint32_t)gv, sg);
        wv[2 * g + 1] = apply_signs4((uint32_t)(gv >> 32), sg >> 4);
      }
      p0 = (int)(w.r[3] & 0xFu);
      p1 = (int)(w.r[3] >> 4);
    } else if (KIND == F1_IQ2S) {
      d = h2f(w.r[0]);
      const uint32_t qs = w.r[1], sgs = w.r[2], qh = w.r[3];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint64_t gv = g_iq2s_grid[((qs >> (8 * g)) & 0xFFu) | (((qh >> (2 * g)) & 3u) << 8)];
        const uint32_t sg = (sgs >> (8 * g)) & 0xFFu;
        wv[2 * g] = apply_signs4((uint32_t)gv, sg);
        wv[2 * g + 1] = apply_signs4((uint32_t)(gv >> 32), sg >> 4);
      }
      p0 = (int)(w.r[4] & 0xFu);
      p1 = (int)(w.r[4] >> 4);
    } else if (KIND == F1_IQ3XXS) {
      d = h2f(w.r[0]);
      const uint32_t qa = w.r[1], qb = w.r[2], aux = w.r[3];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t q = g < 2 ? qa >> (16 * g) : qb >> (16 * (g - 2));
        const uint32_t sg = g_ksigns[(aux >> (7 * g)) & 0x7Fu];
        wv[2 * g] = apply_signs4(g_iq3xxs_grid[q & 0xFFu], sg);
        wv[2 * g + 1] = apply_signs4(g_iq3xxs_grid[(q >> 8) & 0xFFu], sg >> 4);
      }
      p0 = (int)(aux >> 28);
    } else if (KIND == F1_Q2K) {
      // slice s = 4 h + j: bits 2j, 2j + 1 of the 32 bytes qs[32 h ..]
      const int j = s & 3;
#pragma unroll
      for (int e = 0; e < 8; ++e) wv[e] = (int)((w.r[e] >> (2 * j)) & 0x03030303u);
      const uint32_t sc = w.r[8];
      p0 = (int)(sc & 0xFu);
      p1 = (int)((sc >> 8) & 0xFu);
      p2 = (int)((sc >> 4) & 0xFu);
      p3 = (int)(sc >> 12);
      d = h2f(w.r[9]);
      dmin = h2f(w.r[9] >> 16);
    } else {  // IQ1_M
      const uint32_t qs = w.r[0], qh = w.r[1];
      const uint2 sa = make_uint2(w.r[2], w.r[3]);
      const uint32_t dbits = ((sa.x >> 12) & 0x000Fu) | ((sa.x >> 24) & 0x00F0u) | ((sa.y >> 4) & 0x0F00u) | ((sa.y >> 16) & 0xF000u);
      d = h2f(dbits);
      p2 = 0;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t nib = (qh >> (4 * g)) & 0xFu;
        const uint32_t gv = g_iq1_grid[((qs >> (8 * g)) & 0xFFu) | ((nib & 7u) << 8)];
        wv[2 * g] = (int)(gv & 0x0F0F0F0Fu);          // codebook value + 1
        wv[2 * g + 1] = (int)((gv >> 4) & 0x0F0F0F0Fu);
        p2 |= (int)((nib >> 3) << g);                 // bit g: delta of group g is negative
      }
      // 3-bit sub-scales of the 16-value groups 2s, 2s + 1: scale word s / 2, bits 6 (s % 2) and 3 above
      const uint32_t w16 = ((s >> 1) & 2 ? sa.y : sa.x) >> (16 * ((s >> 1) & 1));
      const uint32_t tmp = (w16 & 0xFFFFu) >> (6 * (s & 1));
      p0 = 2 * (int)(tmp & 7u) + 1;
      p1 = 2 * (int)((tmp >> 3) & 7u) + 1;
    }
  }

  // dot with one q8_1 block (u: its 8 quant words, d8: its scale); `grp` receives the integer group sums
  template <bool DUMP>
  __device__ __forceinline__ float dot(const int (&u)[8], float d8, int (&grp)[2]) const {
    if (KIND == F1_IQ2XXS || KIND == F1_IQ3XXS) {
      int sumi = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) sumi = dp4a(wv[e], u[e], sumi);
      if (DUMP) grp[0] = sumi;
      const int v = KIND == F1_IQ2XXS ? (sumi * (2 * p0 + 1)) / 8 : tdiv(p0 * sumi + tdiv(sumi, 1), 1);
      return (d * d8) * (float)v;
    } else if (KIND == F1_IQ2XS || KIND == F1_IQ2S) {
      int s0 = 0, s1 = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s0 = dp4a(wv[e], u[e], s0);
        s1 = dp4a(wv[4 + e], u[4 + e], s1);
      }
      if (DUMP) { grp[0] = s0; grp[1] = s1; }
      const int v = tdiv(s0 * p0 + s1 * p1 + tdiv(s0 + s1, 1), 2);
      return (d * d8) * (float)v;
    } else if (KIND == F1_Q2K) {
      int s0 = 0, s1 = 0, q0 = 0, q1 = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s0 = dp4a(wv[e], u[e], s0);
        s1 = dp4a(wv[4 + e], u[4 + e], s1);
        q0 = dp4a(0x01010101, u[e], q0);
        q1 = dp4a(0x01010101, u[4 + e], q1);
      }
      if (DUMP) { grp[0] = s0; grp[1] = s1; }
      return d8 * (d * (float)(s0 * p0 + s1 * p1) - dmin * (float)(q0 * p2 + q1 * p3));
    } else {  // IQ1_M: sum of (8 g +- 1) * q over each 16-value group
      int s16[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        int acc = 0;
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
          const int g = 2 * h + gg;
          const int i1 = dp4a(wv[2 * g + 1], u[2 * g + 1], dp4a(wv[2 * g], u[2 * g], 0));
          const int y1 = dp4a(0x01010101, u[2 * g + 1], dp4a(0x01010101, u[2 * g], 0));
          acc += 8 * (i1 - y1) + (((p2 >> g) & 1) ? -y1 : y1);
        }
        s16[h] = acc;
      }
      if (DUMP) { grp[0] = s16[0]; grp[1] = s16[1]; }
      return (d * d8) * ((float)(s16[0] * p0 + s16[1] * p1) * 0.125f);
    }
  }
};

constexpr int F1_WARPS = 4;

// weight rows per warp: 4 amortise the activation loads; at 1 and 2 activation rows there is little to amortise and
// twice the warps hide more of the load latency
__host__ __device__ constexpr int f1_rows(int m) { return m <= 2 ? 2 : 4; }

template <int KIND, int M, bool DUMP>
__global__ void __launch_bounds__(F1_WARPS * 32) gemv_f1_kernel(const F1Args a) {
  constexpr int BS = f1_block_bytes(KIND), G = f1_group(KIND), R = f1_rows(M);
  const int lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * F1_WARPS + (threadIdx.x >> 5)) * R;
  if (row0 >= a.nrows) return;
  const int nsb = a.k >> 8, nb32 = a.k >> 5;
  const int sbl = lane >> 3, s = lane & 7;
  float acc[R][M];
#pragma unroll
  for (int i = 0; i < R; ++i) {
#pragma unroll
    for (int m = 0; m < M; ++m) acc[i][m] = 0.0f;
  }
  // raw words of the next step are fetched while this step's are decoded and multiplied
  Raw<KIND> nxt[R];
  auto fetch_step = [&](int sb) {
    if (sb < nsb) {
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int r = min(row0 + i, a.nrows - 1);
        nxt[i].fetch(a.w + (int64_t)r * a.row_bytes + (int64_t)sb * BS, s);
      }
    }
  };
  fetch_step(sbl);
  for (int sb0 = 0; sb0 < nsb; sb0 += 4) {
    const int sb = sb0 + sbl;
    Raw<KIND> cur[R];
#pragma unroll
    for (int i = 0; i < R; ++i) cur[i] = nxt[i];
    fetch_step(sb + 4);
    if (sb < nsb) {
      const int blk = sb * 8 + s;
      // row by row: decode the lane's slice, dot it with every activation block (the blocks of the step stay in L1;
      // holding all rows' decoded slices to load each block once measured slower: registers)
#pragma unroll
      for (int i = 0; i < R; ++i) {
        Slice<KIND> sl;
        sl.decode(cur[i], s);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint32_t* xb = reinterpret_cast<const uint32_t*>(a.xq8 + ((int64_t)m * nb32 + blk) * 36);
          int u[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) u[e] = (int)__ldg(xb + 1 + e);
          const float d8 = h2f(__ldg(xb));
          int grp[2] = {0, 0};
          acc[i][m] += sl.template dot<DUMP>(u, d8, grp);
          if (DUMP && row0 + i < a.nrows) {
            int* o = a.dump + ((int64_t)(a.dump_m0 + m) * a.nrows + row0 + i) * (a.k / G);
            if (G == 32) {
              o[blk] = grp[0];
            } else {
              o[2 * blk] = grp[0];
              o[2 * blk + 1] = grp[1];
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[i][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
      if (lane == 0 && row0 + i < a.nrows) store_out_dyn(a.y, a.y_dtype, (int64_t)m * a.ldy + row0 + i, v);
    }
  }
}

template <int KIND, bool DUMP>
static int launch_f1(const F1Args& a, int m, cudaStream_t st) {
  const int per_block = f1_rows(m) * F1_WARPS;
  const unsigned grid = (unsigned)((a.nrows + per_block - 1) / per_block);
  switch (m) {
#define GSQ_F1_CASE(MM) \
  case MM: gemv_f1_kernel<KIND, MM, DUMP><<<grid, F1_WARPS * 32, 0, st>>>(a); break;
    GSQ_F1_CASE(1) GSQ_F1_CASE(2) GSQ_F1_CASE(3) GSQ_F1_CASE(4) GSQ_F1_CASE(5) GSQ_F1_CASE(6) GSQ_F1_CASE(7) GSQ_F1_CASE(8)
#undef GSQ_F1_CASE
    default: return GSQ_ERR_UNSUPPORTED;
  }
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}

static int f1_kind(int ggml_type) {
  switch (ggml_type) {
    case GSQ_TYPE_Q2_K: return F1_Q2K;
    case GSQ_TYPE_IQ2_XXS: return F1_IQ2XXS;
    case GSQ_TYPE_IQ2_XS: return F1_IQ2XS;
    case GSQ_TYPE_IQ2_S: return F1_IQ2S;
    case GSQ_TYPE_IQ3_XXS: return F1_IQ3XXS;
    case GSQ_TYPE_IQ1_M: return F1_IQ1M;
    default: return -1;
  }
}

bool gemv_f1_applies(int ggml_type) { return f1_kind(ggml_type) >= 0; }

// values per dumped integer sum of this type (32 or 16)
int gemv_f1_group(int ggml_type) {
  const int kind = f1_kind(ggml_type);
  return kind < 0 ? 0 : f1_group(kind);
}

// 1..8 activation rows (block_q8_1) against W in GGUF order
int gemv_f1_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, const void* x_q8, int64_t m, int64_t k,
                 void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump, int dump_m0) {
  if (m == 0 || rows == 0) return GSQ_OK;
  const int kind = f1_kind(ggml_type);
  if (kind < 0 || m < 0 || m > 8 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !x_q8 || !y) return GSQ_ERR_UNSUPPORTED;
  if (rows > INT32_MAX || k > INT32_MAX) return GSQ_ERR_TOO_LARGE;
  if (row_bytes != (k / 256) * f1_block_bytes(kind)) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  F1Args a;
  a.w = (const uint8_t*)w;
  a.row_bytes = row_bytes;
  a.nrows = (int)rows;
  a.k = (int)k;
  a.xq8 = (const uint8_t*)x_q8;
  a.y = y;
  a.y_dtype = y_dtype;
  a.ldy = y_row_stride;
  a.dump = dump;
  a.dump_m0 = dump_m0;
  cudaStream_t st = (cudaStream_t)stream;
#define GSQ_F1_KIND(K) return dump ? launch_f1<K, true>(a, (int)m, st) : launch_f1<K, false>(a, (int)m, st)
  switch (kind) {
    case F1_Q2K: GSQ_F1_KIND(F1_Q2K);
    case F1_IQ2XXS: GSQ_F1_KIND(F1_IQ2XXS);
    case F1_IQ2XS: GSQ_F1_KIND(F1_IQ2XS);
    case F1_IQ2S: GSQ_F1_KIND(F1_IQ2S);
    case F1_IQ3XXS: GSQ_F1_KIND(F1_IQ3XXS);
    default: GSQ_F1_KIND(F1_IQ1M);
  }
#undef GSQ_F1_KIND
}

}  // namespace gsq
