// Codec pieces of the low-bit GGUF types (Q2_K, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ1_M) shared by the dp4a product
// (gsq_gemv_f1.cu) and the row dequantiser (gsq_dequant.cu): codebooks, block geometry, the raw words of a 32-value
// slice and the sign helper. Block structs: csrc/lcpp/ggml/src/ggml-common.h:300-309, 380-411, 430-444 of the reference.
#pragma once
#include "gsq_common.cuh"
#include "gsq_tables_f1.h"

namespace gsq {

enum { F1_Q2K = 0, F1_IQ2XXS = 1, F1_IQ2XS = 2, F1_IQ2S = 3, F1_IQ3XXS = 4, F1_IQ1M = 5 };

static __device__ const uint64_t g_iq2xxs_grid[256] = GSQ_IQ2XXS_GRID_INIT;
static __device__ const uint64_t g_iq2xs_grid[512] = GSQ_IQ2XS_GRID_INIT;
static __device__ const uint64_t g_iq2s_grid[1024] = GSQ_IQ2S_GRID_INIT;
static __device__ const uint32_t g_iq3xxs_grid[256] = GSQ_IQ3XXS_GRID_INIT;
static __device__ const uint32_t g_iq1_grid[2048] = GSQ_IQ1_GRID_INIT;
static __device__ const uint8_t g_ksigns[128] = GSQ_KSIGNS_INIT;

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

}  // namespace gsq
