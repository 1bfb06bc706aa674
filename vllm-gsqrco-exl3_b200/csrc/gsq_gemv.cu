// Streaming dp4a GEMV for 1..8 activation rows over GGUF superblocks (sm_100a).
//
// Replaces, behind gsq_mul_mat_vec_q8, the reference's MMVQ (csrc/lcpp/ggml/src/ggml-cuda/mmvq.cu:599-844
// with the vec_dot_*_q8_1 functions of vecdotq.cuh) and its owned 1..8-row kernels
// (lcpp_shim.cu:498-572, lcpp_owned_k4.cu:116-234, lcpp_owned_iq3_mma.cu:483-600). The per-slice integer
// sums and the slice terms d_w * d_q8 * scale * sumi are the reference's; only the fp32 order in which
// a row's slice terms are added differs (fixed, so results are run-to-run and graph-replay identical).
//
// Shape of the kernel (one persistent CTA of 16 warps per SM):
//   * the q8_1 activations of all rows are staged once per CTA into shared memory as planes
//     (int8 values, fp32 scales, and for Q4_K the fp32 d * sum(q) of every block);
//   * weights stream straight from HBM into registers with 128-bit no-allocate loads, one
//     "record" ahead of the arithmetic; a record is what one warp consumes per step:
//        IQ3_S packed : one 16-row x 256-column tile record of gsq_iq3s_repack (1760 bytes);
//                       lane = (row group a = lane / 8, slice s = lane % 8), rows a, a+4, a+8, a+12
//        Q4_K, IQ4_XS, IQ3_S in GGUF order : 4 rows x 4 superblocks; lane = (superblock, 32-value chunk)
//        Q6_K         : 4 rows x 1 superblock; lane = 4-byte word of ql
//     so every lane decodes its 32 values of 4 weight rows once and dots them with each activation row;
//   * IQ3_S reads its 512-entry codebook from a copy replicated per lane (entry i of lane l at word
//     32 i + l), so the data-dependent lookups never collide on a shared-memory bank;
//   * a CTA step covers `tiles` row tiles x `parts` column parts (tiles * parts = 16 warps); partial
//     sums meet in shared memory and are added in part order.
#include "gsq_common.cuh"
#include "gsq_tables.h"

namespace gsq {

enum { KIND_IQ3S_PACKED = 0, KIND_IQ3S_RAW = 1, KIND_Q4K = 2, KIND_IQ4XS = 3, KIND_Q6K = 4 };

constexpr int GEMV_WARPS = 16;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

__device__ const uint32_t g_iq3s_grid[512] = GSQ_IQ3S_GRID_INIT;
__constant__ uint32_t c_iq4nl_words[4] = {0, 0, 0, 0};  // filled at device init from GSQ_IQ4NL_VALUES_INIT

struct GemvArgs {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;
  int k;
  const uint8_t* xq8;
  void* y;
  int y_dtype;
  int64_t ldy;
  int parts;         // column parts per tile (power of two, <= 16)
  int n_units;       // CTA steps in total
  int nrec;          // records per row tile
  int rec_per_part;  // ceil(nrec / parts)
  int* dump;         // debug only: integer slice sums
  int dump_m0;
};

template <int KIND>
struct KindTraits;
template <>
struct KindTraits<KIND_IQ3S_PACKED> { static constexpr int tile_rows = 16, rec_sb = 1, bs = 110; };
template <>
struct KindTraits<KIND_IQ3S_RAW> { static constexpr int tile_rows = 4, rec_sb = 4, bs = 110; };
template <>
struct KindTraits<KIND_Q4K> { static constexpr int tile_rows = 4, rec_sb = 4, bs = 144; };
template <>
struct KindTraits<KIND_IQ4XS> { static constexpr int tile_rows = 4, rec_sb = 4, bs = 136; };
template <>
struct KindTraits<KIND_Q6K> { static constexpr int tile_rows = 4, rec_sb = 1, bs = 210; };

// ---------------------------------------------------------------------------------------------
// Per-kind record: the raw bytes one lane holds for its 32 values of 4 weight rows.

template <int KIND>
struct Rec;

// Packed IQ3_S record (see gsq_repack.cu for the layout): per lane 9 words of 9-bit codebook indices
// (row i, group e at bit 9 * (8 i + e)), 4 words of sign bits (row i; bit 8 p + e = sign of value p of
// group e), 4 sub-scale nibbles, and the 4 fp16 d of the lane's rows.
template <>
struct Rec<KIND_IQ3S_PACKED> {
  uint32_t idx[9];
  uint32_t sg[4];
  uint32_t sc;
  uint2 dd;
  __device__ __forceinline__ void load(const GemvArgs& a, int row0, int rec, int lane, bool ok) {
    if (!ok) return;
    const uint8_t* p = a.w + (int64_t)row0 * a.row_bytes + (int64_t)rec * 1760;
    const uint4 ia = ldg_stream_v4(p + 16 * lane);
    const uint4 ib = ldg_stream_v4(p + 512 + 16 * lane);
    idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
    idx[4] = ib.x; idx[5] = ib.y; idx[6] = ib.z; idx[7] = ib.w;
    idx[8] = ldg_stream_u32(p + 1024 + 4 * lane);
    const uint4 s = ldg_stream_v4(p + 1152 + 16 * lane);
    sg[0] = s.x; sg[1] = s.y; sg[2] = s.z; sg[3] = s.w;
    sc = ldg_stream_u16(p + 1664 + 2 * lane);
    dd = ldg_stream_v2(p + 1728 + 8 * (lane >> 3));
  }
};

// IQ3_S in GGUF order: 110-byte blocks are only 2-byte aligned, so everything comes in as halfwords.
template <>
struct Rec<KIND_IQ3S_RAW> {
  uint32_t qs[4][2];
  uint32_t sg[4];
  uint32_t qh[4];
  uint32_t ls[4];
  uint32_t d[4];
  __device__ __forceinline__ void load(const GemvArgs& a, int row0, int rec, int lane, bool ok) {
    if (!ok) return;
    const int sb = rec * 4 + (lane >> 3), s = lane & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = min(row0 + i, a.nrows - 1);
      const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 110;
      d[i] = ldg_stream_u16(b);
      const uint8_t* q = b + 2 + 8 * s;
      qs[i][0] = ldg_stream_u16(q) | (ldg_stream_u16(q + 2) << 16);
      qs[i][1] = ldg_stream_u16(q + 4) | (ldg_stream_u16(q + 6) << 16);
      qh[i] = ldg_stream_u8(b + 66 + s);
      const uint8_t* g = b + 74 + 4 * s;
      sg[i] = ldg_stream_u16(g) | (ldg_stream_u16(g + 2) << 16);
      ls[i] = (ldg_stream_u8(b + 106 + (s >> 1)) >> (4 * (s & 1))) & 0x0F;
    }
  }
};

// Q4_K: 144-byte blocks, 16-byte aligned: header (d, dmin, 12 scale bytes) and the lane's 16-byte chunk.
template <>
struct Rec<KIND_Q4K> {
  uint4 hdr[4];
  uint4 qs[4];
  __device__ __forceinline__ void load(const GemvArgs& a, int row0, int rec, int lane, bool ok) {
    if (!ok) return;
    const int sb = rec * 4 + (lane >> 3), p = lane & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = min(row0 + i, a.nrows - 1);
      const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 144;
      hdr[i] = ldg_stream_v4(b);
      qs[i] = ldg_stream_v4(b + 16 + 16 * p);
    }
  }
};

// IQ4_XS: 136-byte blocks, 8-byte aligned: 8-byte header and the lane's 16-byte slice as two 8-byte loads.
template <>
struct Rec<KIND_IQ4XS> {
  uint2 hdr[4];
  uint2 qa[4], qb[4];
  __device__ __forceinline__ void load(const GemvArgs& a, int row0, int rec, int lane, bool ok) {
    if (!ok) return;
    const int sb = rec * 4 + (lane >> 3), p = lane & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = min(row0 + i, a.nrows - 1);
      const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 136;
      hdr[i] = ldg_stream_v2(b);
      qa[i] = ldg_stream_v2(b + 8 + 16 * p);
      qb[i] = ldg_stream_v2(b + 16 + 16 * p);
    }
  }
};

// Q6_K: 210-byte blocks, 2-byte aligned; lane = word index of ql (32 words).
template <>
struct Rec<KIND_Q6K> {
  uint32_t ql[4], qh[4], sc[4], d[4];
  __device__ __forceinline__ void load(const GemvArgs& a, int row0, int rec, int lane, bool ok) {
    if (!ok) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = min(row0 + i, a.nrows - 1);
      const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)rec * 210;
      const uint8_t* l = b + 4 * lane;
      ql[i] = ldg_stream_u16(l) | (ldg_stream_u16(l + 2) << 16);
      const uint8_t* h = b + 128 + 32 * (lane >> 4) + 4 * (lane & 7);
      qh[i] = ldg_stream_u16(h) | (ldg_stream_u16(h + 2) << 16);
      const uint8_t* s = b + 192 + 8 * (lane >> 4) + ((lane & 15) >> 2);
      sc[i] = ldg_stream_u8(s) | (ldg_stream_u8(s + 4) << 8);
      d[i] = ldg_stream_u16(b + 208);
    }
  }
};

// ---------------------------------------------------------------------------------------------
// Decode + dot. `Planes` are the staged activations in shared memory.

struct Planes {
  const int8_t* xq;   // [m][k] int8, 16-byte aligned rows
  const float* xd;    // [m][k/32] block scale d
  const float* xs;    // [m][k/32] d * sum(q) of the block (Q4_K only)
  const uint32_t* grid;  // replicated IQ3_S codebook
  int k;
  // debug dump of the raw integer slice sums (gsq_debug_block_sums): out[(m * nrows + row) * (k / g) + group]
  int* dump;
  int dump_row0, dump_rows, dump_m0;
};

template <int M>
__device__ __forceinline__ void dump_add(const Planes& pl, int m, int row_in_tile, int group, int groups, int v) {
  const int row = pl.dump_row0 + row_in_tile;
  if (row < pl.dump_rows) atomicAdd(pl.dump + ((int64_t)(pl.dump_m0 + m) * pl.dump_rows + row) * groups + group, v);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// wv[i][e] = 4 signed int8 of group e (values 4e..4e+3 of the lane's slice) of row i; common dot loop of
// the kinds whose lane owns one whole 32-value slice with a single integer sub-scale.
template <int M, bool DUMP>
__device__ __forceinline__ void dot_slice(const int (&wv)[4][8], const int (&isc)[4], const float (&dw)[4],
                                          const Planes& pl, int blk, int row_base, int row_step, float (&acc)[4][M]) {
  const int nb32 = pl.k >> 5;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const uint4* up = reinterpret_cast<const uint4*>(pl.xq + (int64_t)m * pl.k + (int64_t)blk * 32);
    const uint4 ua = up[0], ub = up[1];
    const int u[8] = {(int)ua.x, (int)ua.y, (int)ua.z, (int)ua.w, (int)ub.x, (int)ub.y, (int)ub.z, (int)ub.w};
    const float d8 = pl.xd[m * nb32 + blk];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int sumi = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) sumi = dp4a(wv[i][e], u[e], sumi);
      if constexpr (DUMP) dump_add<M>(pl, m, row_base + row_step * i, blk, nb32, sumi);
      acc[i][m] = fmaf(dw[i] * d8, (float)(sumi * isc[i]), acc[i][m]);
    }
  }
}

// RS: log2 of the byte stride between codebook entries in the replicated table (7: one copy per lane,
// 5: one copy per 8 lanes, used when the activations leave less shared memory).
template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_IQ3S_PACKED>& r, int rec, int lane, bool ok,
                                           const Planes& pl, float (&acc)[4][M]) {
  (void)ok;
  constexpr uint32_t mask = RS == 7 ? 0xFF80u : 0x3FE0u;
  const uint32_t lane_off = RS == 7 ? (uint32_t)lane << 2 : (uint32_t)(lane & 7) << 2;
  const char* gbase = reinterpret_cast<const char*>(pl.grid);
  int wv[4][8];
  int isc[4];
  float dw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int bit = 9 * (8 * i + e), word = bit >> 5, off = bit & 31;
      uint32_t t;
      if (off + 9 <= 32) {
        t = off >= RS ? r.idx[word] >> (off - RS) : r.idx[word] << (RS - off);
      } else {
        t = __funnelshift_r(r.idx[word], r.idx[word + 1], off - RS);
      }
      const uint32_t g = *reinterpret_cast<const uint32_t*>(gbase + ((t & mask) | lane_off));
      const uint32_t msk = prmt(r.sg[i] << (7 - e), 0u, 0xBA98u);  // 0xFF where the value is negative
      wv[i][e] = (int)((g ^ msk) + (msk & 0x01010101u));
    }
    isc[i] = 1 + 2 * (int)((r.sc >> (4 * i)) & 15u);
    dw[i] = h2f((i < 2 ? r.dd.x : r.dd.y) >> (16 * (i & 1)));
  }
  dot_slice<M, DUMP>(wv, isc, dw, pl, rec * 8 + (lane & 7), lane >> 3, 4, acc);
}

template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_IQ3S_RAW>& r, int rec, int lane, bool ok,
                                           const Planes& pl, float (&acc)[4][M]) {
  if (!ok) return;
  constexpr uint32_t mask = RS == 7 ? 0xFF80u : 0x3FE0u;
  const uint32_t lane_off = RS == 7 ? (uint32_t)lane << 2 : (uint32_t)(lane & 7) << 2;
  const char* gbase = reinterpret_cast<const char*>(pl.grid);
  int wv[4][8];
  int isc[4];
  float dw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t byte = (r.qs[i][e >> 2] >> (8 * (e & 3))) & 0xFFu;
      const uint32_t idx = byte | ((r.qh[i] << (8 - e)) & 0x100u);
      const uint32_t g = *reinterpret_cast<const uint32_t*>(gbase + (((idx << RS) & mask) | lane_off));
      const uint32_t ones = (((r.sg[i] >> (4 * e)) & 0xFu) * 0x00204081u) & 0x01010101u;
      wv[i][e] = (int)((g ^ (ones * 0xFFu)) + ones);
    }
    isc[i] = 1 + 2 * (int)r.ls[i];
    dw[i] = h2f(r.d[i]);
  }
  dot_slice<M, DUMP>(wv, isc, dw, pl, (rec * 4 + (lane >> 3)) * 8 + (lane & 7), 0, 1, acc);
}

// 8 four-bit indices of v -> the table bytes: lo = entries of the 4 low nibbles, hi = of the 4 high nibbles.
__device__ __forceinline__ void iq4_lookup(uint32_t v, uint32_t& lo, uint32_t& hi) {
  const uint32_t t0 = c_iq4nl_words[0], t1 = c_iq4nl_words[1], t2 = c_iq4nl_words[2], t3 = c_iq4nl_words[3];
  const uint32_t s01 = v & 0x7777u, s23 = (v >> 16) & 0x7777u;
  const uint32_t pick01 = 0x3210u | ((v & 0x8888u) >> 1), pick23 = 0x3210u | (((v >> 16) & 0x8888u) >> 1);
  const uint32_t r01 = prmt(prmt(t0, t1, s01), prmt(t2, t3, s01), pick01);  // nibbles 0..3 of v
  const uint32_t r23 = prmt(prmt(t0, t1, s23), prmt(t2, t3, s23), pick23);  // nibbles 4..7 of v
  lo = prmt(r01, r23, 0x6420u);
  hi = prmt(r01, r23, 0x7531u);
}

template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_IQ4XS>& r, int rec, int lane, bool ok, const Planes& pl,
                                           float (&acc)[4][M]) {
  if (!ok) return;
  const int p = lane & 7;
  int wv[4][8];
  int isc[4];
  float dw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t v[4] = {r.qa[i].x, r.qa[i].y, r.qb[i].x, r.qb[i].y};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t lo, hi;
      iq4_lookup(v[e], lo, hi);
      wv[i][e] = (int)lo;
      wv[i][4 + e] = (int)hi;
    }
    const uint32_t ls = ((r.hdr[i].y >> (4 * p)) & 0xFu) | (((r.hdr[i].x >> (16 + 2 * p)) & 3u) << 4);
    isc[i] = (int)ls - 32;
    dw[i] = h2f(r.hdr[i].x);
  }
  dot_slice<M, DUMP>(wv, isc, dw, pl, (rec * 4 + (lane >> 3)) * 8 + p, 0, 1, acc);
}

template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_Q4K>& r, int rec, int lane, bool ok, const Planes& pl,
                                           float (&acc)[4][M]) {
  if (!ok) return;
  const int p = lane & 7, jj = p >> 1, half = p & 1, jm = jj & 1;
  const int nb32 = pl.k >> 5;
  const int blk = (rec * 4 + (lane >> 3)) * 8 + 2 * jj;  // q8 block of the low nibbles; high nibbles: blk + 1
  int lo[4][4], hi[4][4];
  int sc0[4], sc1[4];
  float dd[4], dmn0[4], dmn1[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t q[4] = {r.qs[i].x, r.qs[i].y, r.qs[i].z, r.qs[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      lo[i][e] = (int)(q[e] & 0x0F0F0F0Fu);
      hi[i][e] = (int)((q[e] >> 4) & 0x0F0F0F0Fu);
    }
    const uint32_t s0 = (r.hdr[i].y >> (16 * jm)) & 0xFFFFu;
    const uint32_t s2 = (r.hdr[i].z >> (16 * jm)) & 0xFFFFu;
    const uint32_t s4 = (r.hdr[i].w >> (16 * jm)) & 0xFFFFu;
    const uint32_t a0 = jj < 2 ? (s0 & 0x3F3Fu) : ((s4 & 0x0F0Fu) | ((s0 & 0xC0C0u) >> 2));
    const uint32_t a1 = jj < 2 ? (s2 & 0x3F3Fu) : (((s4 >> 4) & 0x0F0Fu) | ((s2 & 0xC0C0u) >> 2));
    sc0[i] = (int)(a0 & 0xFFu);
    sc1[i] = (int)(a0 >> 8);
    dd[i] = h2f(r.hdr[i].x);
    // the min term of a whole 32-value sub-block is added by the lane holding its first half
    const float dmin = half == 0 ? h2f(r.hdr[i].x >> 16) : 0.0f;
    dmn0[i] = dmin * (float)(a1 & 0xFFu);
    dmn1[i] = dmin * (float)(a1 >> 8);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int8_t* xr = pl.xq + (int64_t)m * pl.k + (int64_t)blk * 32 + 16 * half;
    const uint4 ul = *reinterpret_cast<const uint4*>(xr);
    const uint4 uh = *reinterpret_cast<const uint4*>(xr + 32);
    const int u0[4] = {(int)ul.x, (int)ul.y, (int)ul.z, (int)ul.w};
    const int u1[4] = {(int)uh.x, (int)uh.y, (int)uh.z, (int)uh.w};
    const float d80 = pl.xd[m * nb32 + blk], d81 = pl.xd[m * nb32 + blk + 1];
    const float xs0 = pl.xs[m * nb32 + blk], xs1 = pl.xs[m * nb32 + blk + 1];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int dl = 0, dh = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dl = dp4a(lo[i][e], u0[e], dl);
        dh = dp4a(hi[i][e], u1[e], dh);
      }
      if constexpr (DUMP) {
        dump_add<M>(pl, m, i, blk, nb32, dl);
        dump_add<M>(pl, m, i, blk + 1, nb32, dh);
      }
      const float sd = d80 * (float)(dl * sc0[i]) + d81 * (float)(dh * sc1[i]);
      const float sm = xs0 * dmn0[i] + xs1 * dmn1[i];
      acc[i][m] += dd[i] * sd - sm;
    }
  }
}

template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_Q6K>& r, int rec, int lane, bool ok, const Planes& pl,
                                           float (&acc)[4][M]) {
  (void)ok;
  const int n = lane >> 4, w16 = lane & 15;
  const int nb32 = pl.k >> 5;
  const int blk = rec * 8 + 4 * n + (w16 >> 3);
  int v0[4], v1[4], s0[4], s1[4];
  float dd[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t vh = r.qh[i] >> (2 * (w16 >> 3));
    const uint32_t x0 = (r.ql[i] & 0x0F0F0F0Fu) | ((vh << 4) & 0x30303030u);
    const uint32_t x1 = ((r.ql[i] >> 4) & 0x0F0F0F0Fu) | (vh & 0x30303030u);
    v0[i] = (int)((((x0 | 0x80808080u) - 0x20202020u)) ^ 0x80808080u);  // per-byte x - 32
    v1[i] = (int)((((x1 | 0x80808080u) - 0x20202020u)) ^ 0x80808080u);
    s0[i] = (int)(int8_t)(r.sc[i] & 0xFFu);
    s1[i] = (int)(int8_t)((r.sc[i] >> 8) & 0xFFu);
    dd[i] = h2f(r.d[i]);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int* xr = reinterpret_cast<const int*>(pl.xq + (int64_t)m * pl.k + (int64_t)blk * 32) + (w16 & 7);
    const int u0 = xr[0], u1 = xr[16];  // 64 values further: q8 block blk + 2
    const float d80 = pl.xd[m * nb32 + blk], d81 = pl.xd[m * nb32 + blk + 2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p0 = dp4a(v0[i], u0, 0), p1 = dp4a(v1[i], u1, 0);
      if constexpr (DUMP) {
        const int g16 = rec * 16 + 8 * n + (w16 >> 2);
        dump_add<M>(pl, m, i, g16, pl.k >> 4, p0);
        dump_add<M>(pl, m, i, g16 + 4, pl.k >> 4, p1);
      }
      const float sf = d80 * (float)(p0 * s0[i]) + d81 * (float)(p1 * s1[i]);
      acc[i][m] = fmaf(dd[i], sf, acc[i][m]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The kernel.

template <int KIND>
__host__ __device__ constexpr bool kind_uses_grid() { return KIND == KIND_IQ3S_PACKED || KIND == KIND_IQ3S_RAW; }

__host__ __device__ inline size_t gemv_smem_bytes(int kind, int rs, int m, int k) {
  size_t s = 0;
  if (kind == KIND_IQ3S_PACKED || kind == KIND_IQ3S_RAW) s += (size_t)512 << rs;  // replicated codebook
  s += (size_t)m * k;                                   // int8 plane
  s += (size_t)m * (k / 32) * 4;                        // d plane
  if (kind == KIND_Q4K) s += (size_t)m * (k / 32) * 4;  // d * sum(q) plane
  s += (size_t)GEMV_WARPS * 16 * m * 4;                 // partial sums
  return s;
}

template <int KIND, int M, int RS, bool DUMP>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int TR = KindTraits<KIND>::tile_rows;
  constexpr int RSB = KindTraits<KIND>::rec_sb;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nb32 = a.k >> 5;

  uint8_t* sp = smem;
  uint32_t* grid_s = reinterpret_cast<uint32_t*>(sp);
  if (kind_uses_grid<KIND>()) sp += (size_t)512 << RS;
  int8_t* xq = reinterpret_cast<int8_t*>(sp);
  sp += (size_t)M * a.k;
  float* xd = reinterpret_cast<float*>(sp);
  sp += (size_t)M * nb32 * 4;
  float* xs = reinterpret_cast<float*>(sp);
  if (KIND == KIND_Q4K) sp += (size_t)M * nb32 * 4;
  float* partial = reinterpret_cast<float*>(sp);  // [warp][16][M]

  // stage the codebook copies and the activation planes
  if (kind_uses_grid<KIND>()) {
    constexpr int REP = 1 << (RS - 2);
    for (int i = tid; i < 512 * REP; i += GEMV_THREADS) grid_s[i] = g_iq3s_grid[i >> (RS - 2)];
  }
  for (int b = tid; b < M * nb32; b += GEMV_THREADS) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.xq8 + (int64_t)b * 36);
    uint32_t q[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) q[e] = __ldg(src + e);
    const uint32_t ds = __ldg(src + 8);
    uint4* dst = reinterpret_cast<uint4*>(xq + (int64_t)b * 32);
    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
    const float d = h2f(ds);
    xd[b] = d;
    if (KIND == KIND_Q4K) {
      int s = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) s = dp4a(0x01010101, (int)q[e], s);
      xs[b] = d * (float)s;
    }
  }
  __syncthreads();

  Planes pl;
  pl.xq = xq; pl.xd = xd; pl.xs = xs; pl.grid = grid_s; pl.k = a.k;
  pl.dump = a.dump; pl.dump_rows = a.nrows; pl.dump_m0 = a.dump_m0; pl.dump_row0 = 0;

  const int parts = a.parts;
  const int tiles = GEMV_WARPS / parts;
  const int tile_l = warp / parts, part = warp - tile_l * parts;
  const int nsb = a.k >> 8;
  const int r_begin = part * a.rec_per_part;
  const int r_end = min(a.nrec, r_begin + a.rec_per_part);

  for (int unit = blockIdx.x; unit < a.n_units; unit += gridDim.x) {
    const int row0 = (unit * tiles + tile_l) * TR;
    pl.dump_row0 = row0;
    float acc[4][M];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[i][m] = 0.0f;

    if (row0 < a.nrows && r_begin < r_end) {
      Rec<KIND> cur;
      bool ok_cur = RSB == 1 || (r_begin * 4 + (lane >> 3)) < nsb;
      cur.load(a, row0, r_begin, lane, ok_cur);
#pragma unroll 1
      for (int rec = r_begin; rec < r_end; ++rec) {
        Rec<KIND> nxt;
        const bool has_next = rec + 1 < r_end;
        const bool ok_nxt = has_next && (RSB == 1 || ((rec + 1) * 4 + (lane >> 3)) < nsb);
        nxt.load(a, row0, rec + 1, lane, ok_nxt);
        accumulate<M, RS, DUMP>(cur, rec, lane, ok_cur, pl, acc);
        cur = nxt;
        ok_cur = ok_nxt;
      }
    }

    // lanes that share weight rows add up; then one lane per row group parks the sums in shared memory
    if (KIND == KIND_IQ3S_PACKED) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float v = acc[i][m];
          v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
          v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
          v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
          acc[i][m] = v;
        }
      if ((lane & 7) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int m = 0; m < M; ++m) partial[(warp * 16 + (lane >> 3) + 4 * i) * M + m] = acc[i][m];
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float v = acc[i][m];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
          acc[i][m] = v;
        }
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int m = 0; m < M; ++m) partial[(warp * 16 + i) * M + m] = acc[i][m];
      }
    }
    __syncthreads();
    const int rows_step = tiles * TR;
    for (int o = tid; o < rows_step * M; o += GEMV_THREADS) {
      const int m = o / rows_step, rr = o - m * rows_step;
      const int tl = rr / TR, ri = rr - tl * TR;
      const int row = (unit * tiles + tl) * TR + ri;
      if (row < a.nrows) {
        float v = 0.0f;
        for (int p = 0; p < parts; ++p) v += partial[((tl * parts + p) * 16 + ri) * M + m];
        store_out_dyn(a.y, a.y_dtype, (int64_t)m * a.ldy + row, v);
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// Host side.

static int g_iq4_table_device_mask = 0;  // bit d set once device d has c_iq4nl_words

int gemv_device_init(int device) {
  if (device < 32 && (g_iq4_table_device_mask >> device) & 1) return GSQ_OK;
  const int8_t vals[16] = GSQ_IQ4NL_VALUES_INIT;
  uint32_t words[4];
  for (int i = 0; i < 4; ++i) {
    words[i] = 0;
    for (int j = 0; j < 4; ++j) words[i] |= (uint32_t)(uint8_t)vals[4 * i + j] << (8 * j);
  }
  GSQ_CUDA_TRY(cudaMemcpyToSymbol(c_iq4nl_words, words, sizeof(words)));
  if (device < 32) g_iq4_table_device_mask |= 1 << device;
  return GSQ_OK;
}

template <int KIND, int M, int RS, bool DUMP = false>
static int launch_gemv(const GemvArgs& a, int grid, size_t smem, cudaStream_t st) {
  auto kern = gemv_kernel<KIND, M, RS, DUMP>;
  static int configured_mask = 0;  // per instantiation: devices whose smem attribute is set
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 32 || !((configured_mask >> dev) & 1)) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev < 32) configured_mask |= 1 << dev;
  }
  kern<<<grid, GEMV_THREADS, smem, st>>>(a);
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}

template <int KIND, int RS>
static int launch_gemv_m(int m, const GemvArgs& a, int grid, size_t smem, cudaStream_t st) {
  switch (m) {
    case 1: return launch_gemv<KIND, 1, RS>(a, grid, smem, st);
    case 2: return launch_gemv<KIND, 2, RS>(a, grid, smem, st);
    case 3: return launch_gemv<KIND, 3, RS>(a, grid, smem, st);
    case 4: return launch_gemv<KIND, 4, RS>(a, grid, smem, st);
    case 5: return launch_gemv<KIND, 5, RS>(a, grid, smem, st);
    case 6: return launch_gemv<KIND, 6, RS>(a, grid, smem, st);
    case 7: return launch_gemv<KIND, 7, RS>(a, grid, smem, st);
    case 8: return launch_gemv<KIND, 8, RS>(a, grid, smem, st);
    default: return GSQ_ERR_UNSUPPORTED;
  }
}

}  // namespace gsq

namespace gsq {
static int gemv_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_q8,
                     int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
                     int dump_m0) {
  if (m == 0 || rows == 0) return GSQ_OK;
  if (m < 0 || m > 8 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !x_q8 || !y) return GSQ_ERR_UNSUPPORTED;
  if (rows > INT32_MAX || k > INT32_MAX) return GSQ_ERR_TOO_LARGE;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  int kind;
  switch (ggml_type) {
    case GSQ_TYPE_IQ3_S: kind = packed ? KIND_IQ3S_PACKED : KIND_IQ3S_RAW; break;
    case GSQ_TYPE_Q4_K: kind = KIND_Q4K; break;
    case GSQ_TYPE_IQ4_XS: kind = KIND_IQ4XS; break;
    case GSQ_TYPE_Q6_K: kind = KIND_Q6K; break;
    default: return GSQ_ERR_UNSUPPORTED;
  }
  if (kind == KIND_IQ3S_PACKED && rows % 16 != 0) return GSQ_ERR_UNSUPPORTED;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;

  const int tile_rows = kind == KIND_IQ3S_PACKED ? 16 : 4;
  const int rec_sb = (kind == KIND_IQ3S_PACKED || kind == KIND_Q6K) ? 1 : 4;
  const int nsb = (int)(k / 256);
  const int nrec = (nsb + rec_sb - 1) / rec_sb;
  const int ntiles = (int)((rows + tile_rows - 1) / tile_rows);
  // column parts: as few as keep every SM busy (each extra part shortens a warp's run of records and
  // adds to the shared-memory reduction), never more than the records of a tile
  int parts = 1;
  while (parts < GEMV_WARPS && parts * 2 <= nrec &&
         (ntiles + (GEMV_WARPS / parts) - 1) / (GEMV_WARPS / parts) < 2 * di.sm_count) {
    parts *= 2;
  }
  const int tiles = GEMV_WARPS / parts;
  GemvArgs a;
  a.w = (const uint8_t*)w;
  a.row_bytes = row_bytes;
  a.nrows = (int)rows;
  a.k = (int)k;
  a.xq8 = (const uint8_t*)x_q8;
  a.y = y;
  a.y_dtype = y_dtype;
  a.ldy = y_row_stride;
  a.parts = parts;
  a.n_units = (ntiles + tiles - 1) / tiles;
  a.nrec = nrec;
  a.rec_per_part = (nrec + parts - 1) / parts;
  a.dump = dump;
  a.dump_m0 = dump_m0;
  const int grid = a.n_units < di.sm_count ? a.n_units : di.sm_count;
  cudaStream_t st = (cudaStream_t)stream;

  const bool uses_grid = kind == KIND_IQ3S_PACKED || kind == KIND_IQ3S_RAW;
  int rs = 7;
  size_t smem = gemv_smem_bytes(kind, rs, (int)m, (int)k);
  if (uses_grid && smem > (size_t)di.max_smem_optin) {
    rs = 5;
    smem = gemv_smem_bytes(kind, rs, (int)m, (int)k);
  }
  if (smem > (size_t)di.max_smem_optin) return GSQ_ERR_TOO_LARGE;

  if (dump) {  // debug build of the same kernel, one activation row per launch
    if (m != 1) return GSQ_ERR_UNSUPPORTED;
    switch (kind) {
      case KIND_IQ3S_PACKED:
        return rs == 7 ? launch_gemv<KIND_IQ3S_PACKED, 1, 7, true>(a, grid, smem, st)
                       : launch_gemv<KIND_IQ3S_PACKED, 1, 5, true>(a, grid, smem, st);
      case KIND_IQ3S_RAW:
        return rs == 7 ? launch_gemv<KIND_IQ3S_RAW, 1, 7, true>(a, grid, smem, st)
                       : launch_gemv<KIND_IQ3S_RAW, 1, 5, true>(a, grid, smem, st);
      case KIND_Q4K: return launch_gemv<KIND_Q4K, 1, 7, true>(a, grid, smem, st);
      case KIND_IQ4XS: return launch_gemv<KIND_IQ4XS, 1, 7, true>(a, grid, smem, st);
      default: return launch_gemv<KIND_Q6K, 1, 7, true>(a, grid, smem, st);
    }
  }
  switch (kind) {
    case KIND_IQ3S_PACKED:
      return rs == 7 ? launch_gemv_m<KIND_IQ3S_PACKED, 7>((int)m, a, grid, smem, st)
                     : launch_gemv_m<KIND_IQ3S_PACKED, 5>((int)m, a, grid, smem, st);
    case KIND_IQ3S_RAW:
      return rs == 7 ? launch_gemv_m<KIND_IQ3S_RAW, 7>((int)m, a, grid, smem, st)
                     : launch_gemv_m<KIND_IQ3S_RAW, 5>((int)m, a, grid, smem, st);
    case KIND_Q4K: return launch_gemv_m<KIND_Q4K, 7>((int)m, a, grid, smem, st);
    case KIND_IQ4XS: return launch_gemv_m<KIND_IQ4XS, 7>((int)m, a, grid, smem, st);
    default: return launch_gemv_m<KIND_Q6K, 7>((int)m, a, grid, smem, st);
  }
}
}  // namespace gsq

extern "C" int gsq_mul_mat_vec_q8(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                                  const void* x_q8, int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride,
                                  void* stream) {
  return gsq::gemv_host(w, row_bytes, rows, ggml_type, packed, x_q8, m, k, y, y_dtype, y_row_stride, stream, nullptr, 0);
}

extern "C" int gsq_debug_block_sums(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                                    const void* x_q8, int64_t m, int64_t k, int32_t* sums, float* y_scratch,
                                    void* stream) {
  if (!sums || !y_scratch) return GSQ_ERR_UNSUPPORTED;
  for (int64_t i = 0; i < m; ++i) {
    const int rc = gsq::gemv_host(w, row_bytes, rows, ggml_type, packed, (const uint8_t*)x_q8 + i * (k / 32) * 36, 1, k,
                                  y_scratch, GSQ_F32, rows, stream, sums, (int)i);
    if (rc != GSQ_OK) return rc;
  }
  return GSQ_OK;
}
