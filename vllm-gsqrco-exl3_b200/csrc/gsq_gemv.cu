// Streaming dp4a GEMV for 1..8 activation rows over GGUF superblocks (sm_100a).
//
// Replaces, behind gsq_mul_mat_vec_q8, the reference's MMVQ (csrc/lcpp/ggml/src/ggml-cuda/mmvq.cu:599-844
// with the vec_dot_*_q8_1 functions of vecdotq.cuh) and its owned 1..8-row kernels
// (lcpp_shim.cu:498-572, lcpp_owned_k4.cu:116-234, lcpp_owned_iq3_mma.cu:483-600). The per-slice integer
// sums and the slice terms d_w * d_q8 * scale * sumi are the reference's; only the fp32 order in which
// a row's slice terms are added differs (fixed, so results are run-to-run and graph-replay identical).
//
// Shape of the kernel: one CTA of 16 warps per SM, CTAs grouped in thread-block clusters of 4.
//   * A "record" is what one warp consumes per step, every lane decoding its 32 values of 4 weight rows
//     once and dotting them with each activation row:
//        IQ3_S packed : one 16-row x 256-column tile record of gsq_iq3s_repack (1760 bytes);
//                       lane = (g = lane / 4, t = lane % 4): rows g, g+8, 4-value groups 2t, 2t+1 of every slice
//        Q4_K, IQ4_XS, IQ3_S in GGUF order : 4 rows x 4 superblocks; lane = (superblock, 32-value chunk)
//        Q6_K         : 4 rows x 1 superblock; lane = 4-byte word of ql
//   * Each cluster owns a contiguous range of row tiles, i.e. a contiguous byte range of W. The records of
//     that range, in memory order, are cut into equal contiguous chunks, one per warp of the cluster, so
//     every warp streams the same number of bytes whatever the shape. A warp reads its chunk with 128-bit
//     no-allocate loads straight into registers, one record ahead of the arithmetic, across tile
//     boundaries, with no block-wide barrier in the loop.
//   * Chunks do not respect tile boundaries: when a warp leaves a tile it parks that tile's partial sums
//     in its CTA's shared memory. After one cluster barrier the threads of the cluster add, for every row,
//     the partial sums of the warps that touched it, in warp order, reading the other CTAs' shared memory
//     (distributed shared memory), and write Y in its final dtype. No atomics, no global scratch.
//   * The q8_1 activations are read where they lie (36-byte blocks) through L1; every SM pulls them from
//     L2 once. IQ3_S reads its 512-entry codebook from a shared-memory copy replicated per lane (entry i of
//     lane l at word 32 i + l), so the data-dependent lookups never collide on a bank.
#include <cooperative_groups.h>

#include "gsq_common.cuh"
#include "gsq_tables.h"

namespace cg = cooperative_groups;

namespace gsq {

enum { KIND_IQ3S_PACKED = 0, KIND_IQ3S_RAW = 1, KIND_Q4K = 2, KIND_IQ4XS = 3, KIND_Q6K = 4 };

constexpr int GEMV_WARPS = 16;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

__device__ const uint32_t g_iq3s_grid[512] = GSQ_IQ3S_GRID_INIT;
// the 16 non-linear IQ4 values, read as four words of four bytes (statically initialised: no upload at run time)
__constant__ __align__(16) int8_t c_iq4nl_bytes[16] = GSQ_IQ4NL_VALUES_INIT;
#define c_iq4nl_words (reinterpret_cast<const uint32_t*>(c_iq4nl_bytes))

constexpr int SEG_CAP = 4;  // most tiles one warp's chunk may touch in a round

struct GemvArgs {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;
  int k;
  const uint8_t* xq8;
  void* y;
  int y_dtype;
  int64_t ldy;
  int ntiles;        // row tiles in W
  int nrec;          // records per row tile
  int tiles_base;    // tiles per cluster: the first tiles_extra clusters own tiles_base + 1
  int tiles_extra;
  int tiles_round;   // tiles a cluster takes per round (<= (SEG_CAP - 2) * warps per cluster)
  int stage_shift;   // log2 of the bulk-copy ring depth per warp (staged variant only)
  int force_direct;  // tests: use the direct-load variant even where the staged one applies
  int* dump;         // debug only: integer slice sums
  int dump_m0;
  int early;         // let the next kernel of a programmatic-launch chain start while this one runs
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

// Packed IQ3_S record (see gsq_repack.cu for the layout): per lane 9 words of 9-bit codebook indices (field
// f = 4 s + 2 h + e: slice s, row g + 8 h, group 2t + e, at bit 9 f), 4 words of sign bits (field f in word f / 8;
// bit 16 ((f % 8) / 4) + 4 p + f % 4 = sign of value p), the sub-scale nibbles and the fp16 d of rows g, g + 8.
template <>
struct Rec<KIND_IQ3S_PACKED> {
  uint32_t idx[9];
  uint32_t sg[4];
  uint2 sc;
  uint32_t dd;
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
    sc = ldg_stream_v2(p + 1664 + 8 * (lane >> 2));
    dd = ldg_stream_u32(p + 1728 + 4 * (lane >> 2));
  }
  // the same record already staged in shared memory by a bulk copy
  __device__ __forceinline__ void load_smem(const uint8_t* p, int lane, bool ok, int = 0) {
    (void)ok;
    const uint4 ia = *reinterpret_cast<const uint4*>(p + 16 * lane);
    const uint4 ib = *reinterpret_cast<const uint4*>(p + 512 + 16 * lane);
    idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
    idx[4] = ib.x; idx[5] = ib.y; idx[6] = ib.z; idx[7] = ib.w;
    idx[8] = *reinterpret_cast<const uint32_t*>(p + 1024 + 4 * lane);
    const uint4 s = *reinterpret_cast<const uint4*>(p + 1152 + 16 * lane);
    sg[0] = s.x; sg[1] = s.y; sg[2] = s.z; sg[3] = s.w;
    sc = *reinterpret_cast<const uint2*>(p + 1664 + 8 * (lane >> 2));
    dd = *reinterpret_cast<const uint32_t*>(p + 1728 + 4 * (lane >> 2));
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
  __device__ __forceinline__ void load_smem(const uint8_t*, int, bool, int = 0) {}
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
  // staged record: row i's superblocks at p + i * row_stride
  __device__ __forceinline__ void load_smem(const uint8_t* p, int lane, bool ok, int row_stride = 576) {
    if (!ok) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint8_t* b = p + i * row_stride + (lane >> 3) * 144;
      hdr[i] = *reinterpret_cast<const uint4*>(b);
      qs[i] = *reinterpret_cast<const uint4*>(b + 16 + 16 * (lane & 7));
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
  // staged record: row i's superblocks at p + i * row_stride
  __device__ __forceinline__ void load_smem(const uint8_t* p, int lane, bool ok, int row_stride = 544) {
    if (!ok) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint8_t* b = p + i * row_stride + (lane >> 3) * 136;
      hdr[i] = *reinterpret_cast<const uint2*>(b);
      qa[i] = *reinterpret_cast<const uint2*>(b + 8 + 16 * (lane & 7));
      qb[i] = *reinterpret_cast<const uint2*>(b + 16 + 16 * (lane & 7));
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
  __device__ __forceinline__ void load_smem(const uint8_t*, int, bool, int = 0) {}
};

// ---------------------------------------------------------------------------------------------
// Decode + dot. Activations are block_q8_1 in global memory (L1-cached reads).

struct Ctx {
  const uint8_t* xq8;    // [m][k/32] blocks of 36 bytes
  const uint32_t* grid;  // replicated IQ3_S codebook (shared memory)
  int k;
  int nb32;
  // debug dump of the raw integer slice sums (gsq_debug_block_sums): out[(m * nrows + row) * (k / g) + group]
  int* dump;
  int dump_rows, dump_m0;
};

__device__ __forceinline__ void dump_add(const Ctx& cx, int m, int row, int group, int groups, int v) {
  if (row < cx.dump_rows) atomicAdd(cx.dump + ((int64_t)(cx.dump_m0 + m) * cx.dump_rows + row) * groups + group, v);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ const uint32_t* q8_block(const Ctx& cx, int m, int blk) {
  return reinterpret_cast<const uint32_t*>(cx.xq8 + ((int64_t)m * cx.nb32 + blk) * 36);
}

// wv[i][e] = 4 signed int8 of group e (values 4e..4e+3 of the lane's slice) of row i; common dot loop of
// the kinds whose lane owns one whole 32-value slice with a single integer sub-scale.
template <int M, bool DUMP>
__device__ __forceinline__ void dot_slice(const int (&wv)[4][8], const int (&isc)[4], const float (&dw)[4],
                                          const Ctx& cx, int blk, int row_base, int row_step, float (&acc)[4][M]) {
  float dws[4];  // d_w times the integer sub-scale: exact in fp32 (11-bit by 6-bit significands)
#pragma unroll
  for (int i = 0; i < 4; ++i) dws[i] = dw[i] * (float)isc[i];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const uint32_t* b = q8_block(cx, m, blk);
    int u[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) u[e] = (int)__ldg(b + 1 + e);  // word 0 of a block is (d, sum), the quants follow
    const float d8 = h2f(__ldg(b));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int sumi = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) sumi = dp4a(wv[i][e], u[e], sumi);
      if constexpr (DUMP) dump_add(cx, m, row_base + row_step * i, blk, cx.nb32, sumi);
      // |sumi| <= 32 * 127 * 127 < 2^22: adding the bit pattern of 1.5 * 2^23 makes it a float without a conversion
      const float sf = __int_as_float(sumi + 0x4B400000) - 12582912.0f;
      acc[i][m] = fmaf(dws[i] * d8, sf, acc[i][m]);
    }
  }
}

// The codebook copy in shared memory holds, per entry and per lane-mod-16 replica, the pair (g, -g) of packed
// int8x4 words (entry i of replica r at byte 128 i + 8 r): a 64-bit load per half-warp touches every bank once.
// A group's signed word is then one byte permute of the pair, the selector built from the record's sign bits.
// The lane dots its two groups of each slice of rows g and g + 8 (accumulator rows 0 and 1; 2 and 3 stay zero);
// the four lanes of a row group add up when the tile is left.
template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_IQ3S_PACKED>& r, int row0, int rec, int lane, bool ok,
                                           const Ctx& cx, float (&acc)[4][M]) {
  (void)ok;
  const uint32_t lane_off = (uint32_t)(lane & 15) << 3;
  const char* gbase = reinterpret_cast<const char*>(cx.grid);
  const int g = lane >> 2, t = lane & 3;
  const float dw[2] = {h2f(r.dd), h2f(r.dd >> 16)};
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    int wv[2][2];
    float dws[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int f = 4 * s + 2 * h + e, bit = 9 * f, word = bit >> 5, off = bit & 31;
        uint32_t v;
        if (off + 9 <= 32) {
          v = off >= 7 ? r.idx[word] >> (off >= 7 ? off - 7 : 0) : r.idx[word] << (off < 7 ? 7 - off : 0);
        } else {
          v = __funnelshift_r(r.idx[word], r.idx[word + 1], off - 7);
        }
        const uint2 gp = *reinterpret_cast<const uint2*>(gbase + ((v & 0xFF80u) | lane_off));
        // sign of value p of field f sits at bit 16 ((f % 8) / 4) + 4 p + f % 4: move it to bit 4 p + 2 of the selector
        const int fl = f & 7, sh = 16 * (fl >> 2) + (fl & 3) - 2;
        const uint32_t sgs = sh >= 0 ? r.sg[f >> 3] >> (sh >= 0 ? sh : 0) : r.sg[f >> 3] << (sh < 0 ? -sh : 0);
        wv[h][e] = (int)prmt(gp.x, gp.y, (sgs & 0x4444u) | 0x3210u);
      }
      const uint32_t scw = h ? r.sc.y : r.sc.x;
      dws[h] = dw[h] * (float)(1 + 2 * (int)((scw >> (4 * s)) & 15u));  // exact in fp32
    }
    const int blk = rec * 8 + s;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint32_t* b = q8_block(cx, m, blk);
      const int u0 = (int)__ldg(b + 1 + 2 * t), u1 = (int)__ldg(b + 2 + 2 * t);
      const float d8 = h2f(__ldg(b));
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int sumi = dp4a(wv[h][1], u1, dp4a(wv[h][0], u0, 0));
        if constexpr (DUMP) dump_add(cx, m, row0 + g + 8 * h, blk, cx.nb32, sumi);
        const float sf = __int_as_float(sumi + 0x4B400000) - 12582912.0f;
        acc[h][m] = fmaf(dws[h] * d8, sf, acc[h][m]);
      }
    }
  }
}

template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_IQ3S_RAW>& r, int row0, int rec, int lane, bool ok,
                                           const Ctx& cx, float (&acc)[4][M]) {
  if (!ok) return;
  const uint32_t lane_off = (uint32_t)(lane & 15) << 3;
  const char* gbase = reinterpret_cast<const char*>(cx.grid);
  int wv[4][8];
  int isc[4];
  float dw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t byte = (r.qs[i][e >> 2] >> (8 * (e & 3))) & 0xFFu;
      const uint32_t idx = byte | ((r.qh[i] << (8 - e)) & 0x100u);
      const uint32_t g = *reinterpret_cast<const uint32_t*>(gbase + ((idx << 7) | lane_off));
      const uint32_t ones = (((r.sg[i] >> (4 * e)) & 0xFu) * 0x00204081u) & 0x01010101u;
      wv[i][e] = (int)((g ^ (ones * 0xFFu)) + ones);
    }
    isc[i] = 1 + 2 * (int)r.ls[i];
    dw[i] = h2f(r.d[i]);
  }
  dot_slice<M, DUMP>(wv, isc, dw, cx, (rec * 4 + (lane >> 3)) * 8 + (lane & 7), row0, 1, acc);
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
__device__ __forceinline__ void accumulate(const Rec<KIND_IQ4XS>& r, int row0, int rec, int lane, bool ok,
                                           const Ctx& cx, float (&acc)[4][M]) {
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
  dot_slice<M, DUMP>(wv, isc, dw, cx, (rec * 4 + (lane >> 3)) * 8 + p, row0, 1, acc);
}

// Q4_K. Lane (superblock b, chunk p) holds 16 bytes of 4 rows: low nibbles = 16 values of sub-block 2 jj,
// high nibbles = 16 values of sub-block 2 jj + 1 (jj = p / 2). The 6-bit scale / min pair of those two
// sub-blocks comes out of the 12 packed bytes with lane-constant byte permutes and masks (no branches):
//   jj < 2 : sc = q16[jj] & 0x3f3f,                                   m = q16[2 + jj] & 0x3f3f
//   jj >= 2: sc = (q16[jj + 2] & 0x0f0f) | ((q16[jj - 2] & 0xc0c0) >> 2), m = ((q16[jj + 2] >> 4) & 0x0f0f) | ((q16[jj] & 0xc0c0) >> 2)
// with q16[] the bytes taken as six halfwords. Integer sums become floats by adding the bit pattern of
// 1.5 * 2^23 inside the integer multiply-add and subtracting it again as a float (exact below 2^22), which
// keeps the conversions off the slow conversion pipe.
template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_Q4K>& r, int row0, int rec, int lane, bool ok,
                                           const Ctx& cx, float (&acc)[4][M]) {
  if (!ok) return;
  const int p = lane & 7, jj = p >> 1, half = p & 1;
  const bool lo4 = jj < 2;
  const uint32_t selh = (jj & 1) ? 0x4432u : 0x4410u;          // halfword jj % 2 of a word, zero-extended
  const uint32_t m_low = lo4 ? 0x3F3Fu : 0u, m_top = lo4 ? 0u : 0xC0C0u, m_nib = lo4 ? 0u : 0x0F0Fu;
  const int blk = (rec * 4 + (lane >> 3)) * 8 + 2 * jj;        // q8 block of the low nibbles; high nibbles: blk + 1
  constexpr int MAGIC = 0x4B400000;
  constexpr float MAGIC_F = 12582912.0f;
  int lo[4][4], hi[4][4];
  int sc0[4], sc1[4];
  float dd[4], dmn0[4], dmn1[4];  // d, and -dmin times each sub-block's 6-bit min
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t q[4] = {r.qs[i].x, r.qs[i].y, r.qs[i].z, r.qs[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      lo[i][e] = (int)(q[e] & 0x0F0F0F0Fu);
      hi[i][e] = (int)((q[e] >> 4) & 0x0F0F0F0Fu);
    }
    const uint32_t A = prmt(r.hdr[i].y, 0u, selh), B = prmt(r.hdr[i].z, 0u, selh), C = prmt(r.hdr[i].w, 0u, selh);
    const uint32_t sc = (A & m_low) | ((A & m_top) >> 2) | (C & m_nib);
    const uint32_t mn = (B & m_low) | ((B & m_top) >> 2) | ((C >> 4) & m_nib);
    sc0[i] = (int)(sc & 0xFFu);
    sc1[i] = (int)(sc >> 8);
    dd[i] = h2f(r.hdr[i].x);
    const float ndm = -h2f(r.hdr[i].x >> 16);
    dmn0[i] = ndm * (__int_as_float((int)(mn & 0xFFu) + MAGIC) - MAGIC_F);
    dmn1[i] = ndm * (__int_as_float((int)(mn >> 8) + MAGIC) - MAGIC_F);
  }
  const uint32_t* b0 = q8_block(cx, 0, blk) + 1 + 4 * half;  // this lane's 4 quant words (word 0 of a block is (d, sum))
  const int64_t mstride = (int64_t)cx.nb32 * 9;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const uint32_t* bm = b0 + m * mstride;
    int u0[4], u1[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      u0[e] = (int)__ldg(bm + e);
      u1[e] = (int)__ldg(bm + 9 + e);
    }
    const float d80 = h2f(__ldg(bm - 1 - 4 * half)), d81 = h2f(__ldg(bm + 8 - 4 * half));
    // sum of the activation quants this lane pairs with its 16 + 16 weights (the min term's factor)
    int q0 = 0, q1 = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      q0 = dp4a(0x01010101, u0[e], q0);
      q1 = dp4a(0x01010101, u1[e], q1);
    }
    const float xs0 = d80 * (__int_as_float(q0 + MAGIC) - MAGIC_F), xs1 = d81 * (__int_as_float(q1 + MAGIC) - MAGIC_F);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int dl = 0, dh = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dl = dp4a(lo[i][e], u0[e], dl);
        dh = dp4a(hi[i][e], u1[e], dh);
      }
      if constexpr (DUMP) {
        dump_add(cx, m, row0 + i, blk, cx.nb32, dl);
        dump_add(cx, m, row0 + i, blk + 1, cx.nb32, dh);
      }
      const float fi0 = __int_as_float(dl * sc0[i] + MAGIC) - MAGIC_F;
      const float fi1 = __int_as_float(dh * sc1[i] + MAGIC) - MAGIC_F;
      const float t = fmaf(fi1, d81, fi0 * d80);
      acc[i][m] = fmaf(xs1, dmn1[i], fmaf(xs0, dmn0[i], fmaf(t, dd[i], acc[i][m])));
    }
  }
}

template <int M, int RS, bool DUMP>
__device__ __forceinline__ void accumulate(const Rec<KIND_Q6K>& r, int row0, int rec, int lane, bool ok,
                                           const Ctx& cx, float (&acc)[4][M]) {
  (void)ok;
  const int n = lane >> 4, w16 = lane & 15;
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
    const uint32_t* b0 = q8_block(cx, m, blk);
    const uint32_t* b1 = q8_block(cx, m, blk + 2);  // 64 values further
    const int u0 = (int)__ldg(b0 + 1 + (w16 & 7)), u1 = (int)__ldg(b1 + 1 + (w16 & 7));
    const float d80 = h2f(__ldg(b0)), d81 = h2f(__ldg(b1));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p0 = dp4a(v0[i], u0, 0), p1 = dp4a(v1[i], u1, 0);
      if constexpr (DUMP) {
        const int g16 = rec * 16 + 8 * n + (w16 >> 2);
        dump_add(cx, m, row0 + i, g16, cx.k >> 4, p0);
        dump_add(cx, m, row0 + i, g16 + 4, cx.k >> 4, p1);
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
// The staged variant moves SUB records per ring stage (one wait, one refill and one round of loop
// bookkeeping per 3.5 - 4.6 KB instead of per 1.8 - 2.3 KB).
constexpr int SUB = 2;
template <int KIND>
__host__ __device__ constexpr int rec_bytes() {
  return KIND == KIND_IQ3S_PACKED ? 1760 : KindTraits<KIND>::rec_sb * KindTraits<KIND>::bs * 4;
}
template <int KIND>
__host__ __device__ constexpr int stage_bytes() { return SUB * rec_bytes<KIND>(); }

// Set (sticky) when a bounded wait on a bulk copy gave up; read through gsq_device_error_flag.
__device__ int g_gemv_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Wait for the phase with the given parity; gives up after about a second and raises the error flag.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity) {
  uint32_t done = 0;
  for (int spin = 0; spin < (1 << 22); ++spin) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return;
  }
  atomicExch(&g_gemv_error, 1);
}

// Lane 0 of a warp: start the bulk copies of one stage (SUB records) into the ring. Row-major kinds copy 4
// row segments (rows past the end of W are replaced by the last row; their results are never stored).
template <int KIND>
__device__ __forceinline__ void issue_record(const GemvArgs& a, uint32_t stage, uint32_t bar, int row0, int rec) {
  const int nsb = a.k >> 8;
  if (KIND == KIND_IQ3S_PACKED) {
    const uint32_t bytes = (uint32_t)min(SUB, nsb - rec * SUB) * 1760u;
    mbar_expect_tx(bar, bytes);
    bulk_g2s(stage, a.w + (int64_t)row0 * a.row_bytes + (int64_t)rec * (SUB * 1760), bytes, bar);
  } else {
    constexpr int BS = KindTraits<KIND>::bs;
    const int here = min(4 * SUB, nsb - rec * (4 * SUB));
    const uint32_t bytes = (uint32_t)(here * BS);
    mbar_expect_tx(bar, 4 * bytes);
    const uint8_t* src = a.w + (int64_t)row0 * a.row_bytes + (int64_t)rec * (4 * SUB * BS);
    const int last = a.nrows - 1 - row0;  // rows of this tile that exist, minus one
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      bulk_g2s(stage + i * (4 * SUB * BS), src + (int64_t)min(i, last) * a.row_bytes, bytes, bar);
    }
  }
}

__host__ __device__ inline size_t gemv_smem_bytes(int kind, int rs, int m, int stages) {
  const int tr = kind == KIND_IQ3S_PACKED ? 16 : 4;
  const int rb = kind == KIND_IQ3S_PACKED ? 1760 : kind == KIND_Q4K ? 2304 : kind == KIND_IQ4XS ? 2176 : 0;
  size_t s = 0;
  if (kind == KIND_IQ3S_PACKED || kind == KIND_IQ3S_RAW) s += (size_t)512 << rs;  // replicated codebook
  s += (size_t)GEMV_WARPS * SEG_CAP * tr * m * 4;                                  // partial sums of a round
  if (stages > 0) s += (size_t)GEMV_WARPS * stages * (SUB * rb + 8);               // ring + its barriers
  return s;
}

// TMA: weights come through a per-warp ring of bulk copies (cp.async.bulk + mbarrier) instead of direct loads.
template <int KIND, int M, int RS, bool DUMP, bool TMA>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TR = KindTraits<KIND>::tile_rows;
  constexpr int RSB = KindTraits<KIND>::rec_sb;
  constexpr int PBUF = GEMV_WARPS * SEG_CAP * TR * M;  // floats per partial buffer
  constexpr int RECB = TMA ? stage_bytes<KIND>() : rec_bytes<KIND>();
  cg::cluster_group cluster = cg::this_cluster();
  const int cs = (int)cluster.num_blocks();
  const int crank = (int)cluster.block_rank();
  const int cluster_id = (int)blockIdx.x / cs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nsb = a.k >> 8;
  const int nrec = a.nrec;

  uint8_t* sp = smem;
  uint32_t* grid_s = reinterpret_cast<uint32_t*>(sp);
  if (kind_uses_grid<KIND>()) sp += (size_t)512 << RS;
  float* partial = reinterpret_cast<float*>(sp);
  sp += (size_t)PBUF * 4;
  const int stages = 1 << a.stage_shift;
  const uint32_t smask = (uint32_t)stages - 1;
  // ring of this warp (16-byte aligned: every size above is a multiple of 16), then all the barriers
  const uint8_t* ring = sp + (size_t)warp * stages * RECB;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t bars_u32 = smem_u32(sp + (size_t)GEMV_WARPS * stages * RECB) + (uint32_t)(warp * stages * 8);

  Ctx cx;
  cx.xq8 = a.xq8; cx.grid = grid_s; cx.k = a.k; cx.nb32 = a.k >> 5;
  cx.dump = a.dump; cx.dump_rows = a.nrows; cx.dump_m0 = a.dump_m0;

  const int tile_begin = cluster_id * a.tiles_base + min(cluster_id, a.tiles_extra);
  const int tile_cnt = a.tiles_base + (cluster_id < a.tiles_extra ? 1 : 0);
  const int wc = cs * GEMV_WARPS;
  const int gw = crank * GEMV_WARPS + warp;

  if (TMA) {
    if (lane == 0) {
      for (int s = 0; s < stages; ++s) mbar_init(bars_u32 + 8 * s, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
  }

  // the first loads go out before anything else, so the codebook staging below hides behind them
  Rec<KIND> cur;
  bool ok_cur = false;
  uint32_t cnt = 0;       // records this warp has consumed (ring position and barrier phase)
  int pre_issued = 0;     // records of round 0 already in flight
  {
    const int tiles_r = min(a.tiles_round, tile_cnt);
    const int rr = tiles_r * nrec, c = (rr + wc - 1) / wc;
    const int idx0 = gw * c, idx1 = min(rr, idx0 + c);
    if (idx0 < idx1) {
      int tl = idx0 / nrec, rec = idx0 - tl * nrec;
      if (TMA) {
        for (; pre_issued < stages && idx0 + pre_issued < idx1; ++pre_issued) {
          if (lane == 0)
            issue_record<KIND>(a, ring_u32 + pre_issued * RECB, bars_u32 + 8 * pre_issued, (tile_begin + tl) * TR, rec);
          if (++rec == nrec) { rec = 0; ++tl; }
        }
      } else {
        ok_cur = RSB == 1 || (rec * 4 + (lane >> 3)) < nsb;
        cur.load(a, (tile_begin + tl) * TR, rec, lane, ok_cur);
      }
    }
  }
  if (kind_uses_grid<KIND>()) {
    // one global load per thread (512 threads, 512 entries), then the 16 replicas of its entry
    const uint32_t g = g_iq3s_grid[tid & 511];
    // per-byte negation: no byte of the codebook is zero, so ~g + 1 per byte never carries
    const uint2 pair = make_uint2(g, ~g + 0x01010101u);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(grid_s) + (tid & 511) * 16);
#pragma unroll
    for (int r2 = 0; r2 < 8; ++r2) dst[r2] = make_uint4(pair.x, pair.y, pair.x, pair.y);
    __syncthreads();
  }

  // Up to here nothing depends on the kernel that wrote the activations: launched with programmatic stream
  // serialisation, the first weight loads and the codebook copy overlap its tail (a no-op otherwise).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int t0 = 0; t0 < tile_cnt; t0 += a.tiles_round) {
    const int tiles_r = min(a.tiles_round, tile_cnt - t0);
    const int rr = tiles_r * nrec;
    const int c = (rr + wc - 1) / wc;  // records per warp this round
    const int idx0 = gw * c, idx1 = min(rr, idx0 + c);
    float* mypart = partial + warp * (SEG_CAP * TR * M);
    if (idx0 < idx1) {
      int tl = idx0 / nrec, rec = idx0 - tl * nrec;
      const int first_tl = tl;
      // issue cursor of the staged variant: the record `stages` ahead of the one being consumed
      int itl = tl, irec = rec, iidx = idx0;
      if (TMA) {
        int ahead = t0 == 0 ? pre_issued : 0;
        for (int j = 0; j < ahead; ++j) { if (++irec == nrec) { irec = 0; ++itl; } }
        iidx = idx0 + ahead;
        for (; ahead < stages && iidx < idx1; ++ahead, ++iidx) {
          const uint32_t st = (cnt + ahead) & smask;
          if (lane == 0) issue_record<KIND>(a, ring_u32 + st * RECB, bars_u32 + 8 * st, (tile_begin + t0 + itl) * TR, irec);
          if (++irec == nrec) { irec = 0; ++itl; }
        }
      } else if (t0 != 0) {
        ok_cur = RSB == 1 || (rec * 4 + (lane >> 3)) < nsb;
        cur.load(a, (tile_begin + t0 + tl) * TR, rec, lane, ok_cur);
      }
      float acc[4][M];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[i][m] = 0.0f;
#pragma unroll 1
      for (int idx = idx0; idx < idx1; ++idx) {
        const bool has_next = idx + 1 < idx1;
        const bool wrap = rec + 1 == nrec;
        const int ntl = wrap ? tl + 1 : tl, nrc = wrap ? 0 : rec + 1;
        Rec<KIND> nxt;
        bool ok_nxt = false;
        if (TMA) {
          const uint32_t st = cnt & smask;
          mbar_wait(bars_u32 + 8 * st, (cnt >> a.stage_shift) & 1u);
#pragma unroll
          for (int h = 0; h < SUB; ++h) {
            const int srec = rec * SUB + h;
            const bool okh = RSB == 1 ? srec < nsb : (srec * 4 + (lane >> 3)) < nsb;
            if (RSB == 1 && !okh) break;  // warp-uniform: the last stage of an odd superblock count is half full
            cur.load_smem(ring + st * RECB + h * (RSB == 1 ? rec_bytes<KIND>() : rec_bytes<KIND>() / 4), lane, okh,
                          RECB / 4);
            accumulate<M, RS, DUMP>(cur, (tile_begin + t0 + tl) * TR, srec, lane, okh, cx, acc);
          }
        } else {
          ok_nxt = has_next && (RSB == 1 || (nrc * 4 + (lane >> 3)) < nsb);
          nxt.load(a, (tile_begin + t0 + ntl) * TR, nrc, lane, ok_nxt);
          accumulate<M, RS, DUMP>(cur, (tile_begin + t0 + tl) * TR, rec, lane, ok_cur, cx, acc);
        }
        if (TMA) {
          // the stage has been read into registers and used: refill it with the record `stages` ahead
          __syncwarp();
          if (iidx < idx1) {
            const uint32_t st = cnt & smask;
            if (lane == 0) issue_record<KIND>(a, ring_u32 + st * RECB, bars_u32 + 8 * st, (tile_begin + t0 + itl) * TR, irec);
            if (++irec == nrec) { irec = 0; ++itl; }
            ++iidx;
          }
          ++cnt;
        }
        if (!has_next || wrap) {
          // leaving tile tl: lanes that share weight rows add up, one lane per row parks the sums
          float* seg = mypart + (tl - first_tl) * (TR * M);
          if (KIND == KIND_IQ3S_PACKED) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
              for (int m = 0; m < M; ++m) {
                float v = acc[i][m];
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                if ((lane & 3) == 0) seg[((lane >> 2) + 8 * i) * M + m] = v;
                acc[i][m] = 0.0f;
              }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int m = 0; m < M; ++m) {
                float v = acc[i][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0) seg[i * M + m] = v;
                acc[i][m] = 0.0f;
              }
          }
        }
        if (!TMA) {
          cur = nxt;
          ok_cur = ok_nxt;
        }
        tl = ntl;
        rec = nrc;
      }
    }
    cluster.sync();
    // The next kernels of a programmatic-launch chain write nothing before their own wait, which holds until this
    // grid has finished, so they may start while the sums are added. Not earlier than this barrier: the warps read
    // the activations through L1 for as long as they stream records, and a kernel launched meanwhile that reads new
    // activations at the same address through the same L1 could be served the old lines.
    if (a.early && t0 + a.tiles_round >= tile_cnt) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // every row of the round: add the partial sums of the warps that touched its tile, in warp order
    const int rows_r = tiles_r * TR;
    for (int e = crank * GEMV_THREADS + tid; e < rows_r * M; e += cs * GEMV_THREADS) {
      const int m = e / rows_r, r2 = e - m * rows_r;
      const int tl = r2 / TR, ri = r2 - tl * TR;
      const int row = (tile_begin + t0 + tl) * TR + ri;
      if (row < a.nrows) {
        const int w0 = (tl * nrec) / c, w1 = ((tl + 1) * nrec - 1) / c;
        float v = 0.0f;
        for (int w = w0; w <= w1; ++w) {
          const int seg = tl - (w * c) / nrec;
          const float* src = cluster.map_shared_rank(partial, w / GEMV_WARPS) +
                             ((w % GEMV_WARPS) * SEG_CAP + seg) * (TR * M) + ri * M + m;
          v += *src;
        }
        store_out_dyn(a.y, a.y_dtype, (int64_t)m * a.ldy + row, v);
      }
    }
    // the partial sums are reused by the next round, and no CTA may leave while another still reads its
    // shared memory
    cluster.sync();
  }
}

// ---------------------------------------------------------------------------------------------
// Host side.

static int g_force_direct = 0;
static int g_force_cluster = 0;  // tests / experiments: 0 = choose, else 1, 2 or 4
// Nothing of this kernel family needs a per-device upload (the tables are statically initialised constants).
int gemv_device_init(int device) {
  (void)device;
  return GSQ_OK;
}

struct ClusterPlan {
  int cs;        // CTAs per cluster
  int clusters;  // clusters launched (all co-resident)
};

// Per kernel instantiation and device: the cluster size that keeps most SMs busy with every cluster resident.
template <int KIND, int M, int RS, bool DUMP, bool TMA>
static int plan_clusters(size_t smem, int sm_count, ClusterPlan* out) {
  static ClusterPlan cache[32];
  static bool have[32];
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 32 && have[dev] && !g_force_cluster) {
    *out = cache[dev];
    return GSQ_OK;
  }
  auto kern = gemv_kernel<KIND, M, RS, DUMP, TMA>;
  GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  ClusterPlan best{1, sm_count};
  for (int cs : {4, 2}) {
    if (g_force_cluster && cs != g_force_cluster) continue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sm_count / cs * cs));
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = cs;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    n = n < sm_count / cs ? n : sm_count / cs;
    if (n * cs > best.cs * best.clusters || (best.cs == 1 && n * cs >= (sm_count * 15) / 16)) best = ClusterPlan{cs, n};
  }
  if (dev < 32 && !g_force_cluster) {
    cache[dev] = best;
    have[dev] = true;
  }
  *out = best;
  return GSQ_OK;
}

template <int KIND, int M, int RS, bool DUMP, bool TMA>
static int launch_gemv_t(GemvArgs a, int sm_count, int max_smem, cudaStream_t st) {
  // ring depth: the deepest power of two that fits beside the codebook and the partial sums
  int shift = 0;
  if (TMA) {
    shift = 2;
    while (shift > 1 && gemv_smem_bytes(KIND, RS, M, 1 << shift) > (size_t)max_smem) --shift;
  }
  a.stage_shift = shift;
  if (TMA) a.nrec = ((a.k >> 8) + KindTraits<KIND>::rec_sb * SUB - 1) / (KindTraits<KIND>::rec_sb * SUB);
  const size_t smem = gemv_smem_bytes(KIND, RS, M, TMA ? 1 << shift : 0);
  if (smem > (size_t)max_smem) return GSQ_ERR_TOO_LARGE;
  ClusterPlan plan;
  int rc = plan_clusters<KIND, M, RS, DUMP, TMA>(smem, sm_count, &plan);
  if (rc != GSQ_OK) return rc;
  const int wc = plan.cs * GEMV_WARPS;
  a.tiles_base = a.ntiles / plan.clusters;
  a.tiles_extra = a.ntiles % plan.clusters;
  a.tiles_round = (SEG_CAP - 2) * wc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(plan.clusters * plan.cs));
  cfg.blockDim = dim3(GEMV_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = plan.cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol.wait in the kernel
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_kernel<KIND, M, RS, DUMP, TMA>, a));
  return GSQ_OK;
}

// The staged variant needs 16-byte aligned row segments of whole 16-byte multiples: always true for packed
// IQ3_S and Q4_K (144-byte blocks), for IQ4_XS (136-byte blocks) only when K is a multiple of 1024.
template <int KIND, int M, int RS, bool DUMP = false>
static int launch_gemv(const GemvArgs& a, int sm_count, int max_smem, cudaStream_t st) {
  constexpr bool can = KIND == KIND_IQ3S_PACKED || KIND == KIND_Q4K || KIND == KIND_IQ4XS;
  if constexpr (can && !DUMP) {
    if (!a.force_direct && (KIND != KIND_IQ4XS || a.k % 1024 == 0)) return launch_gemv_t<KIND, M, RS, DUMP, true>(a, sm_count, max_smem, st);
  }
  return launch_gemv_t<KIND, M, RS, DUMP, false>(a, sm_count, max_smem, st);
}

template <int KIND, int RS>
static int launch_gemv_m(int m, const GemvArgs& a, int sm_count, int max_smem, cudaStream_t st) {
  switch (m) {
    case 1: return launch_gemv<KIND, 1, RS>(a, sm_count, max_smem, st);
    case 2: return launch_gemv<KIND, 2, RS>(a, sm_count, max_smem, st);
    case 3: return launch_gemv<KIND, 3, RS>(a, sm_count, max_smem, st);
    case 4: return launch_gemv<KIND, 4, RS>(a, sm_count, max_smem, st);
    case 5: return launch_gemv<KIND, 5, RS>(a, sm_count, max_smem, st);
    case 6: return launch_gemv<KIND, 6, RS>(a, sm_count, max_smem, st);
    case 7: return launch_gemv<KIND, 7, RS>(a, sm_count, max_smem, st);
    case 8: return launch_gemv<KIND, 8, RS>(a, sm_count, max_smem, st);
    default: return GSQ_ERR_UNSUPPORTED;
  }
}

// gsq_mmv.cu: the tensor-core kernel for 1..48 rows
bool mmv_applies(int ggml_type, int packed, int64_t rows, int64_t m);
bool mmv_early_trigger();
int mmv_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* xq, int x_layout,
             int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
             const gsq_peer_reduce* pr = nullptr);

static int gemv_host_dp4a(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_q8,
                          int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
                          int dump_m0);

// gsq_gemv_f1.cu
bool gemv_f1_applies(int ggml_type);
int gemv_f1_group(int ggml_type);
int gemv_f1_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, const void* x_q8, int64_t m, int64_t k,
                 void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump, int dump_m0);

static int gemv_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_q8,
                     int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
                     int dump_m0) {
  if (m == 0 || rows == 0) return GSQ_OK;
  if (gemv_f1_applies(ggml_type)) {
    // the low-bit types: their own dp4a kernel, eight activation rows per launch
    if (packed || m < 0 || m > 48 || !y || !x_q8 || k <= 0 || k % 32 != 0) return GSQ_ERR_UNSUPPORTED;
    if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
    const int64_t ysz = y_dtype == GSQ_F32 ? 4 : 2;
    for (int64_t i = 0; i < m; i += 8) {
      const int64_t c = m - i < 8 ? m - i : 8;
      const int rc = gemv_f1_host(w, row_bytes, rows, ggml_type, (const uint8_t*)x_q8 + i * (k / 32) * 36, c, k,
                                  (uint8_t*)y + i * y_row_stride * ysz, y_dtype, y_row_stride, stream, dump, dump_m0 + (int)i);
      if (rc != GSQ_OK) return rc;
    }
    return GSQ_OK;
  }
  if (mmv_applies(ggml_type, packed, rows, m)) {
    int* d = dump ? dump + (int64_t)dump_m0 * rows * (k / 32) : nullptr;
    const int rc = mmv_host(w, row_bytes, rows, ggml_type, packed, x_q8, 0, m, k, y, y_dtype, y_row_stride, stream, d);
    if (rc != 1000) return rc;  // 1000: the shape does not fit that kernel
  }
  // repacked Q6_K is read by the small-batch tensor-core kernel only
  if (ggml_type == GSQ_TYPE_Q6_K && packed) return m > 48 ? GSQ_ERR_UNSUPPORTED : GSQ_ERR_TOO_LARGE;
  if (m > 8 && m <= 48 && y && x_q8 && k > 0 && k % 32 == 0 &&
      (y_dtype == GSQ_F32 || y_dtype == GSQ_F16 || y_dtype == GSQ_BF16)) {
    // Row counts only the small-batch kernel takes in one launch, on a shape it declined (its staging area does
    // not fit): the dp4a kernel below, eight rows per launch, so that every count up to
    // gsq_mul_mat_vec_max_rows() is served whatever the shape.
    const int64_t ysz = y_dtype == GSQ_F32 ? 4 : 2;
    for (int64_t i = 0; i < m; i += 8) {
      const int64_t c = m - i < 8 ? m - i : 8;
      int* d = dump ? dump + (int64_t)(dump_m0 + i) * rows * (k / 32) : nullptr;
      if (d) return GSQ_ERR_UNSUPPORTED;  // the dump instantiation takes one row per launch (gsq_debug_block_sums)
      const int rc = gemv_host_dp4a(w, row_bytes, rows, ggml_type, packed, (const uint8_t*)x_q8 + i * (k / 32) * 36, c, k,
                                    (uint8_t*)y + i * y_row_stride * ysz, y_dtype, y_row_stride, stream, nullptr, 0);
      if (rc != GSQ_OK) return rc;
    }
    return GSQ_OK;
  }
  return gemv_host_dp4a(w, row_bytes, rows, ggml_type, packed, x_q8, m, k, y, y_dtype, y_row_stride, stream, dump, dump_m0);
}

// The dp4a kernel proper: 1..8 activation rows.
static int gemv_host_dp4a(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_q8,
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
  GemvArgs a;
  a.w = (const uint8_t*)w;
  a.row_bytes = row_bytes;
  a.nrows = (int)rows;
  a.k = (int)k;
  a.xq8 = (const uint8_t*)x_q8;
  a.y = y;
  a.y_dtype = y_dtype;
  a.ldy = y_row_stride;
  a.ntiles = (int)((rows + tile_rows - 1) / tile_rows);
  a.nrec = (nsb + rec_sb - 1) / rec_sb;
  a.tiles_base = a.tiles_extra = a.tiles_round = 0;
  a.dump = dump;
  a.dump_m0 = dump_m0;
  a.stage_shift = 0;
  a.force_direct = g_force_direct;
  a.early = mmv_early_trigger() ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = di.sm_count, smem = di.max_smem_optin;

  if (dump) {  // debug build of the same kernel, one activation row per launch
    if (m != 1) return GSQ_ERR_UNSUPPORTED;
    switch (kind) {
      case KIND_IQ3S_PACKED: return launch_gemv<KIND_IQ3S_PACKED, 1, 7, true>(a, sms, smem, st);
      case KIND_IQ3S_RAW: return launch_gemv<KIND_IQ3S_RAW, 1, 7, true>(a, sms, smem, st);
      case KIND_Q4K: return launch_gemv<KIND_Q4K, 1, 7, true>(a, sms, smem, st);
      case KIND_IQ4XS: return launch_gemv<KIND_IQ4XS, 1, 7, true>(a, sms, smem, st);
      default: return launch_gemv<KIND_Q6K, 1, 7, true>(a, sms, smem, st);
    }
  }
  switch (kind) {
    case KIND_IQ3S_PACKED: return launch_gemv_m<KIND_IQ3S_PACKED, 7>((int)m, a, sms, smem, st);
    case KIND_IQ3S_RAW: return launch_gemv_m<KIND_IQ3S_RAW, 7>((int)m, a, sms, smem, st);
    case KIND_Q4K: return launch_gemv_m<KIND_Q4K, 7>((int)m, a, sms, smem, st);
    case KIND_IQ4XS: return launch_gemv_m<KIND_IQ4XS, 7>((int)m, a, sms, smem, st);
    default: return launch_gemv_m<KIND_Q6K, 7>((int)m, a, sms, smem, st);
  }
}

}  // namespace gsq

extern "C" int gsq_mul_mat_vec_q8(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                                  const void* x_q8, int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride,
                                  void* stream) {
  return gsq::gemv_host(w, row_bytes, rows, ggml_type, packed, x_q8, m, k, y, y_dtype, y_row_stride, stream, nullptr, 0);
}

extern "C" int gsq_debug_force_direct_loads(int on) {
  const int old = gsq::g_force_direct;
  gsq::g_force_direct = on ? 1 : 0;
  return old;
}

extern "C" int gsq_debug_force_cluster_size(int cs) {
  const int old = gsq::g_force_cluster;
  gsq::g_force_cluster = (cs == 1 || cs == 2 || cs == 4) ? cs : 0;
  return old;
}

namespace gsq {
int gemm_error_flag(int* flag);  // gsq_gemm.cu
}

extern "C" int gsq_device_error_flag(int* flag) {
  if (!flag) return GSQ_ERR_UNSUPPORTED;
  int a = 0, b = 0;
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(&a, gsq::g_gemv_error, sizeof(int)));
  const int rc = gsq::gemm_error_flag(&b);
  if (rc != GSQ_OK) return rc;
  *flag = a | b;
  return GSQ_OK;
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
