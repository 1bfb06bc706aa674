// Register-operand int8 tensor-core product for 1..48 activation rows over GGUF superblocks (sm_100a).
//
// Serves, behind gsq_mul_mat_vec_q8 and gsq_mul_mat_q8, the row counts at which the product is a stream of
// W with a little arithmetic per byte: the reference's owned 1..8-row kernels (lcpp_owned_k4.cu:116-234,
// lcpp_owned_iq3_mma.cu:483-600), its 9..64-row kernel (lcpp_owned_mma_k.cu) and the small-batch end of its
// MMQ (csrc/lcpp/ggml/src/ggml-cuda/mmq.cuh). The per-slice int32 sums are exact and each slice's term is
// d_w * scale * d_x * sum (- dmin * min * sum of the slice's activation quants for Q4_K); only the fp32 order
// in which a row's terms are added differs from the reference (fixed: results repeat run to run).
//
// Why not the shared-memory / tensor-memory pipeline of gsq_gemm.cu here: below about 64 tokens the tensor
// core is idle either way and the cost is decoding W. With mma.sync the decoded weights are the A fragment,
// in registers, so a warp works alone: no decoded tile in shared memory, no block-wide barrier, no drain of
// tensor memory.
//
//   * A record is 16 weight rows x one 256-value superblock. Lane (g = lane / 4, t = lane % 4) holds rows g
//     and g + 8 and, of every 32-value slice, the 4-value words 2t and 2t + 1 (Q4_K, IQ3_S) or word t of each
//     half (IQ4_XS): exactly its share of the m16n8k32 A fragment. The k index inside a slice is permuted the
//     same way on the activation side, which an integer sum does not see.
//   * A cluster of 1, 2, 4 or 8 CTAs owns a contiguous range of 16-row tiles; its CTAs split K. Each CTA first
//     stages its K range of the activations in shared memory, in fragment order and with the scales as fp32
//     (from block_q8_1, 36 bytes, for the vec ops; from block_q8_1_mmq, 144 bytes, [K/128][M], for the ops that
//     quantise for themselves). Columns past M are zeros. The cluster size is the one with the least estimated
//     time among those whose staging area fits.
//   * The records (tile, superblock) of a CTA, in memory order, are cut into equal contiguous chunks, one per
//     warp, so every warp streams the same number of bytes whatever the shape. A warp reads a record with
//     128-bit no-allocate loads, one record ahead of the arithmetic; there is no block-wide barrier in the loop.
//   * A tile a warp covers whole goes straight to the CTA's tile sums; the tile a chunk starts inside and the
//     one it ends inside are parked and added in warp order after one block barrier. After one cluster barrier
//     the CTAs' tile sums (one per K part) are added in rank order through distributed shared memory and stored
//     in Y's dtype. No atomics, no global scratch, the same order every run.
#include <cooperative_groups.h>

#include <cstdio>

#include "gsq_common.cuh"
#include "gsq_tables.h"

namespace cg = cooperative_groups;

namespace gsq {

enum { MK_Q4K = 0, MK_IQ3S = 1, MK_IQ4XS = 2, MK_Q6K = 3 };
enum { XL_Q81 = 0, XL_MMQ = 1 };

constexpr int MMV_WARPS = 16;
constexpr int MMV_THREADS = MMV_WARPS * 32;
constexpr int MMV_TR = 16;  // rows per tile

struct MmvArgs {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;
  int k;
  const uint8_t* xq;
  int m;
  void* y;
  int y_dtype;
  int64_t ldy;
  int ntiles;
  int tiles_base;    // tiles per cluster: the first tiles_extra clusters own tiles_base + 1
  int tiles_extra;
  int tiles_round;   // tiles a cluster takes per round
  int share_cap;     // most tiles of a round one CTA owns (ceil(tiles_round / cluster size))
  int gather_bufs;   // 1: a single round; 2: rounds alternate between two gather areas
  int aligned;       // 1: a warp's chunk is whole tiles (no parked segments, no room reserved for them)
  int pf_first;      // records of its chunk a warp requests from L2 before the activations are staged
  int early;         // let the next kernel of a programmatic-launch chain start its prologue while this one runs
  int xcap_kb;       // 32-value blocks of activations the shared-memory staging area holds per column
  int* dump;         // debug: int32 slice sums [m][nrows][k / 32]
  // fast_div_inv of: 16-byte granules and 36-byte blocks per staged column, for a CTA with nsr_lo superblocks
  // ([0]) and with nsr_lo + 1 ([1]: K does not split evenly); 16-byte pieces per row of block_q8_1_mmq blocks
  int nsr_lo;
  uint32_t inv_gpc[2], inv_nkb[2], inv_per;
  unsigned long long* prof;  // debug: per CTA 8 time stamps (ns) at the phase boundaries
  // Sum over GPUs of the partial results of a K-sharded product, inside this kernel (pr_world > 1; see the end of
  // mmv_kernel): every rank's slot area [2][world][pr_slot_bytes] and flag area [world], the same offsets on every
  // GPU (peer pointers; entry pr_rank is this GPU's own), and this rank's call counter + two tickets.
  void* const* pr_slots;
  uint32_t* const* pr_flags;
  uint32_t* pr_state;
  int pr_rank, pr_world;
  int64_t pr_slot_bytes;
};

__device__ int g_mmv_peer_error = 0;

__device__ __forceinline__ void mmv_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t mmv_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// one element of a partial result in another rank's slot of this GPU's memory: never from L1 (a peer wrote it)
__device__ __forceinline__ float mmv_load_partial(const void* base, int y_dtype, int64_t idx) {
  if (y_dtype == GSQ_F32) return __ldcv(reinterpret_cast<const float*>(base) + idx);
  const unsigned short b = __ldcv(reinterpret_cast<const unsigned short*>(base) + idx);
  return y_dtype == GSQ_F16 ? __half2float(__ushort_as_half(b)) : __uint_as_float((uint32_t)b << 16);
}

__device__ __forceinline__ void mmv_stamp(const MmvArgs& a, int phase) {
  if (a.prof && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.prof[(size_t)blockIdx.x * 8 + phase] = t;
  }
}

constexpr int MAGIC = 0x4B400000;          // bit pattern of 1.5 * 2^23
constexpr float MAGIC_F = 12582912.0f;

__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t vmul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t vadd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t vfma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// (a & b) | c in one logic instruction
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t mprmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// D = A (16 x 32, int8, row) * B (32 x 8, int8, col) + C, all four accumulators starting at `init`
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int init) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(init));
}

// For IQ3_S from two column groups on, and for IQ4_XS always, the integer sub-scale is applied on the floating-point
// side: the tensor-core instruction accumulates onto the bit pattern of 1.5 * 2^23, so its outputs, read as floats, are
// 1.5 * 2^23 + sum (|sum| < 2^22), already the two packed pairs the fp32x2 instructions want. Per slice and column
// group 4 packed instructions (see scale_acc) instead of 4 integer multiply-adds, their moves into pairs and 6
// packed instructions.
constexpr bool mmv_float_scale(int ntl) { return ntl >= 2; }

__device__ __forceinline__ void scale_acc(const int (&c)[4], uint64_t dv2, uint64_t ds0, uint64_t ds1, uint64_t nm0,
                                          uint64_t nm1, uint64_t& a0, uint64_t& a1) {
  // c holds the bit patterns of 1.5 * 2^23 + sum. (1.5 * 2^23 + sum) * ds - 1.5 * 2^23 * ds in one fused operation is
  // the correctly rounded sum * ds: ds = d * sub-scale has at most 17 significant bits, so the subtrahend nm =
  // -1.5 * 2^23 * ds is exact. Two packed operations per pair of columns.
  const uint64_t t01 = vfma2(pk2(__int_as_float(c[0]), __int_as_float(c[1])), ds0, nm0);
  const uint64_t t23 = vfma2(pk2(__int_as_float(c[2]), __int_as_float(c[3])), ds1, nm1);
  a0 = vfma2(t01, dv2, a0);
  a1 = vfma2(t23, dv2, a1);
}

template <bool DUMP>
__device__ __forceinline__ void dump_c(const MmvArgs& ar, const int (&c)[4], int bias, int row0, int lane, int j, int kb) {
  if constexpr (DUMP) {
    const int g = lane >> 2, t = lane & 3, col0 = 8 * j + 2 * t, nb32 = ar.k >> 5;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = row0 + g + 8 * (e >> 1), col = col0 + (e & 1);
      if (row < ar.nrows && col < ar.m) ar.dump[((int64_t)col * ar.nrows + row) * nb32 + kb] = c[e] - bias;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Activations: staged once per CTA in shared memory for the CTA's K range, in the order the fragments want:
//   quants  [column][kb][32 bytes]   lane (g, t) reads words 2t, 2t + 1 (or t, t + 4) of column 8j + g; a column is
//                                    padded by 32 bytes so that the 8 columns of a read fall on different banks
//   d       [kb][column] float       lane reads columns 8j + 2t, 8j + 2t + 1 (its accumulator columns)
//   sum     [kb][column] float       Q4_K only: what multiplies -dmin * min
// Columns past M are zeros. kb counts 32-value blocks from the start of the CTA's K range.

struct XSmem {
  const uint8_t* q;
  const float* d;
  const float* s;
  int q8;  // bytes between quant columns 8 apart
};

// bytes of one staged quant column
__host__ __device__ constexpr int mmv_xq_col_bytes(int nkb_cap) { return nkb_cap * 32 + 32; }

// i / d for 0 <= i * d < 2^32, with inv = fast_div_inv(d) = ceil(2^32 / d), or 0 for d = 1 (2^32 does not fit)
__host__ __device__ inline uint32_t fast_div_inv(int d) {
  return d <= 1 ? 0u : (uint32_t)((0x100000000ull + (uint32_t)d - 1) / (uint32_t)d);
}
__device__ __forceinline__ int fast_div(int i, uint32_t inv) { return inv ? (int)__umulhi((uint32_t)i, inv) : i; }

// columns m..MC-1 of the staging area: zeros
template <int MC, bool DS>
__device__ __forceinline__ void stage_x_pad(int m, int nkb, int colb, uint8_t* xq, float* xd, float* xs, int tid) {
  const int pad = MC - m;
  for (int i = tid; i < nkb * pad; i += MMV_THREADS) {
    const int kb = i / pad, c = m + (i - kb * pad);
    uint4* dst = reinterpret_cast<uint4*>(xq + c * colb + kb * 32);
    dst[0] = make_uint4(0u, 0u, 0u, 0u);
    dst[1] = make_uint4(0u, 0u, 0u, 0u);
    xd[kb * MC + c] = 0.0f;
    if (DS) xs[kb * MC + c] = 0.0f;
  }
}

// block_q8_1 source (36-byte blocks, [column][K/32]): sum = d * (integer sum of the block's quants), as the
// reference's MMVQ and owned vec kernels form the min term. The CTA's share of a column is one run of whole
// 16-byte granules (K is a multiple of 128); every granule is loaded exactly once, by consecutive threads, and
// its four words go where their position in the 9-word blocks says: word 0 of a block is (d, sum), the other
// eight are quants. All 148 CTAs read the same few KB at the same time, so requests per byte are what counts.
// The activations are read with ld.global.cg (L2, never L1): each granule is needed once per CTA, and a kernel that may
// be resident while its predecessors still run must not meet lines they left in this SM's L1.
// slot of quant word w in a staged 32-byte block. PERM: words (t, t + 4) side by side for the kinds whose 4-byte
// weight word holds values 4t..4t+3 in its low and 16+4t..16+4t+3 in its high nibbles (IQ4_XS).
template <bool PERM>
__device__ __forceinline__ int x_slot(int w) { return PERM ? ((w & 3) << 1) | (w >> 2) : w; }

template <int MC, bool DS, bool PERM, typename AfterIssue>
__device__ __forceinline__ void stage_x_q81(const MmvArgs& a, int kb0, int nkb, int colb, uint8_t* xq, float* xd, float* xs,
                                            int tid, AfterIssue after_issue) {
  const int nb32 = a.k >> 5;
  const int gpc = (nkb * 9) >> 2;   // granules per column
  const int total = gpc * a.m;
  const int which = nkb == a.nsr_lo * 8 ? 0 : 1;
  const uint32_t inv = which ? a.inv_gpc[1] : a.inv_gpc[0];
  const uint32_t inv_nkb = which ? a.inv_nkb[1] : a.inv_nkb[0];
  constexpr int U = 4;
  for (int i0 = tid; i0 < total || i0 == tid; i0 += U * MMV_THREADS) {
    uint4 v[U];
    int col[U], gi[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = min(i0 + u * MMV_THREADS, total - 1);
      col[u] = fast_div(i, inv);
      gi[u] = i - col[u] * gpc;
      v[u] = __ldcg(reinterpret_cast<const uint4*>(a.xq + ((int64_t)col[u] * nb32 + kb0) * 36) + gi[u]);
    }
    if (i0 == tid) {
      after_issue();
      mmv_stamp(a, 6);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i0 + u * MMV_THREADS < total) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int wi = 4 * gi[u] + e, kb = wi / 9, pos = wi - kb * 9;
          if (pos == 0) {
            xd[kb * MC + col[u]] = h2f(w[e]);
          } else {
            *reinterpret_cast<uint32_t*>(xq + col[u] * colb + kb * 32 + x_slot<PERM>(pos - 1) * 4) = w[e];
          }
        }
      }
    }
  }
  mmv_stamp(a, 7);
  stage_x_pad<MC, DS>(a.m, nkb, colb, xq, xd, xs, tid);
  if (DS) {
    __syncthreads();
    for (int i = tid; i < nkb * a.m; i += MMV_THREADS) {
      const int col = fast_div(i, inv_nkb), kb = i - col * nkb;
      const uint4* q = reinterpret_cast<const uint4*>(xq + col * colb + kb * 32);
      const uint4 lo = q[0], hi = q[1];
      int sum = dp4a(0x01010101, (int)lo.x, 0);
      sum = dp4a(0x01010101, (int)lo.y, sum);
      sum = dp4a(0x01010101, (int)lo.z, sum);
      sum = dp4a(0x01010101, (int)lo.w, sum);
      sum = dp4a(0x01010101, (int)hi.x, sum);
      sum = dp4a(0x01010101, (int)hi.y, sum);
      sum = dp4a(0x01010101, (int)hi.z, sum);
      sum = dp4a(0x01010101, (int)hi.w, sum);
      xs[kb * MC + col] = xd[kb * MC + col] * (float)sum;
    }
  }
}

// block_q8_1_mmq source (144-byte blocks, [K/128][column]: 16 scale bytes = 4 x half2(d, sum) (DS) or 4 x float
// d, then 128 int8): the stored sums are used as they are, as the reference's MMQ does. The CTA's share is one
// contiguous run of 16-byte pieces, 9 per block.
template <int MC, bool DS, bool PERM, typename AfterIssue>
__device__ __forceinline__ void stage_x_mmq(const MmvArgs& a, int kb0, int nkb, int colb, uint8_t* xq, float* xd, float* xs,
                                            int tid, AfterIssue after_issue) {
  const int per = a.m * 9, total = (nkb >> 2) * per;
  const uint32_t inv = a.inv_per;
  const uint4* src = reinterpret_cast<const uint4*>(a.xq + (int64_t)(kb0 >> 2) * a.m * 144);
  for (int i0 = tid; i0 < total || i0 == tid; i0 += 8 * MMV_THREADS) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcg(src + min(i0 + u * MMV_THREADS, total - 1));
    if (i0 == tid) after_issue();
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * MMV_THREADS;
      if (i < total) {
        const int b = fast_div(i, inv), r = i - b * per, col = r / 9, part = r - col * 9;
        if (part == 0) {
          const uint32_t sc[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (DS) {
              xd[(4 * b + q) * MC + col] = h2f(sc[q]);
              xs[(4 * b + q) * MC + col] = h2f(sc[q] >> 16);
            } else {
              xd[(4 * b + q) * MC + col] = __uint_as_float(sc[q]);
            }
          }
        } else {
          const int kb = 4 * b + ((part - 1) >> 1);
          uint8_t* dst = xq + col * colb + kb * 32;
          if (PERM) {
            const int w0 = ((part - 1) & 1) * 4;
            *reinterpret_cast<uint32_t*>(dst + x_slot<true>(w0) * 4) = v[u].x;
            *reinterpret_cast<uint32_t*>(dst + x_slot<true>(w0 + 1) * 4) = v[u].y;
            *reinterpret_cast<uint32_t*>(dst + x_slot<true>(w0 + 2) * 4) = v[u].z;
            *reinterpret_cast<uint32_t*>(dst + x_slot<true>(w0 + 3) * 4) = v[u].w;
          } else {
            *reinterpret_cast<uint4*>(dst + ((part - 1) & 1) * 16) = v[u];
          }
        }
      }
    }
  }
  stage_x_pad<MC, DS>(a.m, nkb, colb, xq, xd, xs, tid);
}

// ---------------------------------------------------------------------------------------------
// Q4_K

struct RecQ4K {
  uint4 hdr[2];     // rows g, g + 8: d, dmin, 12 scale bytes
  uint2 q[2][4];    // [row][64-value group p]: qs words 2t, 2t + 1 of the group's 32 bytes
  __device__ __forceinline__ void load(const MmvArgs& a, int row0, int sb, int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = min(row0 + g + 8 * h, a.nrows - 1);
      const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 144;
      hdr[h] = ldg_stream_v4(b);
#pragma unroll
      for (int p = 0; p < 4; ++p) q[h][p] = ldg_stream_v2(b + 16 + 32 * p + 8 * t);
    }
  }
  // ask L2 for a record without waiting for it: lane = (row, first / last byte of the row's 144-byte block,
  // which spans two 128-byte lines)
  static __device__ __forceinline__ void prefetch(const MmvArgs& a, int row0, int sb, int lane) {
    const int r = min(row0 + (lane >> 1), a.nrows - 1);
    const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 144 + (lane & 1) * 143;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(b));
  }
};

// float of byte `byte` of `word`: the byte lands in the mantissa of 2^23, which is then subtracted (exact)
__device__ __forceinline__ float byte_float(uint32_t word, int byte) {
  return __uint_as_float(mprmt(word, 0x4B000000u, 0x7650u | (uint32_t)byte)) - 8388608.0f;
}

// xl: this lane's view of the staged activations of the record's superblock: quants at xl.q + j * xl.q8 + 32 s,
// scales of its two accumulator columns at xl.d + s * MC + 8 j.
template <int NTL, bool DUMP>
__device__ __forceinline__ void process(const RecQ4K& r, const MmvArgs& ar, int row0, int sb, int lane, const XSmem& xl,
                                        const uint8_t*, uint64_t (&acc)[NTL][2]) {
  constexpr int MC = 8 * NTL;
  constexpr bool DEFER = NTL <= 2;  // keep the record's sums unscaled by d / dmin until its end (more registers)
  const int g = lane >> 2, t = lane & 3;
  (void)g; (void)t;
  // the 8 six-bit scales and mins of each row as bytes: [h][0] = slices 0..3, [h][1] = slices 4..7
  uint32_t scw[2][2], mnw[2][2];
  float d[2], ndm[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t A = r.hdr[h].y, B = r.hdr[h].z, C = r.hdr[h].w;
    scw[h][0] = A & 0x3F3F3F3Fu;
    mnw[h][0] = B & 0x3F3F3F3Fu;
    scw[h][1] = (C & 0x0F0F0F0Fu) | ((A >> 2) & 0x30303030u);
    mnw[h][1] = ((C >> 4) & 0x0F0F0F0Fu) | ((B >> 2) & 0x30303030u);
    d[h] = h2f(r.hdr[h].x);
    ndm[h] = -h2f(r.hdr[h].x >> 16);
  }
  const uint64_t nm2 = pk2(-MAGIC_F, -MAGIC_F);
  const uint64_t d02 = pk2(d[0], d[0]), d12 = pk2(d[1], d[1]);
  uint64_t tt[NTL][2], uu[NTL][2];
  if constexpr (DEFER) {
#pragma unroll
    for (int j = 0; j < NTL; ++j) tt[j][0] = tt[j][1] = uu[j][0] = uu[j][1] = 0ull;
  }
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const int p = s >> 1;
    // a0..a3: (row g, word 2t) (g + 8, 2t) (g, 2t + 1) (g + 8, 2t + 1); odd slices are the high nibbles
    const uint32_t w[4] = {r.q[0][p].x, r.q[1][p].x, r.q[0][p].y, r.q[1][p].y};
    uint32_t a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = ((s & 1) ? (w[i] >> 4) : w[i]) & 0x0F0F0F0Fu;
    float m0 = byte_float(mnw[0][s >> 2], s & 3), m1 = byte_float(mnw[1][s >> 2], s & 3);
    if constexpr (!DEFER) {
      m0 *= ndm[0];
      m1 *= ndm[1];
    }
    const uint64_t m02 = pk2(m0, m0), m12 = pk2(m1, m1);
    if constexpr (NTL == 1) {
      // one column group: the sub-scale as an integer multiply-add onto the magic pattern (measured faster here)
      const int sc0 = (int)((scw[0][s >> 2] >> (8 * (s & 3))) & 0xFFu), sc1 = (int)((scw[1][s >> 2] >> (8 * (s & 3))) & 0xFFu);
      const uint2 b = *reinterpret_cast<const uint2*>(xl.q + s * 32);
      const uint64_t dv2 = *reinterpret_cast<const uint64_t*>(xl.d + s * MC);
      const uint64_t xs2 = *reinterpret_cast<const uint64_t*>(xl.s + s * MC);
      int c[4];
      mma_s8(c, a, b.x, b.y, 0);
      dump_c<DUMP>(ar, c, 0, row0, lane, 0, sb * 8 + s);
      // |c * sc| <= 32 * 15 * 127 * 63 < 2^22
      const uint64_t f01 = vadd2(pk2(__int_as_float(c[0] * sc0 + MAGIC), __int_as_float(c[1] * sc0 + MAGIC)), nm2);
      const uint64_t f23 = vadd2(pk2(__int_as_float(c[2] * sc1 + MAGIC), __int_as_float(c[3] * sc1 + MAGIC)), nm2);
      tt[0][0] = vfma2(f01, dv2, tt[0][0]);
      tt[0][1] = vfma2(f23, dv2, tt[0][1]);
      uu[0][0] = vfma2(m02, xs2, uu[0][0]);
      uu[0][1] = vfma2(m12, xs2, uu[0][1]);
    } else {
      // several column groups: the sub-scale on the floating-point side, two packed operations per pair of columns
      // (scale_acc); the multiplier (sc, or d * sc where the record's sums are not deferred) has at most 17
      // significant bits, so -1.5 * 2^23 times it is exact
      float f0 = byte_float(scw[0][s >> 2], s & 3), f1 = byte_float(scw[1][s >> 2], s & 3);
      if constexpr (!DEFER) {
        f0 *= d[0];
        f1 *= d[1];
      }
      const uint64_t ds0 = pk2(f0, f0), ds1 = pk2(f1, f1);
      const float g0 = -MAGIC_F * f0, g1 = -MAGIC_F * f1;
      const uint64_t nmA = pk2(g0, g0), nmB = pk2(g1, g1);
#pragma unroll
      for (int j = 0; j < NTL; ++j) {
        const uint2 b = *reinterpret_cast<const uint2*>(xl.q + j * xl.q8 + s * 32);
        const uint64_t dv2 = *reinterpret_cast<const uint64_t*>(xl.d + s * MC + 8 * j);
        const uint64_t xs2 = *reinterpret_cast<const uint64_t*>(xl.s + s * MC + 8 * j);
        int c[4];
        mma_s8(c, a, b.x, b.y, MAGIC);
        dump_c<DUMP>(ar, c, MAGIC, row0, lane, j, sb * 8 + s);
        if constexpr (DEFER) {
          scale_acc(c, dv2, ds0, ds1, nmA, nmB, tt[j][0], tt[j][1]);
          uu[j][0] = vfma2(m02, xs2, uu[j][0]);
          uu[j][1] = vfma2(m12, xs2, uu[j][1]);
        } else {
          scale_acc(c, dv2, ds0, ds1, nmA, nmB, acc[j][0], acc[j][1]);
          acc[j][0] = vfma2(m02, xs2, acc[j][0]);
          acc[j][1] = vfma2(m12, xs2, acc[j][1]);
        }
      }
    }
  }
  if constexpr (DEFER) {
    const uint64_t n02 = pk2(ndm[0], ndm[0]), n12 = pk2(ndm[1], ndm[1]);
#pragma unroll
    for (int j = 0; j < NTL; ++j) {
      acc[j][0] = vfma2(n02, uu[j][0], vfma2(d02, tt[j][0], acc[j][0]));
      acc[j][1] = vfma2(n12, uu[j][1], vfma2(d12, tt[j][1], acc[j][1]));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// IQ3_S in the fragment-ordered layout of gsq_iq3s_repack (see gsq_repack.cu): per lane 9 words of 9-bit
// codebook indices (field f = 4 s + 2 h + e at bit 9 f), 4 words of sign bits, the sub-scale nibbles and d of
// rows g, g + 8. The codebook copy in shared memory holds, per entry and per lane-mod-16 replica, the pair
// (g, -g) of packed int8x4 words (entry i of replica r at byte 128 i + 8 r): a field's signed word is one
// 64-bit load and one byte permute whose selector comes from the sign bits.

__device__ const uint32_t g_iq3s_grid_mmv[512] = GSQ_IQ3S_GRID_INIT;

// 16 replicas (64 KB) keep the lookups free of bank conflicts; from 25 activation rows on the staged activations
// need the room and 8 replicas (32 KB, two lanes per replica) are used
__host__ __device__ constexpr int iq3_replica_shift(int ntl) { return ntl >= 4 ? 3 : 4; }

struct RecIQ3S {
  uint32_t idx[9], sg[4];
  uint2 sc;      // sub-scale nibbles of rows g, g + 8
  uint32_t dd;   // fp16 d of rows g, g + 8
  __device__ __forceinline__ void load(const MmvArgs& a, int row0, int sb, int lane) {
    const uint8_t* p = a.w + (int64_t)row0 * a.row_bytes + (int64_t)sb * 1760;
    const uint4 ia = ldg_stream_v4(p + 16 * lane), ib = ldg_stream_v4(p + 512 + 16 * lane);
    idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
    idx[4] = ib.x; idx[5] = ib.y; idx[6] = ib.z; idx[7] = ib.w;
    idx[8] = ldg_stream_u32(p + 1024 + 4 * lane);
    const uint4 s = ldg_stream_v4(p + 1152 + 16 * lane);
    sg[0] = s.x; sg[1] = s.y; sg[2] = s.z; sg[3] = s.w;
    sc = ldg_stream_v2(p + 1664 + 8 * (lane >> 2));
    dd = ldg_stream_u32(p + 1728 + 4 * (lane >> 2));
  }
  // ask L2 for a record without waiting for it: its 1760 bytes touch at most 15 lines of 128 bytes
  static __device__ __forceinline__ void prefetch(const MmvArgs& a, int row0, int sb, int lane) {
    const uint8_t* p = a.w + (int64_t)row0 * a.row_bytes + (int64_t)sb * 1760;
    if (lane < 15) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + min(128 * lane, 1759)));
  }
};

// RS: log2 of the codebook replicas in shared memory (entry i of replica r at byte (8 << RS) i + 8 r)
template <int F, int RS>
__device__ __forceinline__ uint32_t iq3_field(const RecIQ3S& r, const char* gbase, uint32_t lane_off) {
  constexpr int bit = 9 * F, word = bit >> 5, off = bit & 31, P = 3 + RS;  // the index goes to bits P .. P + 8
  uint32_t t;
  if (off + 9 <= 32) {
    t = off >= P ? r.idx[word] >> (off >= P ? off - P : 0) : r.idx[word] << (off < P ? P - off : 0);
  } else {
    t = __funnelshift_r(r.idx[word], r.idx[word + 1], off - P);
  }
  const uint2 gp = *reinterpret_cast<const uint2*>(gbase + and_or(t, 0x1FFu << P, lane_off));
  constexpr int fl = F & 7, sh = 16 * (fl >> 2) + (fl & 3) - 2;
  const uint32_t sgs = sh >= 0 ? r.sg[F >> 3] >> (sh >= 0 ? sh : 0) : r.sg[F >> 3] << (sh < 0 ? -sh : 0);
  return mprmt(gp.x, gp.y, and_or(sgs, 0x4444u, 0x3210u));
}

template <int S, int NTL, bool DUMP>
__device__ __forceinline__ void iq3_slice(const RecIQ3S& r, const MmvArgs& ar, int row0, int sb, int lane, const XSmem& xl,
                                          const char* gbase, uint32_t lane_off, const uint32_t (&iscw)[2][2],
                                          const uint64_t (&d2)[2], uint64_t (&acc)[NTL][2], uint64_t (&tt)[NTL][2]) {
  constexpr int MC = 8 * NTL;
  constexpr bool DEFER = NTL <= 2;
  uint32_t a[4];
  constexpr int RS = iq3_replica_shift(NTL);
  a[0] = iq3_field<4 * S + 0, RS>(r, gbase, lane_off);   // (row g, group 2t)
  a[1] = iq3_field<4 * S + 2, RS>(r, gbase, lane_off);   // (row g + 8, group 2t)
  a[2] = iq3_field<4 * S + 1, RS>(r, gbase, lane_off);   // (row g, group 2t + 1)
  a[3] = iq3_field<4 * S + 3, RS>(r, gbase, lane_off);   // (row g + 8, group 2t + 1)
  // 2 * nibble + 1 of slice S: byte S / 2 of the even- or odd-slice word
  const uint64_t nm2 = pk2(-MAGIC_F, -MAGIC_F);
  if constexpr (mmv_float_scale(NTL)) {
    float h0, h1;
    upk2(d2[0], h0, h1);
    const float f0 = h0 * byte_float(iscw[0][S & 1], S >> 1);   // d * (2 n + 1), exact
    upk2(d2[1], h0, h1);
    const float f1 = h0 * byte_float(iscw[1][S & 1], S >> 1);
    const uint64_t ds0 = pk2(f0, f0), ds1 = pk2(f1, f1);
    const float g0 = -MAGIC_F * f0, g1 = -MAGIC_F * f1;
    const uint64_t nm0 = pk2(g0, g0), nm1 = pk2(g1, g1);
#pragma unroll
    for (int j = 0; j < NTL; ++j) {
      const uint2 b = *reinterpret_cast<const uint2*>(xl.q + j * xl.q8 + S * 32);
      const uint64_t dv2 = *reinterpret_cast<const uint64_t*>(xl.d + S * MC + 8 * j);
      int c[4];
      mma_s8(c, a, b.x, b.y, MAGIC);
      dump_c<DUMP>(ar, c, MAGIC, row0, lane, j, sb * 8 + S);
      scale_acc(c, dv2, ds0, ds1, nm0, nm1, acc[j][0], acc[j][1]);
    }
  } else {
    const int sc0 = (int)((iscw[0][S & 1] >> (8 * (S >> 1))) & 0xFFu), sc1 = (int)((iscw[1][S & 1] >> (8 * (S >> 1))) & 0xFFu);
#pragma unroll
    for (int j = 0; j < NTL; ++j) {
      const uint2 b = *reinterpret_cast<const uint2*>(xl.q + j * xl.q8 + S * 32);
      const uint64_t dv2 = *reinterpret_cast<const uint64_t*>(xl.d + S * MC + 8 * j);
      int c[4];
      mma_s8(c, a, b.x, b.y, 0);
      dump_c<DUMP>(ar, c, 0, row0, lane, j, sb * 8 + S);
      // |c * (2 n + 1)| <= 32 * 15 * 127 * 31 < 2^22: integer multiply-add onto the magic pattern, read as a float
      const uint64_t f01 = vadd2(pk2(__int_as_float(c[0] * sc0 + MAGIC), __int_as_float(c[1] * sc0 + MAGIC)), nm2);
      const uint64_t f23 = vadd2(pk2(__int_as_float(c[2] * sc1 + MAGIC), __int_as_float(c[3] * sc1 + MAGIC)), nm2);
      tt[j][0] = vfma2(f01, dv2, tt[j][0]);
      tt[j][1] = vfma2(f23, dv2, tt[j][1]);
    }
  }
}

template <int NTL, bool DUMP>
__device__ __forceinline__ void process(const RecIQ3S& r, const MmvArgs& ar, int row0, int sb, int lane, const XSmem& xl,
                                        const uint8_t* grid, uint64_t (&acc)[NTL][2]) {
  constexpr bool DEFER = NTL <= 2;
  const char* gbase = reinterpret_cast<const char*>(grid);
  const uint32_t lane_off = (uint32_t)(lane & ((1 << iq3_replica_shift(NTL)) - 1)) << 3;
  uint32_t iscw[2][2];  // [row half][even / odd slices]: bytes 2 * nibble + 1
  uint64_t d2[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t w = h ? r.sc.y : r.sc.x;
    iscw[h][0] = ((w & 0x0F0F0F0Fu) << 1) | 0x01010101u;
    iscw[h][1] = ((w >> 3) & 0x1E1E1E1Eu) | 0x01010101u;
    const float d = h2f(r.dd >> (16 * h));
    d2[h] = pk2(d, d);
  }
  uint64_t tt[NTL][2];
  if constexpr (DEFER) {
#pragma unroll
    for (int j = 0; j < NTL; ++j) tt[j][0] = tt[j][1] = 0ull;
  }
  iq3_slice<0, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<1, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<2, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<3, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<4, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<5, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<6, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  iq3_slice<7, NTL, DUMP>(r, ar, row0, sb, lane, xl, gbase, lane_off, iscw, d2, acc, tt);
  if constexpr (!mmv_float_scale(NTL)) {
#pragma unroll
    for (int j = 0; j < NTL; ++j) {
      acc[j][0] = vfma2(d2[0], tt[j][0], acc[j][0]);
      acc[j][1] = vfma2(d2[1], tt[j][1], acc[j][1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// IQ4_XS (136-byte blocks as stored: fp16 d, 16 bits of scale high parts, 4 bytes of scale low nibbles, 128
// bytes of 4-bit indices into a 16-entry table). Lane (g, t) takes word t of each 16-byte slice of rows g and
// g + 8: its low nibbles are values 4t..4t+3 (fragment words a0 / a1), its high nibbles 16+4t..16+4t+3 (a2 / a3);
// the activations are staged with words t and t + 4 side by side to match.

__constant__ __align__(16) int8_t c_iq4nl_mmv[16] = GSQ_IQ4NL_VALUES_INIT;

struct RecIQ4XS {
  uint2 hdr[2];
  uint32_t q[2][8];
  __device__ __forceinline__ void load(const MmvArgs& a, int row0, int sb, int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = min(row0 + g + 8 * h, a.nrows - 1);
      const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 136;
      hdr[h] = ldg_stream_v2(b);
#pragma unroll
      for (int s = 0; s < 8; ++s) q[h][s] = __ldg(reinterpret_cast<const uint32_t*>(b + 8 + 16 * s + 4 * t));
    }
  }
  static __device__ __forceinline__ void prefetch(const MmvArgs& a, int row0, int sb, int lane) {
    const int r = min(row0 + (lane >> 1), a.nrows - 1);
    const uint8_t* b = a.w + (int64_t)r * a.row_bytes + (int64_t)sb * 136 + (lane & 1) * 135;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(b));
  }
};

// 8 four-bit indices of v -> the table bytes: lo = entries of the 4 low nibbles, hi = of the 4 high nibbles
__device__ __forceinline__ void iq4_lookup_mmv(uint32_t v, const uint32_t (&tb)[4], uint32_t& lo, uint32_t& hi) {
  const uint32_t s01 = v & 0x7777u, s23 = (v >> 16) & 0x7777u;
  const uint32_t pick01 = 0x3210u | ((v & 0x8888u) >> 1), pick23 = 0x3210u | (((v >> 16) & 0x8888u) >> 1);
  const uint32_t r01 = mprmt(mprmt(tb[0], tb[1], s01), mprmt(tb[2], tb[3], s01), pick01);  // nibbles 0..3 of v
  const uint32_t r23 = mprmt(mprmt(tb[0], tb[1], s23), mprmt(tb[2], tb[3], s23), pick23);  // nibbles 4..7 of v
  lo = mprmt(r01, r23, 0x6420u);
  hi = mprmt(r01, r23, 0x7531u);
}

template <int NTL, bool DUMP>
__device__ __forceinline__ void process(const RecIQ4XS& r, const MmvArgs& ar, int row0, int sb, int lane, const XSmem& xl,
                                        const uint8_t*, uint64_t (&acc)[NTL][2]) {
  constexpr int MC = 8 * NTL;
  const uint32_t* tw = reinterpret_cast<const uint32_t*>(c_iq4nl_mmv);
  const uint32_t tb[4] = {tw[0], tw[1], tw[2], tw[3]};
  uint64_t d2[2];
  uint32_t sh4[2];  // the 2-bit high parts, pre-shifted to bits 4, 5
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float d = h2f(r.hdr[h].x);
    d2[h] = pk2(d, d);
    sh4[h] = (r.hdr[h].x >> 16) << 4;
  }
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    uint32_t a[4];
    iq4_lookup_mmv(r.q[0][s], tb, a[0], a[2]);
    iq4_lookup_mmv(r.q[1][s], tb, a[1], a[3]);
    // 6-bit sub-scale minus 32: low nibble from scales_l, bits 4, 5 from scales_h
    const int sc0 = (int)(((r.hdr[0].y >> (4 * s)) & 0xFu) | ((sh4[0] >> (2 * s)) & 0x30u)) - 32;
    const int sc1 = (int)(((r.hdr[1].y >> (4 * s)) & 0xFu) | ((sh4[1] >> (2 * s)) & 0x30u)) - 32;
    // d * sub-scale, applied on the floating-point side (|sum| <= 32 * 127 * 127 < 2^22)
    float h0, h1;
    upk2(d2[0], h0, h1);
    const float f0 = h0 * (float)sc0;
    upk2(d2[1], h0, h1);
    const float f1 = h0 * (float)sc1;
    const uint64_t ds0 = pk2(f0, f0), ds1 = pk2(f1, f1);
    const float g0 = -MAGIC_F * f0, g1 = -MAGIC_F * f1;
    const uint64_t nm0 = pk2(g0, g0), nm1 = pk2(g1, g1);
#pragma unroll
    for (int j = 0; j < NTL; ++j) {
      const uint2 b = *reinterpret_cast<const uint2*>(xl.q + j * xl.q8 + s * 32);
      const uint64_t dv2 = *reinterpret_cast<const uint64_t*>(xl.d + s * MC + 8 * j);
      int c[4];
      mma_s8(c, a, b.x, b.y, MAGIC);
      dump_c<DUMP>(ar, c, MAGIC, row0, lane, j, sb * 8 + s);
      scale_acc(c, dv2, ds0, ds1, nm0, nm1, acc[j][0], acc[j][1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Q6_K in the fragment-ordered layout of gsq_q6k_repack (see gsq_repack.cu): per lane and row the eight words of low
// nibbles (n, qb, is), the four words of 2-bit high parts (n, is), and per row the 16 int8 sub-scales and d. A
// sub-scale covers 16 values, so the products are m16n8k16 (one per 16-value group G = 8 n + 2 q + is, q = 0..3:
// low nibbles of word (n, q & 1, is) for q < 2, its high nibbles for q >= 2; high parts from bits 2 q, 2 q + 1).
// The two groups of a 32-value slice share the activation scale: their sums are combined as integers
// (sum_a * sc_a + sum_b * sc_b, below 2^24 in magnitude) and converted once.

struct RecQ6K {
  uint4 ql[4];   // [2 h + n]: words (qb, is) = x y z w
  uint4 qh[2];   // [h]: words (n, is)
  uint4 sc[2];   // [h]: 16 int8
  uint32_t dd;   // fp16 d of rows g, g + 8
  __device__ __forceinline__ void load(const MmvArgs& a, int row0, int sb, int lane) {
    const uint8_t* p = a.w + (int64_t)row0 * a.row_bytes + (int64_t)sb * 3360;
    const int g = lane >> 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) ql[i] = ldg_stream_v4(p + 64 * lane + 16 * i);
#pragma unroll
    for (int i = 0; i < 2; ++i) qh[i] = ldg_stream_v4(p + 2048 + 32 * lane + 16 * i);
#pragma unroll
    for (int i = 0; i < 2; ++i) sc[i] = ldg_stream_v4(p + 3072 + 32 * g + 16 * i);
    dd = ldg_stream_u32(p + 3328 + 4 * g);
  }
  static __device__ __forceinline__ void prefetch(const MmvArgs& a, int row0, int sb, int lane) {
    const uint8_t* p = a.w + (int64_t)row0 * a.row_bytes + (int64_t)sb * 3360;
    if (lane < 27) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + min(128 * lane, 3359)));
  }
};

// D = A (16 x 16, int8, row) * B (16 x 8, int8, col), accumulators starting at 0
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ __forceinline__ uint32_t u4_get(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// 4 six-bit values minus 32 as int8: lo = the 4 low nibbles (masked), hf = the high parts at bits 4, 5 of each byte
// with bit 5 already inverted. With bit 5 inverted the byte is x = (v - 32) mod 64 plus, for v < 32, nothing in bits
// 6, 7: adding 6 * (x & 0x20) sets them exactly then (two's complement of a negative value).
__device__ __forceinline__ uint32_t q6_bytes(uint32_t lo, uint32_t hf) {
  const uint32_t x = and_or(hf, 0x30303030u, lo);
  return (x & 0x20202020u) * 6u + x;
}

// int8 byte b of w, sign-extended
__device__ __forceinline__ int sbyte(uint32_t w, int b) {
  return (int)mprmt(w, 0u, 0x8880u | (uint32_t)b | ((uint32_t)b << 4) | ((uint32_t)b << 8) | ((uint32_t)b << 12));
}

template <bool DUMP>
__device__ __forceinline__ void dump_c16(const MmvArgs& ar, const int (&c)[4], int row0, int lane, int j, int group) {
  if constexpr (DUMP) {
    const int g = lane >> 2, t = lane & 3, col0 = 8 * j + 2 * t, nb16 = ar.k >> 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = row0 + g + 8 * (e >> 1), col = col0 + (e & 1);
      if (row < ar.nrows && col < ar.m) ar.dump[((int64_t)col * ar.nrows + row) * nb16 + group] = c[e];
    }
  }
}

template <int NTL, bool DUMP>
__device__ __forceinline__ void process(const RecQ6K& r, const MmvArgs& ar, int row0, int sb, int lane, const XSmem& xl,
                                        const uint8_t*, uint64_t (&acc)[NTL][2]) {
  constexpr int MC = 8 * NTL;
  const int t = lane & 3;
  // the lane's view of the staged quants is set up for words 2t, 2t + 1 of a 32-byte block; here word t of each half
  const uint8_t* xq = xl.q - 4 * t;
  uint64_t tt[NTL][2];
#pragma unroll
  for (int j = 0; j < NTL; ++j) tt[j][0] = tt[j][1] = 0ull;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    // high parts of the two rows for is = 0, 1, the upper bit of every pair inverted once
    uint32_t hf[2][2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      hf[h][0] = u4_get(r.qh[h], 2 * n) ^ 0xAAAAAAAAu;
      hf[h][1] = u4_get(r.qh[h], 2 * n + 1) ^ 0xAAAAAAAAu;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int s = 4 * n + q;   // slice of the superblock: groups 2 s (is = 0) and 2 s + 1 (is = 1)
      uint32_t a[2][2];          // [is][h]
#pragma unroll
      for (int is = 0; is < 2; ++is) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t wl = u4_get(r.ql[2 * h + n], 2 * (q & 1) + is);
          const uint32_t lo = (q < 2 ? wl : wl >> 4) & 0x0F0F0F0Fu;
          const uint32_t hs = q == 0 ? hf[h][is] << 4 : q == 1 ? hf[h][is] << 2 : q == 2 ? hf[h][is] : hf[h][is] >> 2;
          a[is][h] = q6_bytes(lo, hs);
        }
      }
      const int G = 2 * s;
      const int sa0 = sbyte(u4_get(r.sc[0], G >> 2), G & 3), sb0 = sbyte(u4_get(r.sc[0], G >> 2), (G & 3) + 1);
      const int sa1 = sbyte(u4_get(r.sc[1], G >> 2), G & 3), sb1 = sbyte(u4_get(r.sc[1], G >> 2), (G & 3) + 1);
#pragma unroll
      for (int j = 0; j < NTL; ++j) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xq + j * xl.q8 + s * 32);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xq + j * xl.q8 + s * 32 + 16);
        const uint64_t dv2 = *reinterpret_cast<const uint64_t*>(xl.d + s * MC + 8 * j);
        int ca[4], cb[4];
        mma_s8_k16(ca, a[0][0], a[0][1], b0);
        mma_s8_k16(cb, a[1][0], a[1][1], b1);
        dump_c16<DUMP>(ar, ca, row0, lane, j, sb * 16 + G);
        dump_c16<DUMP>(ar, cb, row0, lane, j, sb * 16 + G + 1);
        // |sum * sc| <= 16 * 32 * 127 * 128 per group: the two together stay below 2^24, exact as a float
        const float f0 = (float)(ca[0] * sa0 + cb[0] * sb0), f1 = (float)(ca[1] * sa0 + cb[1] * sb0);
        const float f2 = (float)(ca[2] * sa1 + cb[2] * sb1), f3 = (float)(ca[3] * sa1 + cb[3] * sb1);
        tt[j][0] = vfma2(pk2(f0, f1), dv2, tt[j][0]);
        tt[j][1] = vfma2(pk2(f2, f3), dv2, tt[j][1]);
      }
    }
  }
  const float d0 = h2f(r.dd), d1 = h2f(r.dd >> 16);
  const uint64_t d02 = pk2(d0, d0), d12 = pk2(d1, d1);
#pragma unroll
  for (int j = 0; j < NTL; ++j) {
    acc[j][0] = vfma2(d02, tt[j][0], acc[j][0]);
    acc[j][1] = vfma2(d12, tt[j][1], acc[j][1]);
  }
}

// ---------------------------------------------------------------------------------------------
// The kernel.

template <int KIND>
struct MmvKind;
template <>
struct MmvKind<MK_Q6K> {
  using Rec = RecQ6K;
  static constexpr bool DS = false;
  static constexpr int grid_bytes(int) { return 0; }
  static constexpr bool PERM = false;
};
template <>
struct MmvKind<MK_Q4K> {
  using Rec = RecQ4K;
  static constexpr bool DS = true;       // activations carry sums (for the min term)
  static constexpr int grid_bytes(int) { return 0; }   // codebook copy in shared memory
  static constexpr bool PERM = false;    // staged quant words in the order 0 4 1 5 2 6 3 7
};
template <>
struct MmvKind<MK_IQ3S> {
  using Rec = RecIQ3S;
  static constexpr bool DS = false;
  static constexpr int grid_bytes(int ntl) { return 512 * (8 << iq3_replica_shift(ntl)); }
  static constexpr bool PERM = false;
};
template <>
struct MmvKind<MK_IQ4XS> {
  using Rec = RecIQ4XS;
  static constexpr bool DS = false;
  static constexpr int grid_bytes(int) { return 0; }
  static constexpr bool PERM = true;
};

// bytes of staged activations per 32-value block and padded column
__host__ __device__ constexpr size_t mmv_x_bytes(int cap_kb, int mc, bool ds) {
  return (size_t)mc * mmv_xq_col_bytes(cap_kb) + (size_t)cap_kb * mc * (ds ? 8 : 4);
}

// a warp parks at most two incomplete tile segments per round: the tile its chunk starts inside and the one
// it ends inside (tiles it covers whole go straight to the CTA's tile sums)
__host__ __device__ inline size_t mmv_partial_bytes(int mc) { return (size_t)MMV_WARPS * 2 * MMV_TR * mc * 4; }

// Records per warp in a round of tiles_r tiles of nsr records each: equal chunks (perfect balance, chunks cut
// tiles), or, aligned, whole tiles per warp (nothing to park; used where the parked segments would not fit)
__host__ __device__ inline int mmv_chunk(int tiles_r, int nsr, int aligned) {
  return aligned ? ((tiles_r + MMV_WARPS - 1) / MMV_WARPS) * nsr : (tiles_r * nsr + MMV_WARPS - 1) / MMV_WARPS;
}

// superblocks [first, last) of the K range of CTA `rank` in a cluster of `cs`
__host__ __device__ inline void mmv_k_range(int nsb, int cs, int rank, int* first, int* last) {
  *first = (int)((int64_t)nsb * rank / cs);
  *last = (int)((int64_t)nsb * (rank + 1) / cs);
}

// FUSED: the instantiation that also sums the result over the GPUs (see the end of the kernel); the plain product is
// a separate instantiation so that it carries none of that code or of its registers.
template <int KIND, int NTL, int XL, bool DUMP, bool FUSED = false>
__global__ void __launch_bounds__(MMV_THREADS, 1) mmv_kernel(const MmvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  using Rec = typename MmvKind<KIND>::Rec;
  constexpr bool DS = MmvKind<KIND>::DS;
  constexpr int MC = 8 * NTL;                // padded column count
  constexpr int SEGF = MMV_TR * MC;          // floats per parked tile segment
  cg::cluster_group cluster = cg::this_cluster();
  const int cs = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
  const int cluster_id = (int)blockIdx.x / cs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int nsb = a.k >> 8;
  int sb0, sb1;
  mmv_k_range(nsb, cs, crank, &sb0, &sb1);
  const int nsr = sb1 - sb0;                 // superblocks of this CTA
  const int nkb = nsr * 8;

  constexpr int GRID = MmvKind<KIND>::grid_bytes(NTL);
  const uint8_t* grid = smem;
  float* partial = reinterpret_cast<float*>(smem + GRID);
  // gather area: [buffer][source CTA][owned tile][16][MC]; every CTA of the cluster owns a contiguous share of
  // the round's tiles and receives, through distributed shared memory, each CTA's sums (one K part each) for them
  const size_t part_bytes = a.aligned ? 0 : mmv_partial_bytes(MC);
  float* gath = reinterpret_cast<float*>(smem + GRID + part_bytes);
  const size_t gath_bytes = (size_t)a.gather_bufs * cs * a.share_cap * SEGF * 4;
  uint8_t* xq = smem + GRID + part_bytes + gath_bytes;
  const int colb = mmv_xq_col_bytes(a.xcap_kb);
  float* xd = reinterpret_cast<float*>(xq + (size_t)colb * MC);
  float* xs = xd + (size_t)a.xcap_kb * MC;

  const int tile_begin = cluster_id * a.tiles_base + min(cluster_id, a.tiles_extra);
  const int tile_cnt = a.tiles_base + (cluster_id < a.tiles_extra ? 1 : 0);

  mmv_stamp(a, 0);
  // The warp's first two records are requested from L2 (no register waits on them) ahead of the staging and
  // loaded for real after it.
  int first_tl = 0, first_rec = 0;
  bool have_first = false;
  int first_n = 0;
  {
    const int tiles_r = min(a.tiles_round, tile_cnt);
    const int rr = tiles_r * nsr, c = mmv_chunk(tiles_r, nsr, a.aligned);
    const int idx0 = warp * c, idx1 = min(rr, idx0 + c);
    if (idx0 < idx1) {
      have_first = true;
      first_tl = idx0 / nsr;
      first_rec = idx0 - first_tl * nsr;
      first_n = min(a.pf_first, idx1 - idx0);
    }
  }
  // Everything up to here, the requests to L2 for the warp's first two records and the codebook copy do not
  // depend on the kernel that produced the activations: with programmatic dependent launch they overlap its
  // tail. The wait is a no-op when the launch carries no such dependency.
  {
    int ptl = first_tl, prec = first_rec;
#pragma unroll 1
    for (int u = 0; u < first_n; ++u) {
      Rec::prefetch(a, (tile_begin + ptl) * MMV_TR, sb0 + prec, lane);
      if (++prec == nsr) { prec = 0; ++ptl; }
    }
  }
  if (GRID) {
    // one global load per thread (512 threads, 512 entries), then the replicas of its (g, -g) pair; no byte
    // of the codebook is zero, so ~g + 1 per byte never carries
    const uint32_t gv = g_iq3s_grid_mmv[tid & 511];
    uint4* dst = reinterpret_cast<uint4*>(smem + (tid & 511) * (GRID / 512));
#pragma unroll
    for (int r2 = 0; r2 < GRID / 512 / 16; ++r2) dst[r2] = make_uint4(gv, ~gv + 0x01010101u, gv, ~gv + 0x01010101u);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // fused sum over GPUs: this call's number (the same in every CTA and on every rank) picks the slot pair. Read after
  // the wait: the kernel before this one in a programmatic-launch chain may be the call that publishes it.
  constexpr bool fused = FUSED;
  const uint32_t epoch = fused ? *reinterpret_cast<volatile uint32_t*>(a.pr_state) + 1u : 0u;
  const int64_t push_off = fused ? (int64_t)((epoch & 1u) * a.pr_world + a.pr_rank) * a.pr_slot_bytes : 0;
  auto nothing = []() {};
  if (XL == XL_Q81) {
    stage_x_q81<MC, DS, MmvKind<KIND>::PERM>(a, sb0 * 8, nkb, colb, xq, xd, xs, tid, nothing);
  } else {
    stage_x_mmq<MC, DS, MmvKind<KIND>::PERM>(a, sb0 * 8, nkb, colb, xq, xd, xs, tid, nothing);
  }
  __syncthreads();
  mmv_stamp(a, 1);
  Rec cur;
  if (have_first) cur.load(a, (tile_begin + first_tl) * MMV_TR, sb0 + first_rec, lane);
  XSmem xlane;
  xlane.q = xq + g * colb + 8 * t;
  xlane.q8 = 8 * colb;
  xlane.d = xd + 2 * t;
  xlane.s = xs + 2 * t;

  for (int t0 = 0; t0 < tile_cnt; t0 += a.tiles_round) {
    const int tiles_r = min(a.tiles_round, tile_cnt - t0);
    const int rr = tiles_r * nsr;
    const int c = mmv_chunk(tiles_r, nsr, a.aligned);  // records per warp this round
    const int idx0 = warp * c, idx1 = min(rr, idx0 + c);
    float* mypart = partial + warp * (2 * SEGF);

    if (idx0 < idx1) {
      int tl = idx0 / nsr, rec = idx0 - tl * nsr;
      const int seg_tl = tl;
      if (t0 != 0) cur.load(a, (tile_begin + t0 + tl) * MMV_TR, sb0 + rec, lane);
      uint64_t acc[NTL][2];
#pragma unroll
      for (int j = 0; j < NTL; ++j) acc[j][0] = acc[j][1] = 0ull;
#pragma unroll 1
      for (int idx = idx0; idx < idx1; ++idx) {
        const bool has_next = idx + 1 < idx1;
        const bool wrap = rec + 1 == nsr;
        const int ntl = wrap ? tl + 1 : tl, nrc = wrap ? 0 : rec + 1;
        // Up to 16 columns the next record is loaded into registers while this one is multiplied. Wider than
        // that the accumulators need the registers: the next record is only requested from L2 and loaded after
        // the arithmetic (the other warps of the SM cover the wait; a record then takes ~1000 instructions).
        constexpr bool REGPF = NTL <= 2;
        Rec nxt;
        if (has_next) {
          if constexpr (REGPF) {
            nxt.load(a, (tile_begin + t0 + ntl) * MMV_TR, sb0 + nrc, lane);
          } else {
            Rec::prefetch(a, (tile_begin + t0 + ntl) * MMV_TR, sb0 + nrc, lane);
          }
        }
        XSmem xl;
        xl.q = xlane.q + rec * 256;
        xl.q8 = xlane.q8;
        xl.d = xlane.d + rec * (8 * MC);
        xl.s = xlane.s + rec * (8 * MC);
        process<NTL, DUMP>(cur, a, (tile_begin + t0 + tl) * MMV_TR, sb0 + rec, lane, xl, grid, acc);
        if (!has_next || wrap) {
          // leaving tile tl, [row][column]: a tile this warp covered whole is final for this CTA; otherwise the
          // sums are parked, slot 0 for the tile the chunk started in, slot 1 for the one it ends in
          const bool whole = idx0 <= tl * nsr && idx1 >= (tl + 1) * nsr;
          float* seg = mypart + (tl == seg_tl ? 0 : SEGF);
          if (whole) {
            // everything about the destination is worked out here, once per tile, so that the loop carries no
            // state for it: owner = tl / share_cap, slot of this CTA in the owner's gather area
            const int o = tl / a.share_cap;
            const int bufn = a.gather_bufs == 2 ? (t0 / a.tiles_round) & 1 : 0;
            seg = cluster.map_shared_rank(gath, o) + ((bufn * cs + crank) * a.share_cap + (tl - o * a.share_cap)) * SEGF;
          }
#pragma unroll
          for (int j = 0; j < NTL; ++j) {
            float v0, v1, v2, v3;
            upk2(acc[j][0], v0, v1);
            upk2(acc[j][1], v2, v3);
            *reinterpret_cast<float2*>(seg + g * MC + 8 * j + 2 * t) = make_float2(v0, v1);
            *reinterpret_cast<float2*>(seg + (g + 8) * MC + 8 * j + 2 * t) = make_float2(v2, v3);
            acc[j][0] = acc[j][1] = 0ull;
          }
        }
        if (has_next) {
          if constexpr (REGPF) {
            cur = nxt;
          } else {
            cur.load(a, (tile_begin + t0 + ntl) * MMV_TR, sb0 + nrc, lane);
          }
        }
        tl = ntl;
        rec = nrc;
      }
    }
    // The next kernels of a programmatic-launch chain (an activation quantiser, then the next product) write nothing
    // before their own griddepcontrol.wait, which holds until this grid has finished. Letting them start once the
    // warp has streamed its last record hides their launch, and their prologue (codebook copy, first requests to
    // L2) overlaps the barrier, the sums and the stores here. It comes after this kernel's own wait, so the chain
    // never runs more than one product ahead.
    if (a.early && t0 + a.tiles_round >= tile_cnt) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (t0 == 0) mmv_stamp(a, 2);
    __syncthreads();
    // Tile tl of the round is owned by CTA tl / share_cap of the cluster.
    const int buf = a.gather_bufs == 2 ? (t0 / a.tiles_round) & 1 : 0;
    // (1) inside the CTA: one warp per tile shared by several warps adds their parked sums in warp order and
    // sends them to the tile's owner (a tile with a single contributor was sent whole from the loop)
    for (int tl = warp; tl < tiles_r; tl += MMV_WARPS) {
      const int w0 = (tl * nsr) / c, w1 = ((tl + 1) * nsr - 1) / c;
      if (w0 == w1) continue;
      const int o = tl / a.share_cap;
      float* dst = cluster.map_shared_rank(gath, o) + ((buf * cs + crank) * a.share_cap + (tl - o * a.share_cap)) * SEGF;
      for (int o = lane; o < SEGF; o += 32) {
        float v = 0.0f;
        for (int w = w0; w <= w1; ++w) v += partial[(2 * w + ((w * c) / nsr == tl ? 0 : 1)) * SEGF + o];
        dst[o] = v;
      }
    }
    cluster.sync();
    if (t0 == 0) mmv_stamp(a, 3);
    // (2) the owner adds the CTAs' sums (one per K part) of its tiles in rank order, from its own shared
    // memory, and stores them. Nothing remote is read after the barrier, so no second barrier is needed: the
    // next round writes the other gather area, and a CTA that has passed the last barrier only reads locally.
    const int own_tiles = max(0, min(a.share_cap, tiles_r - crank * a.share_cap));
    const float* g0 = gath + (size_t)buf * cs * a.share_cap * SEGF;
    if constexpr (!fused) {
      for (int r2 = tid; r2 < own_tiles * MMV_TR; r2 += MMV_THREADS) {
        const int row = (tile_begin + t0 + crank * a.share_cap) * MMV_TR + r2;
        if (row < a.nrows) {
#pragma unroll
          for (int c4 = 0; c4 < MC / 4; ++c4) {
            if (4 * c4 < a.m) {
              float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int r = 0; r < 8; ++r) {
                if (r < cs) {
                  const float4 p = *reinterpret_cast<const float4*>(g0 + (size_t)r * a.share_cap * SEGF + r2 * MC + 4 * c4);
                  v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
                }
              }
              const float o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (4 * c4 + e < a.m) store_out_dyn(a.y, a.y_dtype, (int64_t)(4 * c4 + e) * a.ldy + row, o[e]);
              }
            }
          }
        }
      }
    } else {
      // this rank's partial goes into its slot on every GPU (plain stores over peer pointers); one item = one row
      // x four columns, rows fastest, so that all threads of the CTA store and a warp's stores are contiguous
      const int own_rows = own_tiles * MMV_TR;
      for (int it = tid; it < own_rows * (MC / 4); it += MMV_THREADS) {
        const int c4 = it / own_rows, r2 = it - c4 * own_rows;
        const int row = (tile_begin + t0 + crank * a.share_cap) * MMV_TR + r2;
        if (row < a.nrows && 4 * c4 < a.m) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            if (r < cs) {
              const float4 p = *reinterpret_cast<const float4*>(g0 + (size_t)r * a.share_cap * SEGF + r2 * MC + 4 * c4);
              v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
            }
          }
          const float o[4] = {v.x, v.y, v.z, v.w};
          for (int p = 0; p < a.pr_world; ++p) {
            char* dst = reinterpret_cast<char*>(a.pr_slots[p]) + push_off;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (4 * c4 + e < a.m) store_out_dyn(dst, a.y_dtype, (int64_t)(4 * c4 + e) * a.ldy + row, o[e]);
            }
          }
        }
      }
    }
    if (t0 == 0) mmv_stamp(a, 4);
    __syncthreads();  // the parked sums are reused by the next round
    if (t0 == 0) mmv_stamp(a, 5);
  }
  if constexpr (fused) {
    // Sum over GPUs, in this kernel: (1) this CTA's partials are in every GPU's slot of this rank (pushed above); the
    // last CTA of this rank to get here tells every rank "rank r's partial of this call is complete" (the ranks'
    // launch plans may differ -- uneven K shards -- so the hand-off is per rank, not per CTA); (2) every CTA waits
    // (bounded) until every rank has said so; (3) it adds the world's partials of its own tiles, from this GPU's
    // memory, in rank order (bit-identical on all ranks) and stores Y.
    // (the verdict of the wait is kept in the activations' staging area, free by now: the launch plan hands all of
    // the shared memory to the dynamic part, so the kernel must not declare any of its own)
    __threadfence_system();
    __syncthreads();
    volatile int* s_peer_ok = reinterpret_cast<volatile int*>(xq);
    if (tid == 0) *s_peer_ok = 1;
    __syncthreads();
    if (tid == 0 && atomicAdd(a.pr_state + 2, 1u) == gridDim.x - 1) {
      a.pr_state[2] = 0u;
      __threadfence_system();
      for (int p = 0; p < a.pr_world; ++p) mmv_st_release_sys(a.pr_flags[p] + a.pr_rank, epoch);
    }
    if (tid < a.pr_world) {
      const uint32_t* f = a.pr_flags[a.pr_rank] + tid;
      bool ok = false;
      unsigned long long t0c, t1c;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0c));
      for (int spin = 0; spin < (1 << 24); ++spin) {       // bounded twice: by polls and by time (0.2 s)
        if ((int32_t)(mmv_ld_acquire_sys(f) - epoch) >= 0) { ok = true; break; }
        __nanosleep(20);
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1c));
        if (t1c - t0c > 200000000ull) break;
      }
      if (!ok) {
        *s_peer_ok = 0;
        atomicExch(&g_mmv_peer_error, 1);
      }
    }
    __syncthreads();
    if (*s_peer_ok) {
      const char* mine = reinterpret_cast<const char*>(a.pr_slots[a.pr_rank]) + (int64_t)((epoch & 1u) * a.pr_world) * a.pr_slot_bytes;
      for (int t0 = 0; t0 < tile_cnt; t0 += a.tiles_round) {
        const int tiles_r = min(a.tiles_round, tile_cnt - t0);
        const int own_tiles = max(0, min(a.share_cap, tiles_r - crank * a.share_cap));
        const int own_rows = own_tiles * MMV_TR;
        for (int it = tid; it < own_rows * a.m; it += MMV_THREADS) {       // one item = one result, rows fastest
          const int c = it / own_rows, r2 = it - c * own_rows;
          const int row = (tile_begin + t0 + crank * a.share_cap) * MMV_TR + r2;
          if (row < a.nrows) {
            const int64_t yi = (int64_t)c * a.ldy + row;
            float part[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) {                                   // independent loads, then the sum in rank order
              if (p < a.pr_world) part[p] = mmv_load_partial(mine + (int64_t)p * a.pr_slot_bytes, a.y_dtype, yi);
            }
            float v = 0.0f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              if (p < a.pr_world) v += part[p];
            }
            store_out_dyn(a.y, a.y_dtype, yi, v);
          }
        }
      }
    }
    // the last CTA to finish publishes the call number for the next call
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(a.pr_state + 1, 1u) == gridDim.x - 1) {
        a.pr_state[1] = 0u;
        *reinterpret_cast<volatile uint32_t*>(a.pr_state) = epoch;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host side.

static int g_mmv_mode = 0;      // 0 = use this kernel wherever it applies, 1 = never (the older kernels)
static int g_mmv_min_rows = 0;  // fewest activation rows served here; 0 = per type (see mmv_applies)
static int g_mmv_max_rows = 48; // most
static int g_mmv_cluster = 0;   // experiments: 0 = choose, else 1, 2, 4 or 8
static unsigned long long* g_mmv_prof = nullptr;
static int g_mmv_pdl = 2;       // programmatic stream serialisation: 0 off, 1 on, 2 + early start of the dependents where it pays, 3 + everywhere
static int g_mmv_pf_first = 2;  // records requested from L2 ahead of the staging
static int g_mmv_aligned = -1;  // experiments: -1 = choose, 0 / 1 = equal chunks / whole tiles per warp
static int g_mmv_trace = 0;     // one line per launch plan on stderr

// shared with the dp4a kernel: whether a product lets the next kernels of a programmatic-launch chain start early
bool mmv_early_trigger() { return g_mmv_pdl >= 2; }

constexpr int MMV_DECLINED = 1000;  // mmv_host: this shape does not fit; use another kernel

// co-resident clusters of `cs` CTAs with `smem` bytes each (cached per device / size class)
template <int KIND, int NTL, int XL, bool DUMP>
static int mmv_max_clusters(int cs, size_t smem, int sm_count, int* out) {
  struct Entry { int dev, cs, kb, n; };
  static Entry cache[64];
  static int used = 0;
  static bool configured[32];
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  auto kern = mmv_kernel<KIND, NTL, XL, DUMP>;
  if (dev >= 32 || !configured[dev]) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 0));
    if (dev < 32) configured[dev] = true;
  }
  const int kb = (int)((smem + 8191) / 8192);
  for (int i = 0; i < used; ++i) {
    if (cache[i].dev == dev && cache[i].cs == cs && cache[i].kb == kb) {
      *out = cache[i].n;
      return GSQ_OK;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sm_count / cs * cs));
  cfg.blockDim = dim3(MMV_THREADS);
  cfg.dynamicSmemBytes = (size_t)kb * 8192 > 227 * 1024 ? 227 * 1024 : (size_t)kb * 8192;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = cs;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cs == 1) {
    n = sm_count;
  } else if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  n = n < sm_count / cs ? n : sm_count / cs;
  if (used < 64) cache[used++] = Entry{dev, cs, kb, n};
  *out = n;
  return GSQ_OK;
}

template <int KIND, int NTL, int XL, bool DUMP>
static int mmv_launch_t(MmvArgs a, int sm_count, int max_smem, cudaStream_t st) {
  constexpr int MC = 8 * NTL;
  constexpr bool DS = MmvKind<KIND>::DS;
  const int nsb = a.k >> 8;
  // Cluster size: the CTAs of a cluster split K, so each stages 1 / cs of the activations, and the cluster takes
  // its tiles in rounds of as many as the gather areas have room for. Chunking: equal chunks per warp, or (from
  // 17 columns on, where the parked segments take a third of shared memory) whole tiles per warp. Among the
  // combinations that fit, the one with the least estimated time.
  struct Plan { int cs, clusters, cap, round, bufs, per; double t; };
  Plan plans[2] = {{0, 0, 0, 0, 1, 0, 0.0}, {0, 0, 0, 0, 1, 0, 0.0}};
  const int force_aligned = g_mmv_aligned;
  for (int aligned = 0; aligned <= 1; ++aligned) {
    if (force_aligned >= 0 && aligned != force_aligned) continue;
    const size_t fixed = MmvKind<KIND>::grid_bytes(NTL) + (aligned ? 0 : mmv_partial_bytes(MC));
    Plan& best = plans[aligned];
    for (int cs : {1, 2, 4, 8}) {
      if (g_mmv_cluster && cs != g_mmv_cluster) continue;
      if (cs > nsb) break;
      const int cap_kb = ((nsb + cs - 1) / cs) * 8;
      const size_t xb = mmv_x_bytes(cap_kb, MC, DS);
      if (fixed + xb + (size_t)cs * MMV_TR * MC * 4 > (size_t)max_smem) continue;
      // occupancy is asked for with the largest footprint this cluster size could use
      int n = 0;
      const int rc = mmv_max_clusters<KIND, NTL, XL, DUMP>(cs, (size_t)max_smem, sm_count, &n);
      if (rc != GSQ_OK) return rc;
      if (n <= 0) continue;
      const int clusters = n < a.ntiles ? n : a.ntiles;
      const int per = (a.ntiles + clusters - 1) / clusters;
      // tiles per round: all of a cluster's tiles if one gather area for them fits, else rounds that alternate
      // between two areas
      const size_t avail = (size_t)max_smem - fixed - xb, tile_b = (size_t)MMV_TR * MC * 4;
      int round = per, bufs = 1;
      if ((size_t)cs * ((per + cs - 1) / cs) * tile_b > avail) {
        bufs = 2;
        round = (int)(avail / (2 * tile_b)) / cs * cs;
        if (round < cs) continue;
      }
      const int rounds = (per + round - 1) / round;
      // measured: beyond 24 rows a second round costs more than the tcgen05 GEMM (repacked Q6_K has no other kernel)
      if (NTL >= 4 && rounds > 1 && KIND != MK_Q6K) continue;
      // estimated time (us): the stream of W at the rate the loop reaches, stretched by uneven clusters and idle
      // SMs; staging (36-byte blocks per thread, in batches of 4); per round a cluster barrier and the sums
      double balance = ((double)a.ntiles / (per * clusters)) * ((double)(clusters * cs) / sm_count);
      // whole tiles per warp: warps without a tile idle (this ranks the cluster sizes of that mode; the choice
      // between the modes is made below, from measurements)
      if (aligned) balance *= (double)per / (MMV_WARPS * ((per + MMV_WARPS - 1) / MMV_WARPS));
      const double t_loop = (double)a.ntiles * MMV_TR * a.row_bytes / 4.4e6 / balance * (NTL >= 3 ? 0.5 * NTL : 1.0);
      const double t_stage = 1.0 * (double)(((int64_t)a.m * cap_kb + 2047) / 2048);
      const double t = t_loop + t_stage + 0.15 * cs + 2.5 * (rounds - 1);
      if (!best.cs || t < best.t) best = Plan{cs, clusters, cap_kb, round, bufs, per, t};
    }
  }
  // Chunking, as measured: from 17 columns on whole tiles per warp win (no parking code in the loop, the parked
  // segments' third of shared memory goes to a smaller cluster); up to 16 columns they win where a CTA has few
  // records (parking then costs as much as the arithmetic) or where the tiles of a round nearly fill the warps
  // (15 tiles on 16 warps: the estimate, which leaves the parking out, then puts whole tiles within 1 us of equal
  // chunks, and they measured 0.5 - 1.2 us faster); equal chunks otherwise.
  int best_aligned = 0;
  if (plans[1].cs) {
    const int recs_per_cta = plans[1].per * ((nsb + plans[1].cs - 1) / plans[1].cs);
    if (!plans[0].cs || NTL >= 3 || recs_per_cta <= 64 || plans[1].t <= plans[0].t + 1.0) best_aligned = 1;
  }
  const int best_cs = plans[best_aligned].cs, best_clusters = plans[best_aligned].clusters, best_cap = plans[best_aligned].cap,
            best_round = plans[best_aligned].round, best_bufs = plans[best_aligned].bufs;
  const double best_t = plans[best_aligned].t;
  const size_t fixed = MmvKind<KIND>::grid_bytes(NTL) + (best_aligned ? 0 : mmv_partial_bytes(MC));
  if (g_mmv_trace) {
    fprintf(stderr, "mmv plan kind=%d ntl=%d xl=%d m=%d rows=%d k=%d: cs=%d clusters=%d round=%d bufs=%d aligned=%d est=%.1f us%s\n",
            KIND, NTL, XL, a.m, a.nrows, a.k, best_cs, best_clusters, best_round, best_bufs, best_aligned, best_t,
            best_cs ? "" : " (declined)");
  }
  if (!best_cs) return MMV_DECLINED;
  a.xcap_kb = best_cap;
  a.nsr_lo = nsb / best_cs;
  for (int i = 0; i < 2; ++i) {
    a.inv_gpc[i] = fast_div_inv((a.nsr_lo + i) * 18);
    a.inv_nkb[i] = fast_div_inv((a.nsr_lo + i) * 8);
  }
  a.inv_per = fast_div_inv(a.m * 9);
  a.tiles_base = a.ntiles / best_clusters;
  a.tiles_extra = a.ntiles % best_clusters;
  a.tiles_round = best_round;
  a.share_cap = (best_round + best_cs - 1) / best_cs;
  a.gather_bufs = best_bufs;
  a.aligned = best_aligned;
  a.pf_first = g_mmv_pf_first;
  // measured: the early start pays where the next product has a codebook to copy meanwhile and this grid leaves
  // some SMs free for the waiting quantiser (IQ3_S, 132 of 148 SMs: -1 us); it costs up to 1 us elsewhere (on a
  // full GPU the quantiser's blocks all land on the few SMs that drained first)
  a.early = g_mmv_pdl >= 3 || (g_mmv_pdl == 2 && KIND == MK_IQ3S && best_clusters * best_cs + 8 <= sm_count);
  const size_t smem = fixed + mmv_x_bytes(best_cap, MC, DS) + (size_t)best_bufs * best_cs * a.share_cap * MMV_TR * MC * 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(best_clusters * best_cs));
  cfg.blockDim = dim3(MMV_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = best_cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this kernel may start while the previous one in the stream drains; it
  // waits (griddepcontrol.wait) before it reads the activations
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_mmv_pdl ? 2 : 1;
  if (a.pr_world > 1) {
    if constexpr (DUMP) {
      return GSQ_ERR_UNSUPPORTED;
    } else {
      static bool configured[32];
      int dev = 0;
      GSQ_CUDA_TRY(cudaGetDevice(&dev));
      auto kern = mmv_kernel<KIND, NTL, XL, false, true>;
      if (dev >= 32 || !configured[dev]) {
        GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 0));
        if (dev < 32) configured[dev] = true;
      }
      GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a));
      return GSQ_OK;
    }
  }
  GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, mmv_kernel<KIND, NTL, XL, DUMP>, a));
  return GSQ_OK;
}

template <int KIND, int XL>
static int mmv_launch_n(const MmvArgs& a, int sm_count, int max_smem, cudaStream_t st) {
  const int ntl = (a.m + 7) / 8;
  if (a.dump) {
    switch (ntl) {
      case 1: return mmv_launch_t<KIND, 1, XL, true>(a, sm_count, max_smem, st);
      case 2: return mmv_launch_t<KIND, 2, XL, true>(a, sm_count, max_smem, st);
      case 3: return mmv_launch_t<KIND, 3, XL, true>(a, sm_count, max_smem, st);
      case 4: return mmv_launch_t<KIND, 4, XL, true>(a, sm_count, max_smem, st);
      case 5:
      case 6: return mmv_launch_t<KIND, 6, XL, true>(a, sm_count, max_smem, st);
      default: return MMV_DECLINED;
    }
  }
  switch (ntl) {
    case 1: return mmv_launch_t<KIND, 1, XL, false>(a, sm_count, max_smem, st);
    case 2: return mmv_launch_t<KIND, 2, XL, false>(a, sm_count, max_smem, st);
    case 3: return mmv_launch_t<KIND, 3, XL, false>(a, sm_count, max_smem, st);
    case 4: return mmv_launch_t<KIND, 4, XL, false>(a, sm_count, max_smem, st);
    case 5:
    case 6: return mmv_launch_t<KIND, 6, XL, false>(a, sm_count, max_smem, st);
    default: return MMV_DECLINED;
  }
}

// Whether (type, packed, m) may be served here (mmv_host can still decline a shape: MMV_DECLINED).
bool mmv_applies(int ggml_type, int packed, int64_t rows, int64_t m) {
  if ((g_mmv_mode == 1 && !(ggml_type == GSQ_TYPE_Q6_K && packed)) || m > 48 ||
      (m > g_mmv_max_rows && !(ggml_type == GSQ_TYPE_Q6_K && packed))) return false;
  // Below these row counts the dp4a GEMV is faster on the measured shapes (its start-up is shorter: no staging of
  // the activations, no cluster-wide sum); packed IQ3_S has no faster kernel at any count.
  int min_rows;
  switch (ggml_type) {
    case GSQ_TYPE_Q4_K: min_rows = 2; break;
    case GSQ_TYPE_IQ4_XS: min_rows = 4; break;
    case GSQ_TYPE_IQ3_S:
    case GSQ_TYPE_Q6_K:   // (repacked Q6_K has no other kernel: served here at every count)
      if (!packed || rows % 16 != 0) return false;
      min_rows = 1;
      break;
    default: return false;
  }
  if (ggml_type == GSQ_TYPE_Q6_K) return true;
  return m >= (g_mmv_min_rows > 0 ? g_mmv_min_rows : min_rows);
}

// x_layout: 0 = block_q8_1, 1 = block_q8_1_mmq. Returns MMV_DECLINED when the shape does not fit.
int mmv_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* xq, int x_layout,
             int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
             const gsq_peer_reduce* pr) {
  if (pr && (m == 0 || rows == 0)) return GSQ_ERR_UNSUPPORTED;   // every rank must launch: nothing to skip
  if (m == 0 || rows == 0) return GSQ_OK;
  if (m < 0 || m > 48 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !xq || !y) return GSQ_ERR_UNSUPPORTED;
  if (rows > INT32_MAX || k > INT32_MAX) return GSQ_ERR_TOO_LARGE;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  DeviceInfo di;
  const int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  MmvArgs a;
  a.w = (const uint8_t*)w;
  a.row_bytes = row_bytes;
  a.nrows = (int)rows;
  a.k = (int)k;
  a.xq = (const uint8_t*)xq;
  a.m = (int)m;
  a.y = y;
  a.y_dtype = y_dtype;
  a.ldy = y_row_stride;
  a.ntiles = (int)((rows + MMV_TR - 1) / MMV_TR);
  a.tiles_base = a.tiles_extra = a.tiles_round = 0;
  a.aligned = 0;
  a.xcap_kb = 0;
  a.dump = dump;
  a.prof = g_mmv_prof;
  a.pr_slots = nullptr;
  a.pr_flags = nullptr;
  a.pr_state = nullptr;
  a.pr_rank = 0;
  a.pr_world = 1;
  a.pr_slot_bytes = 0;
  if (pr) {
    const int64_t esz = y_dtype == GSQ_F32 ? 4 : 2;
    if (!pr->slots || !pr->flags || !pr->state || pr->world < 2 || pr->world > 8 || pr->rank < 0 || pr->rank >= pr->world ||
        pr->slot_bytes < ((m - 1) * y_row_stride + rows) * esz || pr->slot_bytes % 16 != 0 || dump)
      return GSQ_ERR_UNSUPPORTED;
    a.pr_slots = pr->slots;
    a.pr_flags = pr->flags;
    a.pr_state = pr->state;
    a.pr_rank = pr->rank;
    a.pr_world = pr->world;
    a.pr_slot_bytes = pr->slot_bytes;
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (ggml_type) {
    case GSQ_TYPE_Q4_K:
      return x_layout == XL_Q81 ? mmv_launch_n<MK_Q4K, XL_Q81>(a, di.sm_count, di.max_smem_optin, st)
                                : mmv_launch_n<MK_Q4K, XL_MMQ>(a, di.sm_count, di.max_smem_optin, st);
    case GSQ_TYPE_IQ4_XS:
      return x_layout == XL_Q81 ? mmv_launch_n<MK_IQ4XS, XL_Q81>(a, di.sm_count, di.max_smem_optin, st)
                                : mmv_launch_n<MK_IQ4XS, XL_MMQ>(a, di.sm_count, di.max_smem_optin, st);
    case GSQ_TYPE_IQ3_S:
      if (!packed || rows % 16 != 0) return MMV_DECLINED;
      return x_layout == XL_Q81 ? mmv_launch_n<MK_IQ3S, XL_Q81>(a, di.sm_count, di.max_smem_optin, st)
                                : mmv_launch_n<MK_IQ3S, XL_MMQ>(a, di.sm_count, di.max_smem_optin, st);
    case GSQ_TYPE_Q6_K:
      if (!packed || rows % 16 != 0) return MMV_DECLINED;
      return x_layout == XL_Q81 ? mmv_launch_n<MK_Q6K, XL_Q81>(a, di.sm_count, di.max_smem_optin, st)
                                : mmv_launch_n<MK_Q6K, XL_MMQ>(a, di.sm_count, di.max_smem_optin, st);
    default: return MMV_DECLINED;
  }
}

}  // namespace gsq

extern "C" int gsq_peer_reduce_error_flag(int* flag) {
  if (!flag) return GSQ_ERR_UNSUPPORTED;
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(flag, gsq::g_mmv_peer_error, sizeof(int)));
  return GSQ_OK;
}

extern "C" int gsq_debug_mmv_mode(int mode) {
  const int old = gsq::g_mmv_mode;
  gsq::g_mmv_mode = mode == 1 ? 1 : 0;
  return old;
}

extern "C" int gsq_debug_mmv_min_rows(int n) {
  const int old = gsq::g_mmv_min_rows;
  gsq::g_mmv_min_rows = n < 0 ? 0 : n;
  return old;
}

extern "C" int gsq_debug_mmv_max_rows(int n) {
  const int old = gsq::g_mmv_max_rows;
  gsq::g_mmv_max_rows = n > 48 ? 48 : n;
  return old;
}

extern "C" int gsq_mul_mat_vec_max_rows(int ggml_type, int packed) {
  return gsq::mmv_applies(ggml_type, packed, 16, gsq::g_mmv_max_rows) ? gsq::g_mmv_max_rows : 8;
}

extern "C" int gsq_debug_mmv_prefetch_first(int n) {
  const int old = gsq::g_mmv_pf_first;
  gsq::g_mmv_pf_first = n < 0 ? 0 : n > 64 ? 64 : n;
  return old;
}

extern "C" int gsq_debug_mmv_chunking(int mode) {
  const int old = gsq::g_mmv_aligned;
  gsq::g_mmv_aligned = (mode == 0 || mode == 1) ? mode : -1;
  return old;
}

extern "C" int gsq_debug_mmv_trace(int on) {
  const int old = gsq::g_mmv_trace;
  gsq::g_mmv_trace = on ? 1 : 0;
  return old;
}

extern "C" int gsq_debug_mmv_pdl(int on) {
  const int old = gsq::g_mmv_pdl;
  gsq::g_mmv_pdl = on < 0 ? 0 : on > 3 ? 3 : on;
  return old;
}

extern "C" int gsq_debug_mmv_profile(unsigned long long* stamps) {
  gsq::g_mmv_prof = stamps;
  return GSQ_OK;
}

extern "C" int gsq_debug_mmv_cluster_size(int cs) {
  const int old = gsq::g_mmv_cluster;
  gsq::g_mmv_cluster = (cs == 1 || cs == 2 || cs == 4 || cs == 8) ? cs : 0;
  return old;
}
