// Int8 tensor-core GEMM over GGUF superblocks for any number of activation rows (sm_100a: tcgen05 + TMEM).
//
// Replaces, behind gsq_mul_mat_q8, the reference's MMQ (csrc/lcpp/ggml/src/ggml-cuda/mmq.cuh:961-1385 with its
// tile loaders mmq-load-tiles.cuh:711-800, 1359-1495 and mmq-vec-dot.cuh:143-279, 313-440) and the owned
// mma.sync kernels mma_k (lcpp_owned_mma_k.cu:353-539) and iq3_packed_mmq (lcpp_owned_iq3_mma.cu:768-970).
// The arithmetic is theirs: for every 32-value slice s an exact int32 dot product C_s of int8 weights and int8
// activation quants, then  y += (d_w * sub_scale)[row, s] * d_q8[token, s] * C_s  in fp32 (Q4_K adds the min
// term -(dmin * m)[row, s] * half(sum x)[token, s] and rounds d * sc and dmin * m to fp16 as MMQ's tile loader does).
//
// Operands are swapped relative to the usual GEMM: the 128 weight rows of a tile fill the MMA's M, tokens
// sit on N. Because every slice has its own pair of fp scales, an MMA must not accumulate over slices:
// each K = 32 instruction writes its own 128 x NT int32 block of tensor memory (8 slices x 64 columns =
// all 512 columns), which the CUDA cores drain, scale and add into register accumulators.
//
// One persistent CTA of 8 warps per SM walks (token tile, row tile) pairs, row tiles fastest so that the
// tile of activations stays in L2 while all SMs stream the weights once per token tile. Per superblock:
//   1. all warps decode the 128 x 256 weight tile into int8 in shared memory, in the K-major "core matrix"
//      layout the MMA descriptors describe (8 rows x 16 bytes contiguous), and copy the 64 x 256 activation
//      quants next to it; the loads for the next superblock are already in flight in registers;
//   2. one thread issues the 8 MMAs and commits them to an mbarrier;
//   3. all warps read their quarter of tensor memory (tcgen05.ld), apply the scales and accumulate.
// Every wait is bounded and raises a sticky error flag instead of hanging.
#include <cooperative_groups.h>

#include "gsq_common.cuh"
#include "gsq_tables.h"

namespace cg = cooperative_groups;

namespace gsq {

enum { GK_IQ3S_PACKED = 0, GK_Q4K = 1, GK_IQ4XS = 2 };

constexpr int GEMM_THREADS = 512;
constexpr int TILE_ROWS = 128;   // weight rows per tile = MMA M
constexpr int NT = 64;           // tokens per tile = MMA N
constexpr int SL_A = 4096 + 16;  // bytes between slices of the weight tile (+16: decode stores of the 8 slices hit 8 banks)
constexpr int SL_B = NT * 32 + 16;
constexpr int TMEM_COLS = 512;

__device__ const uint32_t g_iq3s_grid_gemm[512] = GSQ_IQ3S_GRID_INIT;
__constant__ __align__(16) int8_t c_iq4nl_bytes_gemm[16] = GSQ_IQ4NL_VALUES_INIT;  // statically initialised: no upload at run time
#define c_iq4nl_words_gemm (reinterpret_cast<const uint32_t*>(c_iq4nl_bytes_gemm))
__device__ int g_gemm_error = 0;

struct GemmArgs {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;   // N
  int k;
  const uint8_t* xq;  // [k/128][m][144]
  int m;       // tokens
  void* y;
  int y_dtype;
  int64_t ldy;
  int n_row_tiles, n_tok_tiles;
  int swap_lbo_sbo;  // debug: exchange the two stride fields of the shared-memory descriptors
  int* dump;         // debug: raw int32 slice sums, [m][nrows][k/32]
};

// ---------------------------------------------------------------------------------------------
// tcgen05 / mbarrier wrappers

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] = A[smem] * B[smem], int8 x int8 -> int32, K = 32, no accumulation into D
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gemm_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool gemm_mbar_wait(uint32_t bar, uint32_t parity) {
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
    if (done) return true;
  }
  atomicExch(&g_gemm_error, 1);
  return false;
}

// 32 lanes x 32 consecutive 32-bit columns of this warp's quarter of tensor memory
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 16 consecutive columns; the wait is separate so that a load can fly while the previous one is used
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major int8 operand stored as core matrices of 8 rows x 16 bytes
// (128 contiguous bytes): the two core matrices of a row group (K bytes 0-15, 16-31) are 128 bytes apart,
// consecutive 8-row groups 256 bytes apart; no swizzle; descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, int swap) {
  const uint64_t lbo = swap ? 256 : 128, sbo = swap ? 128 : 256;
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (lbo >> 4) << 16;
  d |= (sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// Instruction descriptor: D = s32, A = B = s8, both K-major, N = NT, M = 128, dense, no negation/saturation.
__host__ __device__ constexpr uint32_t make_idesc() {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
}

__device__ __forceinline__ uint32_t gprmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// byte offset of (row r, 16-byte K chunk c16) inside one slice of a K-major core-matrix tile
__device__ __forceinline__ int core_off(int r, int c16) { return (r >> 3) * 256 + c16 * 128 + (r & 7) * 16; }

// ---------------------------------------------------------------------------------------------
// Weights of one superblock of a 128-row tile: global -> registers (fetch), registers -> int8 tile + scales (decode).

struct SmemView {
  uint8_t* a;        // 8 slices x SL_A
  uint8_t* b;        // 8 slices x SL_B
  float* sa;         // [8][128] d_w * sub-scale
  float* sam;        // [8][128] -(dmin * m)            (Q4_K)
  float* sbd;        // [8][NT]  d of the activation block
  float* sbs;        // [8][NT]  sum x of the activation block (Q4_K)
  const uint8_t* grid;  // IQ3_S codebook pairs (g, -g), 16 replicas
};

// P = number of threads that share the tile's 1024 (row, chunk) items
template <int KIND, int P>
struct WRegs;

template <int P>
struct WRegs<GK_IQ3S_PACKED, P> {
  uint32_t idx[9], sg[4];
  uint2 sc;
  uint32_t dd;
  bool ok;
  __device__ __forceinline__ void fetch(const GemmArgs& g, int rt, int sb, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    // P = 512: two warps per 16-row record, four of its eight slices each; P = 256: one warp per record
    const int row0 = rt * TILE_ROWS + 16 * (P == 512 ? warp >> 1 : warp);
    ok = row0 < g.nrows;
    if (!ok) return;
    const uint8_t* p = g.w + (int64_t)row0 * g.row_bytes + (int64_t)sb * 1760;
    const uint4 ia = ldg_stream_v4(p + 16 * lane), ib = ldg_stream_v4(p + 512 + 16 * lane);
    idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
    idx[4] = ib.x; idx[5] = ib.y; idx[6] = ib.z; idx[7] = ib.w;
    idx[8] = ldg_stream_u32(p + 1024 + 4 * lane);
    const uint4 s = ldg_stream_v4(p + 1152 + 16 * lane);
    sg[0] = s.x; sg[1] = s.y; sg[2] = s.z; sg[3] = s.w;
    sc = ldg_stream_v2(p + 1664 + 8 * (lane >> 2));
    dd = ldg_stream_u32(p + 1728 + 4 * (lane >> 2));
  }
  // Lane (g = lane / 4, t = lane % 4) holds, of rows g and g + 8 and every slice, the 4-value groups 2t, 2t + 1
  // (field f = 4 s + 2 h + e of gsq_iq3s_repack): 8 bytes of the row's 32-byte slice, one 64-bit store each.
  __device__ __forceinline__ void decode(const SmemView& sm, int tid) const {
    if (!ok) return;
    const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
    const uint32_t lane_off = (uint32_t)(lane & 15) << 3;
    const int rbase = 16 * (P == 512 ? warp >> 1 : warp) + gq;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (P == 512 && (s >> 2) != (warp & 1)) continue;  // warp-uniform: this warp's half of the record
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t wv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int f = 4 * s + 2 * h + e, bit = 9 * f, word = bit >> 5, off = bit & 31;
          uint32_t v;
          if (off + 9 <= 32) {
            v = off >= 7 ? idx[word] >> (off >= 7 ? off - 7 : 0) : idx[word] << (off < 7 ? 7 - off : 0);
          } else {
            v = __funnelshift_r(idx[word], idx[word + 1], off - 7);
          }
          const uint2 gp = *reinterpret_cast<const uint2*>(sm.grid + ((v & 0xFF80u) | lane_off));
          const int fl = f & 7, sh = 16 * (fl >> 2) + (fl & 3) - 2;
          const uint32_t sgs = sh >= 0 ? sg[f >> 3] >> (sh >= 0 ? sh : 0) : sg[f >> 3] << (sh < 0 ? -sh : 0);
          wv[e] = gprmt(gp.x, gp.y, (sgs & 0x4444u) | 0x3210u);
        }
        const int r = rbase + 8 * h;
        *reinterpret_cast<uint2*>(sm.a + s * SL_A + core_off(r, t >> 1) + 8 * (t & 1)) = make_uint2(wv[0], wv[1]);
        if ((s & 3) == t) {  // the four lanes of a row group share its scales: each writes two slices
          const float d = h2f(dd >> (16 * h));
          const uint32_t scw = h ? sc.y : sc.x;
          sm.sa[s * TILE_ROWS + r] = d * (float)(1 + 2 * (int)((scw >> (4 * s)) & 15u));
        }
      }
    }
  }
};

template <int P>
struct WRegs<GK_Q4K, P> {
  static constexpr int NITEM = 1024 / P;
  uint4 hdr[NITEM], qs[NITEM];
  __device__ __forceinline__ void fetch(const GemmArgs& g, int rt, int sb, int tid) {
#pragma unroll
    for (int q = 0; q < NITEM; ++q) {
      const int item = tid + P * q, r = item >> 3, p = item & 7;
      const int row = min(rt * TILE_ROWS + r, g.nrows - 1);
      const uint8_t* b = g.w + (int64_t)row * g.row_bytes + (int64_t)sb * 144;
      hdr[q] = ldg_stream_v4(b);
      qs[q] = ldg_stream_v4(b + 16 + 16 * p);
    }
  }
  __device__ __forceinline__ void decode(const SmemView& sm, int tid) const {
#pragma unroll
    for (int q = 0; q < NITEM; ++q) {
      const int item = tid + P * q, r = item >> 3, p = item & 7, jj = p >> 1, half = p & 1;
      const uint4 v = qs[q];
      uint8_t* lo = sm.a + (2 * jj) * SL_A + core_off(r, half);
      *reinterpret_cast<uint4*>(lo) = make_uint4(v.x & 0x0F0F0F0Fu, v.y & 0x0F0F0F0Fu, v.z & 0x0F0F0F0Fu, v.w & 0x0F0F0F0Fu);
      *reinterpret_cast<uint4*>(lo + SL_A) = make_uint4((v.x >> 4) & 0x0F0F0F0Fu, (v.y >> 4) & 0x0F0F0F0Fu,
                                                       (v.z >> 4) & 0x0F0F0F0Fu, (v.w >> 4) & 0x0F0F0F0Fu);
      if (half == 0) {
        const uint32_t selh = (jj & 1) ? 0x4432u : 0x4410u;
        const uint32_t A = gprmt(hdr[q].y, 0u, selh), B = gprmt(hdr[q].z, 0u, selh), C = gprmt(hdr[q].w, 0u, selh);
        const uint32_t sc = jj < 2 ? (A & 0x3F3Fu) : ((C & 0x0F0Fu) | ((A & 0xC0C0u) >> 2));
        const uint32_t mn = jj < 2 ? (B & 0x3F3Fu) : (((C >> 4) & 0x0F0Fu) | ((B & 0xC0C0u) >> 2));
        // d * sc and dmin * m rounded to fp16, as the reference's tile loader keeps them (half2 products)
        const __half2 dm = *reinterpret_cast<const __half2*>(&hdr[q].x);
        const float2 p0 = __half22float2(__hmul2(dm, __floats2half2_rn((float)(sc & 0xFFu), (float)(mn & 0xFFu))));
        const float2 p1 = __half22float2(__hmul2(dm, __floats2half2_rn((float)(sc >> 8), (float)(mn >> 8))));
        sm.sa[(2 * jj) * TILE_ROWS + r] = p0.x;
        sm.sam[(2 * jj) * TILE_ROWS + r] = -p0.y;
        sm.sa[(2 * jj + 1) * TILE_ROWS + r] = p1.x;
        sm.sam[(2 * jj + 1) * TILE_ROWS + r] = -p1.y;
      }
    }
  }
};

template <int P>
struct WRegs<GK_IQ4XS, P> {
  static constexpr int NITEM = 1024 / P;
  uint2 hdr[NITEM], qa[NITEM], qb[NITEM];
  __device__ __forceinline__ void fetch(const GemmArgs& g, int rt, int sb, int tid) {
#pragma unroll
    for (int q = 0; q < NITEM; ++q) {
      const int item = tid + P * q, r = item >> 3, p = item & 7;
      const int row = min(rt * TILE_ROWS + r, g.nrows - 1);
      const uint8_t* b = g.w + (int64_t)row * g.row_bytes + (int64_t)sb * 136;
      hdr[q] = ldg_stream_v2(b);
      qa[q] = ldg_stream_v2(b + 8 + 16 * p);
      qb[q] = ldg_stream_v2(b + 16 + 16 * p);
    }
  }
  static __device__ __forceinline__ void lookup(uint32_t v, uint32_t& lo, uint32_t& hi) {
    const uint32_t t0 = c_iq4nl_words_gemm[0], t1 = c_iq4nl_words_gemm[1], t2 = c_iq4nl_words_gemm[2],
                   t3 = c_iq4nl_words_gemm[3];
    const uint32_t s01 = v & 0x7777u, s23 = (v >> 16) & 0x7777u;
    const uint32_t pick01 = 0x3210u | ((v & 0x8888u) >> 1), pick23 = 0x3210u | (((v >> 16) & 0x8888u) >> 1);
    const uint32_t r01 = gprmt(gprmt(t0, t1, s01), gprmt(t2, t3, s01), pick01);
    const uint32_t r23 = gprmt(gprmt(t0, t1, s23), gprmt(t2, t3, s23), pick23);
    lo = gprmt(r01, r23, 0x6420u);
    hi = gprmt(r01, r23, 0x7531u);
  }
  __device__ __forceinline__ void decode(const SmemView& sm, int tid) const {
#pragma unroll
    for (int q = 0; q < NITEM; ++q) {
      const int item = tid + P * q, r = item >> 3, p = item & 7;
      const uint32_t v[4] = {qa[q].x, qa[q].y, qb[q].x, qb[q].y};
      uint32_t lo[4], hi[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) lookup(v[e], lo[e], hi[e]);
      uint8_t* dst = sm.a + p * SL_A;
      *reinterpret_cast<uint4*>(dst + core_off(r, 0)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      *reinterpret_cast<uint4*>(dst + core_off(r, 1)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      const uint32_t ls = ((hdr[q].y >> (4 * p)) & 0xFu) | (((hdr[q].x >> (16 + 2 * p)) & 3u) << 4);
      sm.sa[p * TILE_ROWS + r] = h2f(hdr[q].x) * (float)((int)ls - 32);
    }
  }
};

// Activation quants of one superblock for the NT tokens of a tile (128-value blocks, 144 bytes each).
template <bool DS4, int P>
struct XRegs {
  static constexpr int NITEM = 1024 / P;
  uint4 q[NITEM];
  uint32_t sc[NITEM];
  __device__ __forceinline__ void fetch(const GemmArgs& g, int t0, int sb, int tid) {
#pragma unroll
    for (int i = 0; i < NITEM; ++i) {
      const int item = tid + P * i, c = item >> 4, j = item & 15;
      const int tok = t0 + c;
      q[i] = make_uint4(0, 0, 0, 0);
      sc[i] = 0;
      if (tok < g.m) {
        const uint8_t* b = g.xq + ((int64_t)(2 * sb + (j >> 3)) * g.m + tok) * 144;
        q[i] = __ldg(reinterpret_cast<const uint4*>(b + 16 + (j & 7) * 16));
        if ((j & 1) == 0) sc[i] = __ldg(reinterpret_cast<const uint32_t*>(b + 4 * ((j >> 1) & 3)));
      }
    }
  }
  __device__ __forceinline__ void store(const SmemView& sm, int tid) const {
#pragma unroll
    for (int i = 0; i < NITEM; ++i) {
      const int item = tid + P * i, c = item >> 4, j = item & 15, s = j >> 1;
      *reinterpret_cast<uint4*>(sm.b + s * SL_B + core_off(c, j & 1)) = q[i];
      if ((j & 1) == 0) {
        if (DS4) {
          const float2 ds = __half22float2(*reinterpret_cast<const __half2*>(&sc[i]));
          sm.sbd[s * NT + c] = ds.x;
          sm.sbs[s * NT + c] = ds.y;
        } else {
          sm.sbd[s * NT + c] = __uint_as_float(sc[i]);
        }
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// The kernel.

constexpr int STAGE_BYTES_BASE = 8 * SL_A + 8 * SL_B + 2 * 8 * NT * 4;  // + 1 or 2 weight-scale planes

template <int KIND>
__host__ __device__ constexpr size_t gemm_stage_bytes() {
  return STAGE_BYTES_BASE + (KIND == GK_Q4K ? 2 : 1) * 8 * TILE_ROWS * 4;
}
template <int KIND>
__host__ __device__ constexpr size_t gemm_smem_bytes() {
  return 128 + (KIND == GK_IQ3S_PACKED ? 65536 : 0) + 2 * gemm_stage_bytes<KIND>();
}

template <int KIND>
__device__ __forceinline__ SmemView stage_view(uint8_t* base, const uint8_t* grid) {
  SmemView sm;
  sm.grid = grid;
  sm.a = base;
  base += 8 * SL_A;
  sm.b = base;
  base += 8 * SL_B;
  sm.sa = reinterpret_cast<float*>(base);
  base += 8 * TILE_ROWS * 4;
  sm.sam = reinterpret_cast<float*>(base);
  if (KIND == GK_Q4K) base += 8 * TILE_ROWS * 4;
  sm.sbd = reinterpret_cast<float*>(base);
  base += 8 * NT * 4;
  sm.sbs = reinterpret_cast<float*>(base);
  return sm;
}

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// One slice's 16 columns of this warp: scale and accumulate. The accumulators stay packed two per 64-bit
// register pair (columns 2i, 2i + 1) for the packed fp32 instructions of sm_100 (mul / add / fma .f32x2):
// per pair of elements 2 integer adds and 3 packed floating-point instructions. All 16 columns are processed,
// valid or not (tokens past the end of X were staged as zeros and are never stored): no data-dependent
// branch in the hot loop.
template <bool DS4>
__device__ __forceinline__ void epilogue_slice(const uint32_t (&c)[16], const SmemView& sm, int s, int r_in, int col0,
                                               int ncols, uint64_t (&acc2)[8]) {
  constexpr int MAGIC = 0x4B400000;
  constexpr float MAGIC_F = 12582912.0f;
  (void)ncols;
  const float da = sm.sa[s * TILE_ROWS + r_in];
  const float dam = DS4 ? sm.sam[s * TILE_ROWS + r_in] : 0.0f;
  const float4* bd = reinterpret_cast<const float4*>(sm.sbd + s * NT + col0);
  const float4* bs = reinterpret_cast<const float4*>(sm.sbs + s * NT + col0);
  const uint64_t da2 = pack2(da, da), nm2 = pack2(-MAGIC_F, -MAGIC_F), dam2 = pack2(dam, dam);
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) {
    const float4 d = bd[j4];
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (DS4) t = bs[j4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int j = 4 * j4 + 2 * u;
      const uint64_t dv2 = u == 0 ? pack2(d.x, d.y) : pack2(d.z, d.w);
      // exact int -> float: |c| <= 32 * 127 * 127 < 2^22, so c + bits(1.5 * 2^23) read as a float is 1.5 * 2^23 + c
      const uint64_t f2 = add2(pack2(__int_as_float((int)c[j] + MAGIC), __int_as_float((int)c[j + 1] + MAGIC)), nm2);
      acc2[2 * j4 + u] = fma2(mul2(da2, dv2), f2, acc2[2 * j4 + u]);
      if (DS4) acc2[2 * j4 + u] = fma2(dam2, u == 0 ? pack2(t.x, t.y) : pack2(t.z, t.w), acc2[2 * j4 + u]);
    }
  }
}

__device__ __forceinline__ void dump_slice(const GemmArgs& g, const uint32_t (&c)[16], int row, int tok0, int ncols, int slice) {
  if (row >= g.nrows) return;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (j < ncols) g.dump[((int64_t)(tok0 + j) * g.nrows + row) * (g.k >> 5) + slice] = (int)c[j];
  }
}

// Clusters of `ksplit` CTAs share one (token tile, row tile) item and split its superblocks; the partial
// accumulators meet in the first CTA through distributed shared memory, added in rank order.
template <int KIND>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_kernel(const GemmArgs g) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool DS4 = KIND == GK_Q4K;
  cg::cluster_group cluster = cg::this_cluster();
  const int cs = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem);
  const uint32_t mbar = smem_addr(smem + 16);
  const uint8_t* grid = smem + 128;
  uint8_t* stage0 = smem + 128 + (KIND == GK_IQ3S_PACKED ? 65536 : 0);
  float* red = reinterpret_cast<float*>(stage0);  // [NT][128] partial accumulators (reuses the tile buffers)

  if (warp == 0) tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
  if (tid == 32) {
    gemm_mbar_init(mbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (KIND == GK_IQ3S_PACKED) {
    const uint32_t gv = g_iq3s_grid_gemm[tid & 511];
    uint4* dst = reinterpret_cast<uint4*>(smem + 128 + (tid & 511) * 128);
#pragma unroll
    for (int r2 = 0; r2 < 8; ++r2) dst[r2] = make_uint4(gv, ~gv + 0x01010101u, gv, ~gv + 0x01010101u);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nsb = g.k >> 8;
  const int sb_begin = (int)((int64_t)nsb * crank / cs), sb_end = (int)((int64_t)nsb * (crank + 1) / cs);
  const int n_items = g.n_row_tiles * g.n_tok_tiles;
  const int n_clusters = (int)gridDim.x / cs, cluster_id = (int)blockIdx.x / cs;
  const uint32_t idesc = make_idesc();
  const int q4 = warp & 3, h = warp >> 2;        // tensor-memory lane quarter, 16-column group of this warp
  const int r_in = 32 * q4 + lane;               // row of the tile this thread accumulates
  uint32_t phase = 0;
  bool alive = true;  // false once a bounded wait gave up: skip the remaining work, still free tensor memory

  for (int item = cluster_id; item < n_items; item += n_clusters) {
    const int tt = item / g.n_row_tiles, rt = item - tt * g.n_row_tiles;
    const int t0 = tt * NT;
    // The 4 warps of a lane quarter share the tile's 16-column groups: with 4 groups one group each (all 8
    // slices), with 2 groups two warps per group (4 slices each), with 1 group four warps (2 slices each);
    // warps that share a group add their accumulators through shared memory at the end.
    const int mt = min(NT, g.m - t0);
    const int cgc = mt > 32 ? 4 : mt > 16 ? 2 : 1, wpc = 4 / cgc;
    const int col0 = 16 * (h % cgc), sl0 = h / cgc;
    const int ncols = mt - col0;  // valid columns among this warp's 16 (> 0 by construction)
    const uint32_t t_warp = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)col0;
    uint64_t acc2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc2[j] = 0ull;
    if (alive && sb_begin < sb_end) {
      WRegs<KIND, GEMM_THREADS> wr;
      XRegs<DS4, GEMM_THREADS> xr;
      wr.fetch(g, rt, sb_begin, tid);
      xr.fetch(g, t0, sb_begin, tid);
      {
        const SmemView first = stage_view<KIND>(stage0, grid);
        wr.decode(first, tid);
        xr.store(first, tid);
      }
      if (sb_begin + 1 < sb_end) {
        wr.fetch(g, rt, sb_begin + 1, tid);
        xr.fetch(g, t0, sb_begin + 1, tid);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
      __syncthreads();
      for (int sb = sb_begin; sb < sb_end && alive; ++sb) {
        const int st = (sb - sb_begin) & 1;
        // views are rebuilt from the shared array each time (never indexed from memory) so that every access
        // below compiles to a shared-memory instruction
        const SmemView cur = stage_view<KIND>(stage0 + st * gemm_stage_bytes<KIND>(), grid);
        const SmemView nxt = stage_view<KIND>(stage0 + (st ^ 1) * gemm_stage_bytes<KIND>(), grid);
        if (tid == 0) {
          tc_fence_after();
          const uint32_t a_addr = smem_addr(cur.a), b_addr = smem_addr(cur.b);
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            mma_i8(tmem_base + (uint32_t)(s * NT), make_smem_desc(a_addr + s * SL_A, g.swap_lbo_sbo),
                   make_smem_desc(b_addr + s * SL_B, g.swap_lbo_sbo), idesc);
          }
          mma_commit(mbar);
        }
        // while the tensor core works: the next superblock goes into the other stage, the one after it
        // into registers
        if (sb + 1 < sb_end) {
          wr.decode(nxt, tid);
          xr.store(nxt, tid);
          if (sb + 2 < sb_end) {
            wr.fetch(g, rt, sb + 2, tid);
            xr.fetch(g, t0, sb + 2, tid);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        alive = gemm_mbar_wait(mbar, phase);
        phase ^= 1u;
        tc_fence_after();
        if (alive && ncols > 0) {
          // this warp's slices: every wpc-th one starting at sl0 (all 8 when the tile has 4 column groups)
          uint32_t c0[16], c1[16];
          tmem_ld16_issue(t_warp + (uint32_t)(sl0 * NT), c0);
#pragma unroll 1
          for (int s = sl0; s < 8; s += 2 * wpc) {
            const int s1 = s + wpc;
            tmem_ld_wait();
            if (s1 < 8) tmem_ld16_issue(t_warp + (uint32_t)(s1 * NT), c1);
            if (g.dump) dump_slice(g, c0, rt * TILE_ROWS + r_in, t0 + col0, ncols, sb * 8 + s);
            epilogue_slice<DS4>(c0, cur, s, r_in, col0, ncols, acc2);
            if (s1 < 8) {
              tmem_ld_wait();
              if (s1 + wpc < 8) tmem_ld16_issue(t_warp + (uint32_t)((s1 + wpc) * NT), c0);
              if (g.dump) dump_slice(g, c1, rt * TILE_ROWS + r_in, t0 + col0, ncols, sb * 8 + s1);
              epilogue_slice<DS4>(c1, cur, s1, r_in, col0, ncols, acc2);
            }
          }
        }
        tc_fence_before();
        __syncthreads();  // tensor memory and stage st are free again; stage st ^ 1 is complete
      }
    }
    float acc[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) unpack2(acc2[j], acc[2 * j], acc[2 * j + 1]);
    const int row = rt * TILE_ROWS + r_in;
    if (wpc > 1) {
      // warps sharing a column group: the one with sl0 == 0 adds the others' accumulators in warp order
      if (sl0 != 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) red[((sl0 - 1) * NT + col0 + j) * TILE_ROWS + r_in] = acc[j];
      }
      __syncthreads();
      if (sl0 == 0) {
        for (int w = 1; w < wpc; ++w) {
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] += red[((w - 1) * NT + col0 + j) * TILE_ROWS + r_in];
        }
      }
      __syncthreads();
    }
    if (cs > 1) {
      // combine the K-parts: every CTA parks its accumulators, the first one adds them in rank order
      if (sl0 == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) red[(col0 + j) * TILE_ROWS + r_in] = acc[j];
      }
      cluster.sync();
      if (crank == 0 && sl0 == 0) {
        for (int r = 1; r < cs; ++r) {
          const float* rr = cluster.map_shared_rank(red, r);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] += rr[(col0 + j) * TILE_ROWS + r_in];
        }
      }
    }
    if (alive && crank == 0 && sl0 == 0 && row < g.nrows) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (j < ncols) store_out_dyn(g.y, g.y_dtype, (int64_t)(t0 + col0 + j) * g.ldy + row, acc[j]);
      }
    }
    if (cs > 1) cluster.sync();  // the partial sums have been read: the tile buffers may be overwritten
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Warp-specialised variant: 8 producer warps (fetch + decode into a 2-stage ring), 1 MMA warp, 8 consumer
// warps (tensor-memory drain + scaling). The phases of consecutive superblocks overlap: while the consumers
// scale superblock sb, the tensor core multiplies sb + 1 (tensor memory is used as two halves of 4 slices)
// and the producers decode sb + 2. Hand-offs are mbarriers; every wait is bounded and a wait that gives up
// raises a CTA-wide abort flag that makes all other waits return at once.

constexpr int WS_PROD = 256, WS_CONS = 256, WS_THREADS = WS_PROD + WS_CONS + 32;

template <int KIND>
__host__ __device__ constexpr size_t gemm_ws_smem_bytes() {
  return 128 + (KIND == GK_IQ3S_PACKED ? 65536 : 0) + 2 * gemm_stage_bytes<KIND>() + NT * TILE_ROWS * 4;
}

__device__ __forceinline__ bool ws_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
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
    if (done) return true;
    if ((spin & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(&g_gemm_error, 1);
  return false;
}
__device__ __forceinline__ void ws_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int KIND>
__global__ void __launch_bounds__(WS_THREADS, 1) gemm_ws_kernel(const GemmArgs g) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool DS4 = KIND == GK_Q4K;
  cg::cluster_group cluster = cg::this_cluster();
  const int cs = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 4);
  const uint32_t bars = smem_addr(smem + 16);
  // barrier i at bars + 8 i: full[2] = 0,1; ab_free[2] = 2,3; sc_free[2] = 4,5; tmem_full[2] = 6,7; tmem_empty[2] = 8,9
  const uint8_t* grid = smem + 128;
  uint8_t* stage0 = smem + 128 + (KIND == GK_IQ3S_PACKED ? 65536 : 0);
  float* red = reinterpret_cast<float*>(stage0 + 2 * gemm_stage_bytes<KIND>());  // [NT][128]

  if (warp == 16) tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      gemm_mbar_init(bars + 8 * (0 + i), WS_PROD);
      gemm_mbar_init(bars + 8 * (2 + i), 1);
      gemm_mbar_init(bars + 8 * (4 + i), WS_CONS);
      gemm_mbar_init(bars + 8 * (6 + i), 1);
      gemm_mbar_init(bars + 8 * (8 + i), WS_CONS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (KIND == GK_IQ3S_PACKED && tid < 512) {
    const uint32_t gv = g_iq3s_grid_gemm[tid];
    uint4* dst = reinterpret_cast<uint4*>(smem + 128 + tid * 128);
#pragma unroll
    for (int r2 = 0; r2 < 8; ++r2) dst[r2] = make_uint4(gv, ~gv + 0x01010101u, gv, ~gv + 0x01010101u);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nsb = g.k >> 8;
  const int sb_begin = (int)((int64_t)nsb * crank / cs), sb_end = (int)((int64_t)nsb * (crank + 1) / cs);
  const int n_items = g.n_row_tiles * g.n_tok_tiles;
  const int n_clusters = (int)gridDim.x / cs, cluster_id = (int)blockIdx.x / cs;
  uint32_t n = 0;      // superblocks handled so far by this role (ring position and barrier phases)
  bool alive = true;

  if (warp < 8) {
    // ------------------------------------------------------------------ producers
    for (int item = cluster_id; item < n_items; item += n_clusters) {
      const int tt = item / g.n_row_tiles, rt = item - tt * g.n_row_tiles, t0 = tt * NT;
      if (alive && sb_begin < sb_end) {
        WRegs<KIND, WS_PROD> wr;
        XRegs<DS4, WS_PROD> xr;
        wr.fetch(g, rt, sb_begin, tid);
        xr.fetch(g, t0, sb_begin, tid);
        for (int sb = sb_begin; sb < sb_end; ++sb, ++n) {
          const uint32_t st = n & 1u, par = ((n >> 1) & 1u) ^ 1u;
          alive = ws_wait(bars + 8 * (2 + st), par, abort_flag) && ws_wait(bars + 8 * (4 + st), par, abort_flag);
          if (!alive) break;
          const SmemView v = stage_view<KIND>(stage0 + st * gemm_stage_bytes<KIND>(), grid);
          wr.decode(v, tid);
          xr.store(v, tid);
          if (sb + 1 < sb_end) {
            wr.fetch(g, rt, sb + 1, tid);
            xr.fetch(g, t0, sb + 1, tid);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          ws_arrive(bars + 8 * (0 + st));
        }
      }
      if (cs > 1) {
        cluster.sync();
        cluster.sync();
      }
    }
  } else if (warp == 16) {
    // ------------------------------------------------------------------ MMA issue (one thread)
    const uint32_t idesc = make_idesc();
    for (int item = cluster_id; item < n_items; item += n_clusters) {
      if (lane == 0 && alive) {
        for (int sb = sb_begin; sb < sb_end; ++sb, ++n) {
          const uint32_t st = n & 1u;
          alive = ws_wait(bars + 8 * (0 + st), (n >> 1) & 1u, abort_flag);
          if (!alive) break;
          tc_fence_after();
          const SmemView v = stage_view<KIND>(stage0 + st * gemm_stage_bytes<KIND>(), grid);
          const uint32_t a_addr = smem_addr(v.a), b_addr = smem_addr(v.b);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            alive = ws_wait(bars + 8 * (8 + half), (n & 1u) ^ 1u, abort_flag);
            if (!alive) break;
            tc_fence_after();
#pragma unroll
            for (int sl = 0; sl < 4; ++sl) {
              const int s = 4 * half + sl;
              mma_i8(tmem_base + (uint32_t)(s * NT), make_smem_desc(a_addr + s * SL_A, g.swap_lbo_sbo),
                     make_smem_desc(b_addr + s * SL_B, g.swap_lbo_sbo), idesc);
            }
            mma_commit(bars + 8 * (6 + half));
          }
          if (!alive) break;
          mma_commit(bars + 8 * (2 + st));  // the stage's operand tiles are free once these MMAs have read them
        }
      }
      if (cs > 1) {
        cluster.sync();
        cluster.sync();
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 8, q4 = cw & 3, pair = cw >> 2;
    const int r_in = 32 * q4 + lane;
    for (int item = cluster_id; item < n_items; item += n_clusters) {
      const int tt = item / g.n_row_tiles, rt = item - tt * g.n_row_tiles, t0 = tt * NT;
      const int mt = min(NT, g.m - t0);
      // more than 32 tokens: the two warps of a lane quarter take 32 columns each; otherwise both take columns
      // 0..31 and share the slices (pair p: slices p and p + 2 of each half), summed through shared memory
      const bool by_cols = mt > 32;
      const int col0 = by_cols ? 32 * pair : 0;
      const uint32_t t_warp = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)col0;
      uint64_t acc_lo[8], acc_hi[8];  // columns col0 .. col0 + 15 and the next 16, two per register pair
#pragma unroll
      for (int j = 0; j < 8; ++j) acc_lo[j] = acc_hi[j] = 0ull;
      const bool need_hi = mt - col0 > 16;  // warp-uniform: skip the upper 16 columns when no token is there
      if (alive) {
        for (int sb = sb_begin; sb < sb_end; ++sb, ++n) {
          const uint32_t st = n & 1u;
          const SmemView v = stage_view<KIND>(stage0 + st * gemm_stage_bytes<KIND>(), grid);
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            alive = ws_wait(bars + 8 * (6 + half), n & 1u, abort_flag);
            if (!alive) break;
            tc_fence_after();
            // 16 columns at a time, the next load in flight while the previous one is scaled
            uint32_t c0[16], c1[16];
            const int sl_first = by_cols ? 0 : pair, sl_step = by_cols ? 1 : 2;
            tmem_ld16_issue(t_warp + (uint32_t)((4 * half + sl_first) * NT), c0);
#pragma unroll 1
            for (int sl = sl_first; sl < 4; sl += sl_step) {
              const int s = 4 * half + sl;
              tmem_ld_wait();
              if (need_hi) {
                tmem_ld16_issue(t_warp + (uint32_t)(s * NT + 16), c1);
              } else if (sl + sl_step < 4) {
                tmem_ld16_issue(t_warp + (uint32_t)((s + sl_step) * NT), c1);
              }
              if (g.dump) dump_slice(g, c0, rt * TILE_ROWS + r_in, t0 + col0, mt - col0, sb * 8 + s);
              epilogue_slice<DS4>(c0, v, s, r_in, col0, 16, acc_lo);
              if (need_hi) {
                tmem_ld_wait();
                if (sl + sl_step < 4) tmem_ld16_issue(t_warp + (uint32_t)((s + sl_step) * NT), c0);
                if (g.dump) dump_slice(g, c1, rt * TILE_ROWS + r_in, t0 + col0 + 16, mt - col0 - 16, sb * 8 + s);
                epilogue_slice<DS4>(c1, v, s, r_in, col0 + 16, 16, acc_hi);
              } else if (sl + sl_step < 4) {
                // lower 16 columns only: c1 receives the next slice (its load overlapped the scaling above);
                // once it has landed make it the current one
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) c0[j] = c1[j];
              }
            }
            tc_fence_before();
            ws_arrive(bars + 8 * (8 + half));  // this half of tensor memory may be overwritten
          }
          if (!alive) break;
          ws_arrive(bars + 8 * (4 + st));      // the stage's scale planes have been read
        }
      }
      float acc[32];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        unpack2(acc_lo[j], acc[2 * j], acc[2 * j + 1]);
        unpack2(acc_hi[j], acc[16 + 2 * j], acc[17 + 2 * j]);
      }
      const int row = rt * TILE_ROWS + r_in;
      if (!by_cols) {
        if (pair == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) red[j * TILE_ROWS + r_in] = acc[j];
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (pair == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] += red[j * TILE_ROWS + r_in];
        }
      }
      const bool owner = by_cols || pair == 0;
      if (cs > 1) {
        if (owner) {
#pragma unroll
          for (int j = 0; j < 32; ++j) red[(col0 + j) * TILE_ROWS + r_in] = acc[j];
        }
        cluster.sync();
        if (crank == 0 && owner) {
          for (int r = 1; r < cs; ++r) {
            const float* rr = cluster.map_shared_rank(red, r);
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] += rr[(col0 + j) * TILE_ROWS + r_in];
          }
        }
      }
      if (alive && crank == 0 && owner && row < g.nrows) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < mt) store_out_dyn(g.y, g.y_dtype, (int64_t)(t0 + col0 + j) * g.ldy + row, acc[j]);
        }
      }
      if (cs > 1) cluster.sync();
      if (!by_cols) asm volatile("bar.sync 1, 256;" ::: "memory");  // red is reused by the next item
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 16) tmem_dealloc(tmem_base, TMEM_COLS);
}

static int g_swap_lbo_sbo = 0;
static int* g_gemm_dump = nullptr;
static int g_gemm_ksplit = 0;  // experiments: 0 = choose, else 1, 2 or 4
static int g_gemm_variant = 0;  // behind gsq_linear: 0 = choose by shape, 3 = always a prefill GEMM (gsq_gemm3.cu for repacked IQ3_S, else gsq_gemm2.cu; 5 / 6 / 7: with its split / rounded / integer form forced; 9 / 8: split / rounded on pairs of CTAs), 4 = always gsq_gemm2.cu; the kernels of this file: 1 = warp-specialised, 2 = lockstep

int gemm2_error_flag(int* flag);  // gsq_gemm2.cu
int gemm3_error_flag(int* flag);  // gsq_gemm3.cu

int gemm_error_flag(int* flag) {
  int a = 0, b = 0, c = 0;
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(&a, g_gemm_error, sizeof(int)));
  int rc = gemm2_error_flag(&b);
  if (rc != GSQ_OK) return rc;
  rc = gemm3_error_flag(&c);
  if (rc != GSQ_OK) return rc;
  *flag = a | b | c;
  return GSQ_OK;
}

int* gemm_dump_pointer() { return g_gemm_dump; }
int gemm_variant() { return g_gemm_variant; }

template <int KIND>
static int launch_gemm(const GemmArgs& g, int sm_count, cudaStream_t st) {
  static int configured_mask = 0;
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  const bool ws = g_gemm_variant == 1;   // (0 and 2: the lockstep kernel)
  const size_t smem = ws ? gemm_ws_smem_bytes<KIND>() : gemm_smem_bytes<KIND>();
  if (dev >= 32 || !((configured_mask >> dev) & 1)) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)gemm_smem_bytes<KIND>()));
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm_ws_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)gemm_ws_smem_bytes<KIND>()));
    if (dev < 32) configured_mask |= 1 << dev;
  }
  const int n_items = g.n_row_tiles * g.n_tok_tiles;
  // split K over a cluster when there are too few tiles to occupy the SMs (decode-sized token counts)
  int ks = 1;
  const int nsb = g.k >> 8;
  if (g_gemm_ksplit) {
    ks = g_gemm_ksplit;
  } else {
    while (ks < 4 && n_items * ks * 2 <= sm_count && nsb / (ks * 2) >= 2) ks *= 2;
  }
  int clusters = n_items < sm_count / ks ? n_items : sm_count / ks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(clusters * ks));
  cfg.blockDim = dim3(ws ? WS_THREADS : GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = ks;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (ws) {
    GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_ws_kernel<KIND>, g));
  } else {
    GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_kernel<KIND>, g));
  }
  return GSQ_OK;
}

}  // namespace gsq

extern "C" int gsq_debug_swap_descriptor_strides(int on) {
  const int old = gsq::g_swap_lbo_sbo;
  gsq::g_swap_lbo_sbo = on ? 1 : 0;
  return old;
}

extern "C" int gsq_debug_gemm_variant(int v) {
  const int old = gsq::g_gemm_variant;
  gsq::g_gemm_variant = (v >= 1 && v <= 9) ? v : 0;
  return old;
}

extern "C" int gsq_debug_gemm_ksplit(int ks) {
  const int old = gsq::g_gemm_ksplit;
  gsq::g_gemm_ksplit = (ks == 1 || ks == 2 || ks == 4) ? ks : 0;
  return old;
}

extern "C" int gsq_debug_gemm_dump_sums(int32_t* sums) {
  gsq::g_gemm_dump = sums;
  return GSQ_OK;
}

extern "C" size_t gsq_mul_mat_scratch_bytes(int64_t rows, int64_t m, int64_t k, int ggml_type) {
  (void)rows; (void)m; (void)k; (void)ggml_type;
  return 0;  // every CTA owns whole rows over all of K: nothing to combine through global memory
}

namespace gsq {
// gsq_mmv.cu: the register-operand tensor-core kernel for 1..48 rows
bool mmv_applies(int ggml_type, int packed, int64_t rows, int64_t m);
int mmv_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* xq, int x_layout,
             int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
             const gsq_peer_reduce* pr = nullptr);
}  // namespace gsq

extern "C" int gsq_mul_mat_q8(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                              const void* x_q8_mmq, int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride,
                              void* scratch, size_t scratch_bytes, void* stream) {
  using namespace gsq;
  (void)scratch;
  (void)scratch_bytes;
  if (m == 0 || rows == 0) return GSQ_OK;
  if (mmv_applies(ggml_type, packed, rows, m)) {
    const int rc = mmv_host(w, row_bytes, rows, ggml_type, packed, x_q8_mmq, 1, m, k, y, y_dtype, y_row_stride, stream,
                            g_gemm_dump);
    if (rc != 1000) return rc;  // 1000: the shape does not fit that kernel
  }
  if (m < 0 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !x_q8_mmq || !y) return GSQ_ERR_UNSUPPORTED;
  if (rows > INT32_MAX || k > INT32_MAX || m > INT32_MAX) return GSQ_ERR_TOO_LARGE;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  int kind;
  if (ggml_type == GSQ_TYPE_IQ3_S && packed && rows % 16 == 0) {
    kind = GK_IQ3S_PACKED;
  } else if (ggml_type == GSQ_TYPE_Q4_K) {
    kind = GK_Q4K;
  } else if (ggml_type == GSQ_TYPE_IQ4_XS) {
    kind = GK_IQ4XS;
  } else {
    return GSQ_ERR_UNSUPPORTED;  // Q6_K and IQ3_S in GGUF order: the caller runs the GEMV 8 rows at a time
  }
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  GemmArgs g;
  g.w = (const uint8_t*)w;
  g.row_bytes = row_bytes;
  g.nrows = (int)rows;
  g.k = (int)k;
  g.xq = (const uint8_t*)x_q8_mmq;
  g.m = (int)m;
  g.y = y;
  g.y_dtype = y_dtype;
  g.ldy = y_row_stride;
  g.n_row_tiles = (int)((rows + TILE_ROWS - 1) / TILE_ROWS);
  g.n_tok_tiles = (int)((m + NT - 1) / NT);
  g.swap_lbo_sbo = g_swap_lbo_sbo;
  g.dump = g_gemm_dump;
  cudaStream_t st = (cudaStream_t)stream;
  switch (kind) {
    case GK_IQ3S_PACKED: return launch_gemm<GK_IQ3S_PACKED>(g, di.sm_count, st);
    case GK_Q4K: return launch_gemm<GK_Q4K>(g, di.sm_count, st);
    default: return launch_gemm<GK_IQ4XS>(g, di.sm_count, st);
  }
}
