// Prefill GEMM over GGUF superblocks (sm_100a: tcgen05 kind::i8, TMEM accumulators), warp-specialised.
//
// Serves gsq_linear above the small-batch row counts: the reference's MMQ (csrc/lcpp/ggml/src/ggml-cuda/mmq.cuh:
// 961-1385, tile loaders mmq-load-tiles.cuh:711-800, 1359-1495) and its owned prefill kernels mma_k
// (lcpp_owned_mma_k.cu:353-539) and iq3_packed_mmq (lcpp_owned_iq3_mma.cu:768-970). Arithmetic as there: per 32-value
// slice s an exact int32 dot product C_s of int8 weights and int8 activation quants, then
//   y += fma(float(C_s) * dA[row, s], dB[token, s], y)        dA = d_w * sub-scale, dB = d of the q8_1 block
// (Q4_K adds -(dmin * m)[row, s] * sum_x[token, s] and rounds d * sc, dmin * m to fp16 as MMQ's tile loader does).
//
// A CTA owns a tile of 128 weight rows x 256 tokens and walks K one superblock (256 values = 8 slices) at a time:
//   * 3 producer warps fetch the raw superblocks of the 128 rows (cp.async into a 3-deep ring) and decode them ONCE
//     into an int8 tile in shared memory, in the K-major core-matrix layout the MMA descriptors describe, plus the
//     per-row slice scales;
//   * one thread streams the activation units (one slice x 256 tokens, already in that same layout in global memory,
//     written so by quantize_q8_1_tiles_kernel, gsq_quantize.cu) with one bulk copy per unit into an 8-deep ring, and
//     issues one MMA of 128 x 256 x 32 per unit into one half of tensor memory (256 columns), the other half being
//     drained meanwhile (N = 256: the weight slice is read from shared memory once per 256 tokens);
//   * 16 consumer warps (4 per tensor-memory lane quarter, 64 columns each) read the int32 sums with tcgen05.ld,
//     scale them (one logic instruction + 2 packed fp32 FMAs per pair of elements) and accumulate 64 fp32 values per
//     thread (row = lane of tensor memory) in registers over the whole of K.
// All hand-offs are mbarriers; every wait is bounded and raises a CTA-wide abort flag (and the sticky device flag
// read by gsq_device_error_flag) instead of hanging. Register budget: setmaxnreg moves registers from the producer
// warpgroup to the four consumer warpgroups.
#include "gsq_common.cuh"
#include "gsq_tables.h"
#include "gsq_tc.cuh"

namespace gsq {

enum { G2_IQ3S = 0, G2_Q4K = 1, G2_IQ4XS = 2 };

namespace g2 {

constexpr int TR = 128;                 // weight rows per tile (MMA M)
constexpr int NT = 256;                 // tokens per tile (MMA N)
constexpr int PROD_WARPS = 3;
constexpr int PROD_THREADS = PROD_WARPS * 32;
constexpr int CONS_WARPS = 16;
constexpr int THREADS = 128 + CONS_WARPS * 32;   // warps 0-2 producers, warp 3 MMA + bulk copies, warps 4-19 consumers
constexpr int SL_A = 4096;              // bytes of one slice of the decoded weight tile (128 rows x 32)
constexpr int SL_B = 8192;              // bytes of the quants of one activation unit (256 tokens x 32)
constexpr int A_STAGES = 2;
constexpr int B_SLOTS = 8;
constexpr int B_AHEAD = 6;              // units the bulk copies run ahead of the MMAs
constexpr int RAW_STAGES = 3;
constexpr int TMEM_COLS = 512;

// bytes of one unit (one slice of a 256-token block) of the activation tiles: quants, d (+ sum for Q4_K)
__host__ __device__ constexpr int unit_bytes(bool ds) { return SL_B + NT * 4 * (ds ? 2 : 1); }
__host__ __device__ constexpr int raw_bytes(int kind) { return kind == G2_IQ3S ? 8 * 1760 : kind == G2_Q4K ? 128 * 144 : 128 * 136; }
__host__ __device__ constexpr int grid_bytes(int kind) { return kind == G2_IQ3S ? 512 * 64 : 0; }  // (g, -g) x 8 replicas
__host__ __device__ constexpr int scale_planes(int kind) { return kind == G2_Q4K ? 2 : 1; }

struct Args {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;
  int k;
  const uint8_t* xt;   // activation units: [token block of 256][superblock][slice][unit_bytes]
  int m;
  void* y;
  int y_dtype;
  int64_t ldy;
  int n_row_tiles, n_tok_blocks;
  int* dump;           // debug: raw int32 slice sums [m][nrows][k / 32]
  unsigned long long* prof;  // debug: per CTA 16 clock counts (see gsq_debug_gemm_profile)
};

// shared-memory map (byte offsets from the 1024-byte aligned base)
template <int KIND>
struct Smem {
  static constexpr int BAR = 0;                                       // mbarriers + tmem slot + abort flag
  static constexpr int GRID = 1024;
  static constexpr int RAW = GRID + grid_bytes(KIND);
  static constexpr int A = RAW + RAW_STAGES * ((raw_bytes(KIND) + 127) / 128 * 128);
  static constexpr int SA = A + A_STAGES * 8 * SL_A;                  // [stage][plane][8][128] floats
  static constexpr int B = SA + A_STAGES * scale_planes(KIND) * 8 * TR * 4;
  static constexpr int TOTAL = B + B_SLOTS * unit_bytes(KIND == G2_Q4K);
};

__device__ int g_error = 0;

using namespace tc;

// K-major int8 operand: the two core matrices of a row group (K bytes 0-15, 16-31) 128 bytes apart, consecutive 8-row
// groups 256 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) { return tc::smem_desc(addr, 128, 256); }
// Instruction descriptor: D = s32, A = B = s8, both K-major, N = 256, M = 128, dense.
__host__ __device__ constexpr uint32_t idesc() {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TR >> 4) << 24);
}
// byte offset of (row r, 16-byte K chunk c16) inside one slice of a K-major core-matrix tile
__device__ __forceinline__ int core_off(int r, int c16) { return (r >> 3) * 256 + c16 * 128 + (r & 7) * 16; }


__device__ const uint32_t g_iq3s_grid[512] = GSQ_IQ3S_GRID_INIT;
__constant__ __align__(16) int8_t c_iq4nl[16] = GSQ_IQ4NL_VALUES_INIT;

// ---------------------------------------------------------------------------------------------
// Producers: raw superblocks of the tile's 128 rows, global -> shared (cp.async), then raw -> int8 tile + scales.

template <int KIND>
__device__ __forceinline__ void fetch_raw(const Args& g, int rt, int sb, uint8_t* raw, int ptid) {
  const uint32_t dst = saddr(raw);
  if (KIND == G2_IQ3S) {
    // 8 records of 1760 contiguous bytes (16 rows each); records past the last row are not fetched (nor decoded)
    for (int i = ptid; i < 8 * 110; i += PROD_THREADS) {
      const int rec = i / 110, c = i - rec * 110;
      const int row0 = rt * TR + 16 * rec;
      if (row0 < g.nrows) cp_async16(dst + rec * 1760 + c * 16, g.w + (int64_t)row0 * g.row_bytes + (int64_t)sb * 1760 + c * 16);
    }
  } else if (KIND == G2_Q4K) {
    for (int i = ptid; i < 128 * 9; i += PROD_THREADS) {
      const int r = i / 9, c = i - r * 9;
      const int row = min(rt * TR + r, g.nrows - 1);
      cp_async16(dst + r * 144 + c * 16, g.w + (int64_t)row * g.row_bytes + (int64_t)sb * 144 + c * 16);
    }
  } else {
    for (int i = ptid; i < 128 * 17; i += PROD_THREADS) {
      const int r = i / 17, c = i - r * 17;
      const int row = min(rt * TR + r, g.nrows - 1);
      cp_async8(dst + r * 136 + c * 8, g.w + (int64_t)row * g.row_bytes + (int64_t)sb * 136 + c * 8);
    }
  }
}

// IQ3_S in the fragment-ordered layout of gsq_iq3s_repack: lane (gq = lane / 4, t = lane % 4) of a record holds, of
// rows gq and gq + 8 and every slice, the 4-value groups 2t, 2t + 1 (field f = 4 s + 2 h + e at bit 9 f of its nine
// index words; sign bits pre-arranged as byte-permute selectors). A warp decodes one half (4 slices) of a record.
__device__ __forceinline__ void decode_iq3s(const uint8_t* raw, uint8_t* a, float* sa, const uint8_t* grid, int nrows_left,
                                            int pwarp, int lane) {
  const int gq = lane >> 2, t = lane & 3;
  const uint32_t lane_off = (uint32_t)(lane & 7) << 3;
  for (int u = pwarp; u < 16; u += PROD_WARPS) {
    const int rec = u >> 1, hf = u & 1;
    if (16 * rec >= nrows_left) continue;
    const uint8_t* p = raw + rec * 1760;
    // index words 4 hf .. 4 hf + 4 of this lane (fields 16 hf .. 16 hf + 15 start at bit 144 hf = word 4.5 hf)
    uint32_t idx[5];
    if (hf == 0) {
      const uint4 ia = *reinterpret_cast<const uint4*>(p + 16 * lane);
      idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
      idx[4] = *reinterpret_cast<const uint32_t*>(p + 512 + 16 * lane);
    } else {
      const uint4 ib = *reinterpret_cast<const uint4*>(p + 512 + 16 * lane);
      idx[0] = ib.x; idx[1] = ib.y; idx[2] = ib.z; idx[3] = ib.w;
      idx[4] = *reinterpret_cast<const uint32_t*>(p + 1024 + 4 * lane);
    }
    const uint2 sg = *reinterpret_cast<const uint2*>(p + 1152 + 16 * lane + 8 * hf);
    const uint2 sc = *reinterpret_cast<const uint2*>(p + 1664 + 8 * gq);
    const uint32_t dd = *reinterpret_cast<const uint32_t*>(p + 1728 + 4 * gq);
#pragma unroll
    for (int sl = 0; sl < 4; ++sl) {
      const int s = 4 * hf + sl;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t wv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          // field 4 sl + 2 h + e of this half: bit offset within the half's words (hf = 1 starts 16 bits into word 4)
          const int f = 4 * sl + 2 * h + e;
          const int bit = 9 * f + 16 * hf, word = bit >> 5, off = bit & 31;
          uint32_t v;
          if (off + 9 <= 32) {
            v = off >= 6 ? idx[word] >> (off >= 6 ? off - 6 : 0) : idx[word] << (off < 6 ? 6 - off : 0);
          } else {
            v = __funnelshift_r(idx[word], idx[word + 1], off - 6);
          }
          const uint2 gp = *reinterpret_cast<const uint2*>(grid + ((v & 0x7FC0u) | lane_off));
          const int fl = f & 7, sh = 16 * (fl >> 2) + (fl & 3) - 2;
          const uint32_t sgw = (f >> 3) ? sg.y : sg.x;
          const uint32_t sgs = sh >= 0 ? sgw >> (sh >= 0 ? sh : 0) : sgw << (sh < 0 ? -sh : 0);
          wv[e] = prmt(gp.x, gp.y, (sgs & 0x4444u) | 0x3210u);
        }
        const int r = 16 * rec + gq + 8 * h;
        *reinterpret_cast<uint2*>(a + s * SL_A + core_off(r, t >> 1) + 8 * (t & 1)) = make_uint2(wv[0], wv[1]);
        if (sl == t) {  // the four lanes of a row group share its scales: each writes one slice of this half
          const float d = h2f(dd >> (16 * h));
          const uint32_t scw = h ? sc.y : sc.x;
          sa[s * TR + r] = d * (float)(1 + 2 * (int)((scw >> (4 * s)) & 15u));
        }
      }
    }
  }
}

// Q4_K: item (row r, 16-byte piece p of the 128 quant bytes): low nibbles are slice 2 (p / 2), high nibbles the next.
__device__ __forceinline__ void decode_q4k(const uint8_t* raw, uint8_t* a, float* sa, float* sam, int ptid) {
  for (int item = ptid; item < 1024; item += PROD_THREADS) {
    const int r = item >> 3, p = item & 7, jj = p >> 1, half = p & 1;
    const uint4 v = *reinterpret_cast<const uint4*>(raw + r * 144 + 16 + 16 * p);
    uint8_t* lo = a + (2 * jj) * SL_A + core_off(r, half);
    *reinterpret_cast<uint4*>(lo) = make_uint4(v.x & 0x0F0F0F0Fu, v.y & 0x0F0F0F0Fu, v.z & 0x0F0F0F0Fu, v.w & 0x0F0F0F0Fu);
    *reinterpret_cast<uint4*>(lo + SL_A) = make_uint4((v.x >> 4) & 0x0F0F0F0Fu, (v.y >> 4) & 0x0F0F0F0Fu,
                                                     (v.z >> 4) & 0x0F0F0F0Fu, (v.w >> 4) & 0x0F0F0F0Fu);
    if (half == 0) {
      const uint4 hdr = *reinterpret_cast<const uint4*>(raw + r * 144);
      const uint32_t selh = (jj & 1) ? 0x4432u : 0x4410u;
      const uint32_t A = prmt(hdr.y, 0u, selh), B = prmt(hdr.z, 0u, selh), C = prmt(hdr.w, 0u, selh);
      const uint32_t sc = jj < 2 ? (A & 0x3F3Fu) : ((C & 0x0F0Fu) | ((A & 0xC0C0u) >> 2));
      const uint32_t mn = jj < 2 ? (B & 0x3F3Fu) : (((C >> 4) & 0x0F0Fu) | ((B & 0xC0C0u) >> 2));
      // d * sc and dmin * m rounded to fp16, as the reference's tile loader keeps them (half2 products)
      const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
      const float2 p0 = __half22float2(__hmul2(dm, __floats2half2_rn((float)(sc & 0xFFu), (float)(mn & 0xFFu))));
      const float2 p1 = __half22float2(__hmul2(dm, __floats2half2_rn((float)(sc >> 8), (float)(mn >> 8))));
      sa[(2 * jj) * TR + r] = p0.x;
      sam[(2 * jj) * TR + r] = -p0.y;
      sa[(2 * jj + 1) * TR + r] = p1.x;
      sam[(2 * jj + 1) * TR + r] = -p1.y;
    }
  }
}

// IQ4_XS: item (row r, slice p): 16 bytes of 4-bit indices into the 16-entry table; low nibbles are values 0..15 of
// the slice, high nibbles 16..31.
__device__ __forceinline__ void iq4_lookup(uint32_t v, const uint32_t (&tb)[4], uint32_t& lo, uint32_t& hi) {
  const uint32_t s01 = v & 0x7777u, s23 = (v >> 16) & 0x7777u;
  const uint32_t pick01 = 0x3210u | ((v & 0x8888u) >> 1), pick23 = 0x3210u | (((v >> 16) & 0x8888u) >> 1);
  const uint32_t r01 = prmt(prmt(tb[0], tb[1], s01), prmt(tb[2], tb[3], s01), pick01);
  const uint32_t r23 = prmt(prmt(tb[0], tb[1], s23), prmt(tb[2], tb[3], s23), pick23);
  lo = prmt(r01, r23, 0x6420u);
  hi = prmt(r01, r23, 0x7531u);
}
__device__ __forceinline__ void decode_iq4xs(const uint8_t* raw, uint8_t* a, float* sa, int ptid) {
  const uint32_t* tw = reinterpret_cast<const uint32_t*>(c_iq4nl);
  const uint32_t tb[4] = {tw[0], tw[1], tw[2], tw[3]};
  for (int item = ptid; item < 1024; item += PROD_THREADS) {
    const int r = item >> 3, p = item & 7;
    const uint8_t* b = raw + r * 136;
    const uint2 hdr = *reinterpret_cast<const uint2*>(b);
    const uint2 qa = *reinterpret_cast<const uint2*>(b + 8 + 16 * p), qb = *reinterpret_cast<const uint2*>(b + 16 + 16 * p);
    const uint32_t v[4] = {qa.x, qa.y, qb.x, qb.y};
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) iq4_lookup(v[e], tb, lo[e], hi[e]);
    uint8_t* dst = a + p * SL_A;
    *reinterpret_cast<uint4*>(dst + core_off(r, 0)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    *reinterpret_cast<uint4*>(dst + core_off(r, 1)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    const uint32_t ls = ((hdr.y >> (4 * p)) & 0xFu) | (((hdr.x >> (16 + 2 * p)) & 3u) << 4);
    sa[p * TR + r] = h2f(hdr.x) * (float)((int)ls - 32);
  }
}

// ---------------------------------------------------------------------------------------------
// Consumers: one unit = the int32 sums of 4 slices x 64 tokens in one half of tensor memory.

// 8 columns of one slice: acc += fma(float(C) * dA, dB, acc) (+ dAm * sum for Q4_K). float(C) * dA is formed as
// fma(bits(C + 1.5 * 2^23), dA, -1.5 * 2^23 * dA): dA has at most 17 significant bits, so the subtrahend is exact and
// the result is the correctly rounded product. acc: the 4 register pairs of these 8 columns.
template <bool DS>
__device__ __forceinline__ void scale8(const uint32_t (&c)[8], float da, float dam, const float* bd, const float* bs,
                                       float2* acc) {
  // packed fp32 FMAs (two elements per instruction; measured against scalar FMAs: the same pipe time, half the
  // issue slots)
  const float2 da2 = make_float2(da, da), nmda2 = make_float2(-MAGIC_F * da, -MAGIC_F * da), dam2 = make_float2(dam, dam);
#pragma unroll
  for (int j4 = 0; j4 < 2; ++j4) {
    const float4 d = *reinterpret_cast<const float4*>(bd + 4 * j4);
    const float2 t0 = __ffma2_rn(make_float2(biased_float(c[4 * j4]), biased_float(c[4 * j4 + 1])), da2, nmda2);
    const float2 t1 = __ffma2_rn(make_float2(biased_float(c[4 * j4 + 2]), biased_float(c[4 * j4 + 3])), da2, nmda2);
    acc[2 * j4] = __ffma2_rn(t0, make_float2(d.x, d.y), acc[2 * j4]);
    acc[2 * j4 + 1] = __ffma2_rn(t1, make_float2(d.z, d.w), acc[2 * j4 + 1]);
    if (DS) {
      const float4 s = *reinterpret_cast<const float4*>(bs + 4 * j4);
      acc[2 * j4] = __ffma2_rn(dam2, make_float2(s.x, s.y), acc[2 * j4]);
      acc[2 * j4 + 1] = __ffma2_rn(dam2, make_float2(s.z, s.w), acc[2 * j4 + 1]);
    }
  }
}

__device__ __forceinline__ void dump8(const Args& g, const uint32_t (&c)[8], int row, int tok0, int slice) {
  if (row >= g.nrows) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (tok0 + j < g.m) g.dump[((int64_t)(tok0 + j) * g.nrows + row) * (g.k >> 5) + slice] = (int)c[j];
  }
}

// ring cursor: position and phase parity of an n-deep ring of mbarriers 8 bytes apart
struct Ring {
  uint32_t i, ph;
  __device__ __forceinline__ void next(uint32_t n) {
    if (++i == n) { i = 0; ph ^= 1u; }
  }
};

template <int KIND, int MODE>
__global__ void __launch_bounds__(THREADS, 1) gemm2_kernel(const Args g) {
  constexpr bool DUMP = MODE == 1, PROF = MODE == 2;
  unsigned long long pw[4] = {0ull, 0ull, 0ull, 0ull};   // debug (MODE 2): clocks spent in this thread's waits / work
  auto tick = [&]() -> unsigned long long { return PROF ? (unsigned long long)clock64() : 0ull; };
  extern __shared__ __align__(1024) uint8_t smem[];
  using S = Smem<KIND>;
  constexpr bool DS = KIND == G2_Q4K;
  constexpr int UB = unit_bytes(DS);
  constexpr int RAWB = (raw_bytes(KIND) + 127) / 128 * 128;
  constexpr int STAGE_A = 8 * SL_A, STAGE_SA = scale_planes(KIND) * 8 * TR * 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // barriers (8 bytes each): a_full[2] a_empty[2] b_full[8] b_empty[8] d_full[2] d_empty[2]
  const uint32_t bar0 = saddr(smem + S::BAR);
  const uint32_t a_full = bar0, a_empty = bar0 + 16, b_full = bar0 + 32, b_empty = b_full + 8 * B_SLOTS,
                 d_full = b_empty + 8 * B_SLOTS, d_empty = d_full + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::BAR + 260);
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool { return mbar_wait(bar, parity, abort_flag, &g_error); };

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(a_full + 8 * i, PROD_THREADS);
      mbar_init(a_empty + 8 * i, CONS_WARPS);
      mbar_init(d_full + 8 * i, 1);
      mbar_init(d_empty + 8 * i, CONS_WARPS);
    }
    for (int i = 0; i < B_SLOTS; ++i) {
      mbar_init(b_full + 8 * i, 1);
      mbar_init(b_empty + 8 * i, CONS_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 3) tmem_alloc(saddr(tmem_slot), TMEM_COLS);
  if (KIND == G2_IQ3S) {
    for (int i = tid; i < 512; i += THREADS) {
      const uint32_t gv = g_iq3s_grid[i];
      uint4* dst = reinterpret_cast<uint4*>(smem + S::GRID + i * 64);
#pragma unroll
      for (int r2 = 0; r2 < 4; ++r2) dst[r2] = make_uint4(gv, ~gv + 0x01010101u, gv, ~gv + 0x01010101u);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nsb = g.k >> 8;
  const int n_items = g.n_row_tiles * g.n_tok_blocks;
  // items of this CTA: row tiles fastest, so that the CTAs running at one time share a token block's activations in L2
  auto item_rt = [&](int item) { return item % g.n_row_tiles; };
  auto item_tb = [&](int item) { return item / g.n_row_tiles; };

  if (warp < PROD_WARPS) {
    // ------------------------------------------------------------------------------------ producers
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    const int ptid = tid;
    // the flat stream of (item, superblock) pairs of this CTA; raw loads run two ahead of the decode
    int f_item = blockIdx.x, f_sb = 0;        // fetch cursor
    auto fetch_next = [&](int n_fetch) {
      if (f_item < n_items) {
        fetch_raw<KIND>(g, item_rt(f_item), f_sb, smem + S::RAW + (n_fetch % RAW_STAGES) * RAWB, ptid);
        if (++f_sb == nsb) { f_sb = 0; f_item += gridDim.x; }
      }
      cp_async_commit();
    };
    fetch_next(0);
    fetch_next(1);
    uint32_t n = 0;
    Ring ra = {0u, 0u};
    bool alive = true;
    // (after a wait has given up the loop still runs to its end, without work: every producer thread passes the
    // same number of named barriers)
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const int rt = item_rt(item);
      for (int sb = 0; sb < nsb; ++sb, ++n) {
        cp_async_wait<1>();                                  // this thread's pieces of stream position n have landed
        asm volatile("bar.sync 1, %0;" ::"n"(PROD_THREADS) : "memory");   // everyone's have; everyone is done with n - 1
        fetch_next((int)n + 2);
        const unsigned long long p0 = tick();
        alive = alive && wait(a_empty + 8 * ra.i, ra.ph ^ 1u);
        const unsigned long long p1 = tick();
        pw[0] += p1 - p0;
        if (alive) {
          const uint8_t* raw = smem + S::RAW + (n % RAW_STAGES) * RAWB;
          uint8_t* a = smem + S::A + ra.i * STAGE_A;
          float* sa = reinterpret_cast<float*>(smem + S::SA + ra.i * STAGE_SA);
          if (KIND == G2_IQ3S) {
            decode_iq3s(raw, a, sa, smem + S::GRID, g.nrows - rt * TR, warp, lane);
          } else if (KIND == G2_Q4K) {
            decode_q4k(raw, a, sa, sa + 8 * TR, ptid);
          } else {
            decode_iq4xs(raw, a, sa, ptid);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor-core reads
          mbar_arrive(a_full + 8 * ra.i);
          pw[1] += tick() - p1;
        }
        ra.next(A_STAGES);
      }
    }
    if (PROF && tid == 0) {
      g.prof[blockIdx.x * 16 + 0] = pw[0];   // producer: waiting for a free stage
      g.prof[blockIdx.x * 16 + 1] = pw[1];   // producer: decoding
    }
    cp_async_wait<0>();
  } else if (warp == 3) {
    // ------------------------------------------------------------------------------------ bulk copies + MMA issue
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (lane == 0) {
      // This one thread is on every unit's critical path: everything it does per unit is kept to a few dozen
      // instructions (no divisions, descriptors and source addresses by increments).
      const uint32_t id = idesc();
      const uint64_t desc_hi = smem_desc(0u) & 0xFFFFFFFF00000000ull;
      const uint32_t a_lo0 = (uint32_t)smem_desc(saddr(smem + S::A)), b_lo0 = (uint32_t)smem_desc(saddr(smem + S::B));
      auto desc = [&](uint32_t lo) { return desc_hi | (uint64_t)lo; };
      const uint32_t b_smem0 = saddr(smem + S::B);
      // load cursor over the stream of units (item, superblock, slice), B_AHEAD ahead of the MMAs; the units of a
      // token block are contiguous in global memory
      int l_item = blockIdx.x, l_u = 0;
      const int units_item = 8 * nsb;
      const uint8_t* l_base = nullptr;
      auto load_item = [&]() {
        if (l_item < n_items) l_base = g.xt + (int64_t)item_tb(l_item) * units_item * UB;
      };
      load_item();
      Ring rl = {0u, 0u};
      uint32_t n_loaded = 0;
      bool alive = true;
      auto load_next = [&]() {
        if (l_item >= n_items || !alive) return;
        alive = wait(b_empty + 8 * rl.i, rl.ph ^ 1u);
        if (!alive) return;
        mbar_expect_tx(b_full + 8 * rl.i, UB);
        bulk_g2s(b_smem0 + rl.i * UB, l_base + (int64_t)l_u * UB, UB, b_full + 8 * rl.i);
        rl.next(B_SLOTS);
        ++n_loaded;
        if (++l_u == units_item) {
          l_u = 0;
          l_item += gridDim.x;
          load_item();
        }
      };
      for (int i = 0; i < B_AHEAD; ++i) load_next();
      Ring ra = {0u, 0u}, rb = {0u, 0u}, rd = {0u, 0u};
      uint32_t n_used = 0;
      for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
        for (int sb = 0; sb < nsb && alive; ++sb) {
          const unsigned long long m0 = tick();
          alive = wait(a_full + 8 * ra.i, ra.ph);
          pw[0] += tick() - m0;
          if (!alive) break;
          const uint32_t a_lo = a_lo0 + ra.i * (STAGE_A >> 4);
#pragma unroll 1
          for (int sl = 0; sl < 8; ++sl) {
            // the consumers have drained this half of tensor memory (two units ago)
            const unsigned long long m1 = tick();
            alive = wait(d_empty + 8 * rd.i, rd.ph ^ 1u);
            pw[1] += tick() - m1;
            if (!alive) break;
            const unsigned long long m3 = tick();
            alive = wait(b_full + 8 * rb.i, rb.ph);
            pw[2] += tick() - m3;
            if (!alive) break;
            tc_fence_after();
            mma_i8(tmem_base + rd.i * 256, desc(a_lo + sl * (SL_A >> 4)), desc(b_lo0 + rb.i * (UB >> 4)), id);
            mma_commit(d_full + 8 * rd.i);
            rb.next(B_SLOTS);
            rd.next(2);
            ++n_used;
            load_next();   // after the MMA is on its way: the copy for B_AHEAD units further on
          }
          ra.next(A_STAGES);
        }
      }
      if (PROF) {
        g.prof[blockIdx.x * 16 + 2] = pw[0];   // MMA thread: waiting for a decoded weight tile
        g.prof[blockIdx.x * 16 + 3] = pw[1];   // MMA thread: waiting for a drained half of tensor memory
        g.prof[blockIdx.x * 16 + 4] = pw[2];   // MMA thread: waiting for an activation unit
      }
      if (!alive) {
        // a wait gave up: let the copies already issued land (bounded) before the CTA's shared memory goes away
        for (; n_used < n_loaded; ++n_used) {
          wait(b_full + 8 * rb.i, rb.ph);
          rb.next(B_SLOTS);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------------------------ consumers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int cw = warp - 4, q4 = warp & 3, cg = cw >> 2;   // tensor-memory lane quarter = warp id mod 4
    const int r_in = 32 * q4 + lane;
    const uint32_t t_warp = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)(64 * cg);
    Ring ra = {0u, 0u}, rb = {0u, 0u}, rd = {0u, 0u};
    bool alive = true;
    for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
      const int rt = item_rt(item), tok0 = item_tb(item) * NT + 64 * cg;
      float2 acc[32];   // this thread's row x 64 tokens
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.0f, 0.0f);
      for (int sb = 0; sb < nsb && alive; ++sb) {
        const unsigned long long c0t = tick();
        alive = wait(a_full + 8 * ra.i, ra.ph);   // the producers' scale planes are visible
        pw[0] += tick() - c0t;
        if (!alive) break;
        const float* sap = reinterpret_cast<const float*>(smem + S::SA + ra.i * STAGE_SA) + r_in;
#pragma unroll 1
        for (int sl = 0; sl < 8; ++sl) {
          const unsigned long long c1t = tick();
          alive = alive && wait(b_full + 8 * rb.i, rb.ph);   // the unit's scales are visible
          const unsigned long long c2t = tick();
          alive = alive && wait(d_full + 8 * rd.i, rd.ph);
          const unsigned long long c3t = tick();
          pw[1] += c2t - c1t;
          pw[2] += c3t - c2t;
          if (alive) {
            tc_fence_after();
            const float* bd = reinterpret_cast<const float*>(smem + S::B + rb.i * UB + SL_B) + 64 * cg;
            const float* bs = bd + NT;
            const float da = sap[sl * TR], dam = DS ? sap[(8 + sl) * TR] : 0.0f;
            const uint32_t t_unit = t_warp + rd.i * 256;
            const int slice = sb * 8 + sl;
            // chunks of 8 columns, the next chunk's load in flight while one is scaled
            uint32_t c0[8], c1[8];
            tmem_ld8(t_unit, c0);
#pragma unroll
            for (int ch = 0; ch < 8; ch += 2) {
              tmem_ld_wait();
              tmem_ld8(t_unit + 8 * (ch + 1), c1);
              if (DUMP) dump8(g, c0, rt * TR + r_in, tok0 + 8 * ch, slice);
              scale8<DS>(c0, da, dam, bd + 8 * ch, bs + 8 * ch, &acc[4 * ch]);
              tmem_ld_wait();
              if (ch < 6) tmem_ld8(t_unit + 8 * (ch + 2), c0);
              if (DUMP) dump8(g, c1, rt * TR + r_in, tok0 + 8 * (ch + 1), slice);
              scale8<DS>(c1, da, dam, bd + 8 * (ch + 1), bs + 8 * (ch + 1), &acc[4 * (ch + 1)]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(b_empty + 8 * rb.i);
              mbar_arrive(d_empty + 8 * rd.i);
            }
            pw[3] += tick() - c3t;
          }
          rb.next(B_SLOTS);
          rd.next(2);
        }
        __syncwarp();
        if (lane == 0 && alive) mbar_arrive(a_empty + 8 * ra.i);   // the stage's scale planes (and, the MMAs done, its tile) are free
        ra.next(A_STAGES);
      }
      // results of the item: thread = weight row, 64 tokens
      const int row = rt * TR + r_in;
      if (alive && row < g.nrows) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int tok = tok0 + 2 * i;
          if (tok < g.m) store_out_dyn(g.y, g.y_dtype, (int64_t)tok * g.ldy + row, acc[i].x);
          if (tok + 1 < g.m) store_out_dyn(g.y, g.y_dtype, (int64_t)(tok + 1) * g.ldy + row, acc[i].y);
        }
      }
    }
  }
  if (PROF && warp >= 4 && lane == 0 && (warp == 4 || warp == 7 || warp == 19)) {
    // three of the consumer warps (lane quarters 0, 3, 3; column groups 0, 0, 3): clocks waiting for scale planes,
    // activation unit, MMA result; clocks scaling
    const int o = warp == 4 ? 5 : warp == 7 ? 9 : 12;
    g.prof[blockIdx.x * 16 + o] = pw[1];
    g.prof[blockIdx.x * 16 + o + 1] = pw[2];
    g.prof[blockIdx.x * 16 + o + 2] = pw[3];
    if (warp == 4) g.prof[blockIdx.x * 16 + 8] = pw[0];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 3) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int KIND>
static int launch(const Args& g, int sm_count, cudaStream_t st) {
  static bool configured[64];
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  constexpr int smem = Smem<KIND>::TOTAL;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  if (dev < 0 || dev >= 64) return GSQ_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm2_kernel<KIND, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm2_kernel<KIND, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm2_kernel<KIND, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  const int n_items = g.n_row_tiles * g.n_tok_blocks;
  const int grid = n_items < sm_count ? n_items : sm_count;
  if (g.dump) {
    gemm2_kernel<KIND, 1><<<grid, THREADS, smem, st>>>(g);
  } else if (g.prof) {
    gemm2_kernel<KIND, 2><<<grid, THREADS, smem, st>>>(g);
  } else {
    gemm2_kernel<KIND, 0><<<grid, THREADS, smem, st>>>(g);
  }
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}

}  // namespace g2

// gsq_gemm.cu
int* gemm_dump_pointer();

static unsigned long long* g_prof = nullptr;
unsigned long long* gemm_profile_pointer() { return g_prof; }

int gemm2_error_flag(int* flag) {
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(flag, g2::g_error, sizeof(int)));
  return GSQ_OK;
}

// bytes of the activation units of m tokens x k columns (tokens padded to whole blocks of 256)
size_t gemm2_tile_bytes(int64_t m, int64_t k, int ggml_type) {
  const int64_t tb = (m + g2::NT - 1) / g2::NT;
  return (size_t)(tb * (k / 256) * 8 * g2::unit_bytes(ggml_type == GSQ_TYPE_Q4_K));
}

bool gemm2_applies(int ggml_type, int packed, int64_t rows) {
  return ggml_type == GSQ_TYPE_Q4_K || ggml_type == GSQ_TYPE_IQ4_XS || (ggml_type == GSQ_TYPE_IQ3_S && packed && rows % 16 == 0);
}

// x_tiles: the output of quantize_q8_1_tiles for this type
int gemm2_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_tiles, int64_t m,
               int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream) {
  if (m == 0 || rows == 0) return GSQ_OK;
  if (m < 0 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !x_tiles || !y) return GSQ_ERR_UNSUPPORTED;
  if (rows > INT32_MAX || k > INT32_MAX || m > INT32_MAX) return GSQ_ERR_TOO_LARGE;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs || !gemm2_applies(ggml_type, packed, rows)) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  DeviceInfo di;
  const int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  g2::Args g;
  g.w = (const uint8_t*)w;
  g.row_bytes = row_bytes;
  g.nrows = (int)rows;
  g.k = (int)k;
  g.xt = (const uint8_t*)x_tiles;
  g.m = (int)m;
  g.y = y;
  g.y_dtype = y_dtype;
  g.ldy = y_row_stride;
  g.n_row_tiles = (int)((rows + g2::TR - 1) / g2::TR);
  g.n_tok_blocks = (int)((m + g2::NT - 1) / g2::NT);
  g.dump = gemm_dump_pointer();
  g.prof = g_prof;
  cudaStream_t st = (cudaStream_t)stream;
  switch (ggml_type) {
    case GSQ_TYPE_IQ3_S: return g2::launch<G2_IQ3S>(g, di.sm_count, st);
    case GSQ_TYPE_Q4_K: return g2::launch<G2_Q4K>(g, di.sm_count, st);
    default: return g2::launch<G2_IQ4XS>(g, di.sm_count, st);
  }
}

}  // namespace gsq

extern "C" int gsq_debug_gemm_profile(unsigned long long* clocks) {
  gsq::g_prof = clocks;
  return GSQ_OK;
}
