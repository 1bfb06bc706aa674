// Prefill GEMMs with the sub-scales folded into the tensor-core operand (sm_100a: tcgen05 kind::f16 with fp32
// accumulators in tensor memory), warp-specialised. Two kernels:
//   gemm3_kernel      repacked IQ3_S; exact integer slice sums, scaled per 32-value slice (described next);
//   gemm3_acc_kernel  repacked IQ3_S, IQ4_XS, Q4_K; the activation scale in the operand too, sums over a superblock
//                     in tensor memory, one FMA per result and superblock (described further down, at the kernel).
//
// Serves gsq_linear above the small-batch row counts for IQ3_S in the fragment-ordered layout: the reference's
// iq3_packed_mmq (plugin/vllm_gguf_plugin/csrc/lcpp_owned_iq3_mma.cu:768-970) and, behind it, MMQ (csrc/lcpp/ggml/src/
// ggml-cuda/mmq.cuh:961-1385). Their arithmetic per 32-value slice s: an exact int32 dot product C_s of the int8
// weights g (codebook value times sign, odd, |g| <= 15) and the int8 activation quants q, then
//   y += d_w * (1 + 2 ls_s) * float(C_s) * d_x[token, s].
// With int8 operands (gsq_gemm2.cu) the int -> float conversion and two FMAs per result and slice bound the kernel at
// a tenth of the tensor cores' rate. Here the integer sub-scale moves into the operand: the weight tile holds
// (1 + 2 ls_s) * g as fp16 (odd integers, magnitude <= 465, exact), the activation tile holds q as fp16 (exact), and
// the tensor cores return S_s = (1 + 2 ls_s) * C_s in fp32 -- an integer below 2^21, so every partial sum is exact
// whatever the order of accumulation. What is left per result and slice is y += (S_s * d_w) * d_x[token, s]: no
// conversion, and the tensor cores' instruction covers 256 tokens. The integer sums C_s = S_s / (1 + 2 ls_s) are still
// there bit for bit (debug dump mode divides them out and the tests compare them with the integer oracle).
//
// A CTA owns a tile of 128 weight rows x 256 tokens and walks K half a superblock (4 slices = 128 values) at a time:
//   * 7 producer warps fetch the raw records of the 128 rows (cp.async, one superblock ahead) and decode a half ONCE
//     into the fp16 tile (K-major core matrices) plus d_w per row;
//   * one thread streams the activation units (one slice x 256 tokens, already in operand order in global memory:
//     quantize_q8_1_tiles_kernel, fp16 layout) with one bulk copy per unit into a 5-deep ring and issues the MMAs:
//     2 instructions of 128 x 256 x 16 per unit into one half of tensor memory, the other half being drained
//     meanwhile. (N = 256 reads the weight slice from shared memory once per 256 tokens; with four N = 64 sub-tiles
//     the operand reads alone took a third of the shared-memory bandwidth.)
//   * 16 consumer warps (4 per tensor-memory lane quarter, 64 columns each) read the sums with tcgen05.ld and
//     accumulate y += (S * d_w) * d_x in 64 fp32 registers per thread over the whole of K.
// All hand-offs are mbarriers; every wait is bounded and raises a CTA-wide abort flag (and the sticky device flag read
// by gsq_device_error_flag) instead of hanging.
#include <cuda_fp16.h>

#include "gsq_common.cuh"
#include "gsq_tables.h"
#include "gsq_tc.cuh"

namespace gsq {
namespace g3 {

using namespace tc;

constexpr int TR = 128;                 // weight rows per tile (MMA M)
constexpr int NT = 256;                 // tokens per tile (MMA N)
constexpr int PROD_WARPS = 7;
constexpr int PROD_THREADS = PROD_WARPS * 32;
constexpr int MMA_WARP = PROD_WARPS;    // bulk copies + MMA issue
constexpr int CONS_WARP0 = 8;           // first consumer warp (a multiple of 4: tensor-memory lane quarter = warp % 4)
constexpr int CONS_WARPS = 16;
constexpr int THREADS = (CONS_WARP0 + CONS_WARPS) * 32;
// registers: 768 threads start with 80 each; the two producer warpgroups give up 32 each, the four consumer
// warpgroups take 16 each
constexpr int PROD_REGS = 48, CONS_REGS = 96;
constexpr int SL_A = 8192;              // bytes of one slice of the weight tile (128 rows x 32 fp16)
constexpr int SL_B = 16384;             // bytes of the quants of one activation unit (256 tokens x 32 fp16)
constexpr int STAGE_A = 4 * SL_A;       // half a superblock
constexpr int A_STAGES = 2;
constexpr int B_SLOTS = 5;
constexpr int B_AHEAD = 3;              // units the bulk copies run ahead of the MMAs
constexpr int RAW_STAGES = 2;
constexpr int RAWB = 8 * 1760;          // one superblock of 128 rows: 8 records
constexpr int UB = SL_B + NT * 4;        // one activation unit: quants as fp16, then d
constexpr int SA_STAGE = 5 * TR * 4;    // per stage: d_w [128], then 1 + 2 ls [4 slices][128] (read in dump mode only)
constexpr int TMEM_COLS = 512;
constexpr int GRIDB = 512 * 64;         // codebook: (g, -g) biased by 128, 8 replicas

struct Args {
  const uint8_t* w;
  int64_t row_bytes;
  int nrows;
  int k;
  const uint8_t* xt;   // activation units: [token block of 256][superblock][slice][UB]
  int m;
  void* y;
  int y_dtype;
  int64_t ldy;
  int n_row_tiles, n_tok_blocks;
  int* dump;           // debug: raw int32 slice sums [m][nrows][k / 32]
  unsigned long long* prof;  // debug: per CTA 16 clock counts (see gsq_debug_gemm_profile)
  uint32_t wait_hint;  // 0: poll the mbarriers with short sleeps; else nanoseconds the hardware suspends a waiting thread per try
  const float* inv_scale;  // gemm3_acc_kernel: 2^-e per token of the padded range (behind the last unit)
};

struct Smem {
  static constexpr int BAR = 0;
  static constexpr int GRID = 1024;
  static constexpr int RAW = GRID + GRIDB;
  static constexpr int A = RAW + RAW_STAGES * RAWB;
  static constexpr int SA = A + A_STAGES * STAGE_A;
  static constexpr int B = SA + A_STAGES * SA_STAGE;
  static constexpr int TOTAL = B + B_SLOTS * UB;
};
static_assert(Smem::A % 128 == 0 && Smem::B % 128 == 0 && RAWB % 16 == 0 && UB % 16 == 0, "operand and copy alignment");

__device__ int g_error = 0;

__device__ const uint32_t g_iq3s_grid3[512] = GSQ_IQ3S_GRID_INIT;

// K-major fp16 operand slice (32 values along K): four core matrices of a row group 128 bytes apart, consecutive 8-row
// groups 512 bytes apart; one MMA (K = 16) takes two of the four, the second MMA starts 256 bytes further.
__device__ __forceinline__ uint64_t desc16(uint32_t addr) { return tc::smem_desc(addr, 128, 512); }
// Instruction descriptor: D = f32, A = B = f16, both K-major, N = 256, M = 128, dense.
__host__ __device__ constexpr uint32_t idesc() {
  return (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TR >> 4) << 24);
}

__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, __half2 b, __half2 c) {
  const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), b, c);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// ---------------------------------------------------------------------------------------------
// Producers.

__device__ __forceinline__ void fetch_raw(const Args& g, int rt, int sb, uint8_t* raw, int ptid) {
  // 8 records of 1760 contiguous bytes (16 rows each); records past the last row are not fetched (nor decoded)
  const uint32_t dst = saddr(raw);
  for (int i = ptid; i < 8 * 110; i += PROD_THREADS) {
    const int rec = i / 110, c = i - rec * 110;
    const int row0 = rt * TR + 16 * rec;
    if (row0 < g.nrows) cp_async16(dst + rec * 1760 + c * 16, g.w + (int64_t)row0 * g.row_bytes + (int64_t)sb * 1760 + c * 16);
  }
}

// Two slices (2 SP, 2 SP + 1 of half HF) of one record, by one warp. Lane (gq = lane / 4, t = lane % 4) holds, of rows
// gq and gq + 8 and every slice, the 4-value groups 2t, 2t + 1 (field f = 4 s + 2 h + e at bit 9 f of its nine index
// words; sign bits pre-arranged as byte-permute selectors): the 8 values 8t .. 8t + 7 of the slice, one 16-byte row of
// a core matrix. The codebook bytes in shared memory carry a bias of 128, so that a byte b under the high byte 0x64 is
// the fp16 number 1152 + value; (1152 + value) * sub - 1152 * sub in one fused multiply-add is value * sub, exact.
// Thread i of the warp plays lane (i % 8) * 4 + i / 8 of the record, so that the eight threads of a store's quarter
// phase write the 128 contiguous bytes of one core matrix (threads in record order would hit four banks four times).
template <int HF, int SP>
__device__ __forceinline__ void decode_pair(const uint8_t* p, uint8_t* a, float* sa, const uint8_t* grid, int rec, int thread) {
  const int gq = thread & 7, t = thread >> 3, lane = 4 * gq + t;
  const uint32_t lane_off = (uint32_t)(thread & 7) << 3;
  uint32_t idx[5];
  if (HF == 0) {
    const uint4 ia = *reinterpret_cast<const uint4*>(p + 16 * lane);
    idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
    idx[4] = *reinterpret_cast<const uint32_t*>(p + 512 + 16 * lane);
  } else {
    const uint4 ib = *reinterpret_cast<const uint4*>(p + 512 + 16 * lane);
    idx[0] = ib.x; idx[1] = ib.y; idx[2] = ib.z; idx[3] = ib.w;
    idx[4] = *reinterpret_cast<const uint32_t*>(p + 1024 + 4 * lane);
  }
  const uint32_t sgw = *reinterpret_cast<const uint32_t*>(p + 1152 + 16 * lane + 8 * HF + 4 * SP);
  const uint2 sc = *reinterpret_cast<const uint2*>(p + 1664 + 8 * gq);
  const uint32_t dd = *reinterpret_cast<const uint32_t*>(p + 1728 + 4 * gq);
#pragma unroll
  for (int sl = 0; sl < 2; ++sl) {
    const int s_half = 2 * SP + sl;        // slice within the half = slice of the stage
    const int s = 4 * HF + s_half;         // slice within the superblock
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t wv[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int f = 4 * s_half + 2 * h + e;          // field within the half
        const int bit = 9 * f + 16 * HF, word = bit >> 5, off = bit & 31;
        uint32_t v;
        if (off + 9 <= 32) {
          v = off >= 6 ? idx[word] >> (off >= 6 ? off - 6 : 0) : idx[word] << (off < 6 ? 6 - off : 0);
        } else {
          v = __funnelshift_r(idx[word], idx[word + 1], off - 6);
        }
        const uint2 gp = *reinterpret_cast<const uint2*>(grid + ((v & 0x7FC0u) | lane_off));
        const int fl = f & 7, sh = 16 * (fl >> 2) + (fl & 3) - 2;
        const uint32_t sgs = sh >= 0 ? sgw >> (sh >= 0 ? sh : 0) : sgw << (sh < 0 ? -sh : 0);
        wv[e] = prmt(gp.x, gp.y, (sgs & 0x4444u) | 0x3210u);
      }
      const int r = 16 * rec + gq + 8 * h;
      const uint32_t scw = h ? sc.y : sc.x;
      const int sub = 1 + 2 * (int)((scw >> (4 * s)) & 15u);
      const __half subh = __int2half_rn(sub);
      const __half2 sub2 = __half2half2(subh);
      const __half2 nb2 = __half2half2(__hmul(__float2half_rn(-1152.0f), subh));   // exact: 1152 * sub = 2^7 * (9 sub)
      uint4 o;
      o.x = hfma2_bits(prmt(wv[0], 0x64646464u, 0x4140u), sub2, nb2);
      o.y = hfma2_bits(prmt(wv[0], 0x64646464u, 0x4342u), sub2, nb2);
      o.z = hfma2_bits(prmt(wv[1], 0x64646464u, 0x4140u), sub2, nb2);
      o.w = hfma2_bits(prmt(wv[1], 0x64646464u, 0x4342u), sub2, nb2);
      *reinterpret_cast<uint4*>(a + s_half * SL_A + (r >> 3) * 512 + t * 128 + (r & 7) * 16) = o;
      if (t == sl) sa[(1 + s_half) * TR + r] = (float)sub;
      if (SP == 0 && sl == 0 && t == 2) sa[r] = h2f(dd >> (16 * h));
    }
  }
}

template <int HF>
__device__ __forceinline__ void decode_half(const uint8_t* raw, uint8_t* a, float* sa, const uint8_t* grid, int nrows_left,
                                            int pwarp, int lane) {
  // 16 pieces over 7 warps: the two halves of a superblock start at different warps, so that over a superblock the
  // warps get 5, 5, 5, 5, 4, 4, 4 pieces (the warps meet at a barrier once per superblock)
  for (int u = HF ? (pwarp + PROD_WARPS - 2) % PROD_WARPS : pwarp; u < 16; u += PROD_WARPS) {
    const int rec = u >> 1;
    if (16 * rec >= nrows_left) continue;
    if (u & 1) {
      decode_pair<HF, 1>(raw + rec * 1760, a, sa, grid, rec, lane);
    } else {
      decode_pair<HF, 0>(raw + rec * 1760, a, sa, grid, rec, lane);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Consumers.

// 8 columns of one slice: y += (S * d_w) * d_x. Packed fp32 instructions: measured against scalar ones and against
// packed multiplies with scalar FMAs (to use both fp32 pipes), all-packed is fastest: issue slots count for more.
__device__ __forceinline__ void scale8(const uint32_t (&c)[8], const float* bd, float dw, float2* acc) {
  const float2 dw2 = make_float2(dw, dw);
#pragma unroll
  for (int j4 = 0; j4 < 2; ++j4) {
    const float4 d = *reinterpret_cast<const float4*>(bd + 4 * j4);
    const float2 s0 = __fmul2_rn(make_float2(__uint_as_float(c[4 * j4]), __uint_as_float(c[4 * j4 + 1])), dw2);
    const float2 s1 = __fmul2_rn(make_float2(__uint_as_float(c[4 * j4 + 2]), __uint_as_float(c[4 * j4 + 3])), dw2);
    acc[2 * j4] = __ffma2_rn(s0, make_float2(d.x, d.y), acc[2 * j4]);
    acc[2 * j4 + 1] = __ffma2_rn(s1, make_float2(d.z, d.w), acc[2 * j4 + 1]);
  }
}

__device__ __forceinline__ void dump8(const Args& g, const uint32_t (&c)[8], float sub, int row, int tok0, int slice) {
  if (row >= g.nrows) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (tok0 + j < g.m) g.dump[((int64_t)(tok0 + j) * g.nrows + row) * (g.k >> 5) + slice] = __float2int_rn(__uint_as_float(c[j]) / sub);
  }
}

// ring cursor: position and phase parity of an n-deep ring of mbarriers 8 bytes apart
struct Ring {
  uint32_t i, ph;
  __device__ __forceinline__ void next(uint32_t n) {
    if (++i == n) { i = 0; ph ^= 1u; }
  }
};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) gemm3_kernel(const Args g) {
  constexpr bool DUMP = MODE == 1, PROF = MODE == 2;
  unsigned long long pw[4] = {0ull, 0ull, 0ull, 0ull};   // debug (MODE 2): clocks spent in this thread's waits / work
  auto tick = [&]() -> unsigned long long { return PROF ? (unsigned long long)clock64() : 0ull; };
  extern __shared__ __align__(1024) uint8_t smem[];
  using S = Smem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // barriers (8 bytes each): a_full[2] a_empty[2] b_full[5] b_empty[5] d_full[2] d_empty[2]
  const uint32_t bar0 = saddr(smem + S::BAR);
  const uint32_t a_full = bar0, a_empty = bar0 + 16, b_full = bar0 + 32, b_empty = b_full + 8 * B_SLOTS,
                 d_full = b_empty + 8 * B_SLOTS, d_empty = d_full + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::BAR + 260);
  const uint32_t hint = g.wait_hint;
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    return hint ? mbar_wait_hw(bar, parity, hint, abort_flag, &g_error) : mbar_wait(bar, parity, abort_flag, &g_error);
  };

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
  if (warp == MMA_WARP) tmem_alloc(saddr(tmem_slot), TMEM_COLS);
  for (int i = tid; i < 512; i += THREADS) {
    const uint32_t gv = g_iq3s_grid3[i];
    const uint32_t pos = gv ^ 0x80808080u, neg = (~gv + 0x01010101u) ^ 0x80808080u;   // no codebook byte is zero
    uint4* dst = reinterpret_cast<uint4*>(smem + S::GRID + i * 64);
#pragma unroll
    for (int r2 = 0; r2 < 4; ++r2) dst[r2] = make_uint4(pos, neg, pos, neg);
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
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PROD_REGS));
    const int ptid = tid;
    int f_item = blockIdx.x, f_sb = 0;        // fetch cursor over the (item, superblock) pairs of this CTA
    auto fetch_next = [&](uint32_t n_fetch) {
      if (f_item < n_items) {
        fetch_raw(g, item_rt(f_item), f_sb, smem + S::RAW + (n_fetch & 1u) * RAWB, ptid);
        if (++f_sb == nsb) { f_sb = 0; f_item += gridDim.x; }
      }
      cp_async_commit();
    };
    fetch_next(0);
    uint32_t ns = 0;            // superblocks so far
    Ring ra = {0u, 0u};         // weight-tile stages
    bool alive = true;
    // (after a wait has given up the loop still runs to its end, without work: every producer thread passes the
    // same number of named barriers)
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const int rt = item_rt(item);
      for (int sb = 0; sb < nsb; ++sb, ++ns) {
        cp_async_wait<0>();                                  // this thread's pieces of superblock ns have landed
        asm volatile("bar.sync 1, %0;" ::"n"(PROD_THREADS) : "memory");   // everyone's have; everyone is done with ns - 1
        fetch_next(ns + 1);
        const uint8_t* raw = smem + S::RAW + (ns & 1u) * RAWB;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const unsigned long long p0 = tick();
          alive = alive && wait(a_empty + 8 * ra.i, ra.ph ^ 1u);
          const unsigned long long p1 = tick();
          pw[0] += p1 - p0;
          if (alive) {
            uint8_t* a = smem + S::A + ra.i * STAGE_A;
            float* sa = reinterpret_cast<float*>(smem + S::SA + ra.i * SA_STAGE);
            if (hf == 0) {
              decode_half<0>(raw, a, sa, smem + S::GRID, g.nrows - rt * TR, warp, lane);
            } else {
              decode_half<1>(raw, a, sa, smem + S::GRID, g.nrows - rt * TR, warp, lane);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor-core reads
            mbar_arrive(a_full + 8 * ra.i);
            pw[1] += tick() - p1;
          }
          ra.next(A_STAGES);
        }
      }
    }
    if (PROF && tid == 0) {
      g.prof[blockIdx.x * 16 + 0] = pw[0];   // producer: waiting for a free stage
      g.prof[blockIdx.x * 16 + 1] = pw[1];   // producer: decoding
    }
    cp_async_wait<0>();
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------------------------ bulk copies + MMA issue
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PROD_REGS));
    if (lane == 0) {
      // This one thread is on every unit's critical path: everything it does per unit is kept to a few dozen
      // instructions (no divisions, descriptors and source addresses by increments).
      const uint32_t id = idesc();
      const uint64_t desc_hi = desc16(0u) & 0xFFFFFFFF00000000ull;
      const uint32_t a_lo0 = (uint32_t)desc16(saddr(smem + S::A)), b_lo0 = (uint32_t)desc16(saddr(smem + S::B));
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
        for (int st2 = 0; st2 < 2 * nsb && alive; ++st2) {
          const unsigned long long m0 = tick();
          alive = wait(a_full + 8 * ra.i, ra.ph);
          pw[0] += tick() - m0;
          if (!alive) break;
          const uint32_t a_lo = a_lo0 + ra.i * (STAGE_A >> 4);
#pragma unroll 1
          for (int sl = 0; sl < 4; ++sl) {
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
            const uint32_t b_lo = b_lo0 + rb.i * (UB >> 4), as_lo = a_lo + sl * (SL_A >> 4);
            const uint32_t d_addr = tmem_base + rd.i * 256;
            mma_f16(d_addr, desc(as_lo), desc(b_lo), id, 0u);
            mma_f16(d_addr, desc(as_lo + (256 >> 4)), desc(b_lo + (256 >> 4)), id, 1u);
            mma_commit(d_full + 8 * rd.i);
            rb.next(B_SLOTS);
            rd.next(2);
            ++n_used;
            load_next();   // after the MMAs are on their way: the copy for B_AHEAD units further on
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(CONS_REGS));
    const int cw = warp - CONS_WARP0, q4 = warp & 3, cg = cw >> 2;   // tensor-memory lane quarter = warp id mod 4
    const int r_in = 32 * q4 + lane;
    const uint32_t t_warp = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)(64 * cg);
    Ring ra = {0u, 0u}, rb = {0u, 0u}, rd = {0u, 0u};
    bool alive = true;
    for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
      const int rt = item_rt(item), tok0 = item_tb(item) * NT + 64 * cg;
      float2 acc[32];   // this thread's row x 64 tokens
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.0f, 0.0f);
      for (int st2 = 0; st2 < 2 * nsb && alive; ++st2) {
        const unsigned long long c0t = tick();
        alive = wait(a_full + 8 * ra.i, ra.ph);   // the producers' d_w plane is visible
        pw[0] += tick() - c0t;
        if (!alive) break;
        const float* sa = reinterpret_cast<const float*>(smem + S::SA + ra.i * SA_STAGE);
        const float dw = sa[r_in];
#pragma unroll 1
        for (int sl = 0; sl < 4; ++sl) {
          const unsigned long long c1t = tick();
          alive = alive && wait(b_full + 8 * rb.i, rb.ph);   // the unit's d_x are visible
          const unsigned long long c2t = tick();
          alive = alive && wait(d_full + 8 * rd.i, rd.ph);
          const unsigned long long c3t = tick();
          pw[1] += c2t - c1t;
          pw[2] += c3t - c2t;
          if (alive) {
            tc_fence_after();
            const float* bd = reinterpret_cast<const float*>(smem + S::B + rb.i * UB + SL_B) + 64 * cg;
            const uint32_t t_unit = t_warp + rd.i * 256;
            const float sub = DUMP ? sa[(1 + sl) * TR + r_in] : 0.0f;
            const int slice = (st2 >> 1) * 8 + 4 * (st2 & 1) + sl;
            // chunks of 8 columns, the next chunk's load in flight while one is scaled
            uint32_t c0[8], c1[8];
            tmem_ld8(t_unit, c0);
#pragma unroll
            for (int ch = 0; ch < 8; ch += 2) {
              tmem_ld_wait();
              tmem_ld8(t_unit + 8 * (ch + 1), c1);
              if (DUMP) dump8(g, c0, sub, rt * TR + r_in, tok0 + 8 * ch, slice);
              scale8(c0, bd + 8 * ch, dw, &acc[4 * ch]);
              tmem_ld_wait();
              if (ch < 6) tmem_ld8(t_unit + 8 * (ch + 2), c0);
              if (DUMP) dump8(g, c1, sub, rt * TR + r_in, tok0 + 8 * (ch + 1), slice);
              scale8(c1, bd + 8 * (ch + 1), dw, &acc[4 * (ch + 1)]);
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
        if (lane == 0 && alive) mbar_arrive(a_empty + 8 * ra.i);   // the stage's planes (and, the MMAs done, its tile) are free
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
  if (PROF && lane == 0 && (warp == CONS_WARP0 || warp == CONS_WARP0 + 3 || warp == CONS_WARP0 + 15)) {
    // three of the consumer warps: clocks waiting for d_w planes, activation unit, MMA result; clocks scaling
    const int o = warp == CONS_WARP0 ? 5 : warp == CONS_WARP0 + 3 ? 9 : 12;
    g.prof[blockIdx.x * 16 + o] = pw[1];
    g.prof[blockIdx.x * 16 + o + 1] = pw[2];
    g.prof[blockIdx.x * 16 + o + 2] = pw[3];
    if (warp == CONS_WARP0) g.prof[blockIdx.x * 16 + 8] = pw[0];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// The same product with the activation scale inside the operand as well, so that tensor memory accumulates over a whole
// superblock and the sums are read once per 256 values of K instead of once per 32.
//
// Operands: the weight tile as above ((1 + 2 ls) * g, exact); the activation tile holds p = d_x * q * 2^e[token]
// as fp16, either rounded (HU = 1: relative error of an element up to 2^-11, of a result about 2e-4 of its row norm) or
// as the pair hi = fp16(p), lo = fp16(p - hi) multiplied one after the other into the same accumulator (HU = 2: 22 bits
// of every p, the fp32 accumulation's own rounding is what is left). 2^e[token] keeps every p below 2^14 whatever
// the activations' range (quantize_q8_1_tiles_kernel, scaled products). Per superblock and result the consumers do one
// FMA, y' += C * d_w, and at the end of K y = y' * 2^-e[token].
//
// Against the kernel above: the activation slots are released by the MMAs' completion (tcgen05.commit), not by the
// consumers, and so are the weight stages; the consumers take d_w from the record in global memory (2 bytes per
// thread and superblock, fetched one superblock ahead), so nothing but tensor memory couples them to the rest.
constexpr int HB = 16384;               // one fp16 plane of one slice: 256 tokens x 32 values
constexpr int UBA = 2 * HB;             // one copy and one turn of the MMA thread: two slices (HU = 1) or hi + lo of one (HU = 2)
constexpr int ACC_B_SLOTS = 3;
constexpr int ACC_B_AHEAD = 2;

// weight formats of this kernel: IQ3_S in the fragment-ordered layout (decode_pair above), IQ4_XS and Q4_K in GGUF order
enum { WK_IQ3S = 0, WK_IQ4XS = 1, WK_Q4K = 2 };
constexpr int RAWB_IQ4XS = 128 * 136;   // one superblock of 128 rows
constexpr int RAWB_Q4K = 128 * 144;
constexpr int SUB = 8192;               // Q4_K: one unit of per-slice activation terms (256 tokens x 16 fp16)
constexpr int AMINB = 4096;             // Q4_K: the per-slice weight terms of a superblock that go with them (128 rows x 16 fp16)

template <int WK>
struct SmemAcc {
  static constexpr int BAR = 0;
  static constexpr int GRID = 1024;
  static constexpr int RAWBK = WK == WK_IQ3S ? RAWB : WK == WK_IQ4XS ? RAWB_IQ4XS : RAWB_Q4K;
  static constexpr int RAW = GRID + (WK == WK_IQ3S ? GRIDB : 0);   // (IQ4_XS: a 16-entry table, in registers)
  static constexpr int A = (RAW + RAW_STAGES * RAWBK + 127) / 128 * 128;
  static constexpr int B = A + A_STAGES * STAGE_A;
  static constexpr int AMIN = B + ACC_B_SLOTS * UBA;     // Q4_K only: the operand of per-slice weight terms, then one unit of sums
  static constexpr int BS = AMIN + (WK == WK_Q4K ? AMINB : 0);
  static constexpr int SAX = BS + (WK == WK_Q4K ? SUB : 0);   // scratch the IQ3_S decoder writes its scale planes to (unused here)
  static constexpr int TOTAL = SAX + (WK == WK_IQ3S ? SA_STAGE : 0);
};
static_assert(SmemAcc<0>::B % 128 == 0 && SmemAcc<1>::B % 128 == 0 && SmemAcc<2>::B % 128 == 0 && RAWB_IQ4XS % 16 == 0, "operand alignment");
static_assert(SmemAcc<0>::TOTAL <= 227 * 1024 && SmemAcc<1>::TOTAL <= 227 * 1024 && SmemAcc<2>::TOTAL <= 227 * 1024, "shared memory budget");

__constant__ __align__(16) int8_t c_iq4nl3[16] = GSQ_IQ4NL_VALUES_INIT;

__device__ __forceinline__ void fetch_raw_iq4xs(const Args& g, int rt, int sb, uint8_t* raw, int ptid) {
  // 128 blocks of 136 bytes, 8-byte aligned in global memory; rows past the last one repeat it (never stored)
  const uint32_t dst = saddr(raw);
  for (int i = ptid; i < 128 * 17; i += PROD_THREADS) {
    const int r = i / 17, c = i - r * 17;
    const int row = min(rt * TR + r, g.nrows - 1);
    cp_async8(dst + r * 136 + c * 8, g.w + (int64_t)row * g.row_bytes + (int64_t)sb * 136 + c * 8);
  }
}

// 8 nibbles of v -> table bytes: lo = those of the low nibbles of bytes 0..3, hi = of the high nibbles
__device__ __forceinline__ void iq4_lookup3(uint32_t v, const uint32_t (&tb)[4], uint32_t& lo, uint32_t& hi) {
  const uint32_t s01 = v & 0x7777u, s23 = (v >> 16) & 0x7777u;
  const uint32_t pick01 = 0x3210u | ((v & 0x8888u) >> 1), pick23 = 0x3210u | (((v >> 16) & 0x8888u) >> 1);
  const uint32_t r01 = prmt(prmt(tb[0], tb[1], s01), prmt(tb[2], tb[3], s01), pick01);
  const uint32_t r23 = prmt(prmt(tb[0], tb[1], s23), prmt(tb[2], tb[3], s23), pick23);
  lo = prmt(r01, r23, 0x6420u);
  hi = prmt(r01, r23, 0x7531u);
}

// IQ4_XS, one (row, slice) of half HF of a superblock: 16 bytes of 4-bit indices (low nibbles = values 0..15 of the
// slice, high nibbles 16..31) -> 32 fp16 numbers (ls - 32) * table[index], four 16-byte rows of core matrices. `tb`
// is the table with 128 added to every byte, so that a byte under the high byte 0x64 is the fp16 number 1152 + value
// and one fused multiply-add gives value * (ls - 32) with a single rounding (exact up to 2048 in magnitude; of the
// larger products, up to 4064, the odd ones round to even: a relative error of at most 2.4e-4 of that element).
// item = slice-in-half * 128 + row: a store's 8 threads write one whole 128-byte core matrix.
template <int HF>
__device__ __forceinline__ void decode_iq4xs_f16(const uint8_t* raw, uint8_t* a, int item, const uint32_t (&tb)[4]) {
  const int r = item & 127, s_half = item >> 7, p = 4 * HF + s_half;
  const uint8_t* b = raw + r * 136;
  const uint2 hdr = *reinterpret_cast<const uint2*>(b);
  const uint2 qa = *reinterpret_cast<const uint2*>(b + 8 + 16 * p), qb = *reinterpret_cast<const uint2*>(b + 16 + 16 * p);
  const uint32_t v[4] = {qa.x, qa.y, qb.x, qb.y};
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) iq4_lookup3(v[e], tb, lo[e], hi[e]);
  const uint32_t ls = ((hdr.y >> (4 * p)) & 0xFu) | (((hdr.x >> (16 + 2 * p)) & 3u) << 4);
  const __half subh = __int2half_rn((int)ls - 32);
  const __half2 sub2 = __half2half2(subh);
  const __half2 nb2 = __half2half2(__hmul(__float2half_rn(-1152.0f), subh));   // exact: 2^7 * 9 * (ls - 32)
  uint8_t* dst = a + s_half * SL_A + (r >> 3) * 512 + (r & 7) * 16;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const uint32_t w0 = t < 2 ? lo[2 * t] : hi[2 * t - 4], w1 = t < 2 ? lo[2 * t + 1] : hi[2 * t - 3];
    uint4 o;
    o.x = hfma2_bits(prmt(w0, 0x64646464u, 0x4140u), sub2, nb2);
    o.y = hfma2_bits(prmt(w0, 0x64646464u, 0x4342u), sub2, nb2);
    o.z = hfma2_bits(prmt(w1, 0x64646464u, 0x4140u), sub2, nb2);
    o.w = hfma2_bits(prmt(w1, 0x64646464u, 0x4342u), sub2, nb2);
    *reinterpret_cast<uint4*>(dst + t * 128) = o;
  }
}

__device__ __forceinline__ void fetch_raw_q4k(const Args& g, int rt, int sb, uint8_t* raw, int ptid) {
  const uint32_t dst = saddr(raw);
  for (int i = ptid; i < 128 * 9; i += PROD_THREADS) {
    const int r = i / 9, c = i - r * 9;
    const int row = min(rt * TR + r, g.nrows - 1);
    cp_async16(dst + r * 144 + c * 16, g.w + (int64_t)row * g.row_bytes + (int64_t)sb * 144 + c * 16);
  }
}

// Q4_K: the scale the consumers apply per superblock and row. Normally d itself, so that the weight operand holds the
// integers sc * q exactly; where dmin is more than 64 times d (or d is zero), dmin / 64, so that the minimum-term
// operand -(dmin / sigma) * m * 16 stays inside fp16 (at most 64 * 63 * 16).
__device__ __forceinline__ float q4k_sigma(uint32_t d_dmin) {
  const float d = h2f(d_dmin), dm = h2f(d_dmin >> 16);
  float sigma = fabsf(dm) > 64.0f * fabsf(d) ? fabsf(dm) * (1.0f / 64.0f) : d;
  return sigma == 0.0f ? 1.0f : sigma;
}
// 6-bit scales and minimums of slices 2 jj, 2 jj + 1 (low / high byte of the results) from the 12 packed bytes
__device__ __forceinline__ void q4k_scale_min(const uint4& hdr, int jj, uint32_t& sc, uint32_t& mn) {
  const uint32_t selh = (jj & 1) ? 0x4432u : 0x4410u;
  const uint32_t A = prmt(hdr.y, 0u, selh), B = prmt(hdr.z, 0u, selh), C = prmt(hdr.w, 0u, selh);
  sc = jj < 2 ? (A & 0x3F3Fu) : ((C & 0x0F0Fu) | ((A & 0xC0C0u) >> 2));
  mn = jj < 2 ? (B & 0x3F3Fu) : (((C >> 4) & 0x0F0Fu) | ((B & 0xC0C0u) >> 2));
}

// Q4_K, item = (slice pair, 16-byte piece, row) of half HF: 16 bytes of quants (low nibbles: 16 values of slice 2 jj,
// high nibbles: of slice 2 jj + 1) -> (d / sigma) * sc * q as fp16, two 16-byte core-matrix rows per slice. A nibble
// under the high byte 0x64 is the fp16 number 1024 + q; (1024 + q) * f - 1024 * f in one fused multiply-add is q * f
// with one rounding (none whenever sigma = d: f is the integer sc).
template <int HF>
__device__ __forceinline__ void decode_q4k_f16(const uint8_t* raw, uint8_t* a, int item) {
  const int r = item & 127, sub = item >> 7, jj = 2 * HF + (sub >> 1), half = sub & 1;
  const uint8_t* b = raw + r * 144;
  const uint4 hdr = *reinterpret_cast<const uint4*>(b);
  const uint4 v = *reinterpret_cast<const uint4*>(b + 16 + 32 * jj + 16 * half);
  uint32_t sc, mn;
  q4k_scale_min(hdr, jj, sc, mn);
  const float ratio = h2f(hdr.x) / q4k_sigma(hdr.x);    // exactly 1 in the normal case
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int hi = 0; hi < 2; ++hi) {
    const __half fh = __float2half_rn(ratio * (float)((sc >> (8 * hi)) & 0xFFu));
    const __half2 f2 = __half2half2(fh);
    const __half2 nb2 = __half2half2(__hmul(__float2half_rn(-1024.0f), fh));
    uint8_t* dst = a + (2 * (sub >> 1) + hi) * SL_A + (r >> 3) * 512 + (2 * half) * 128 + (r & 7) * 16;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint32_t n0 = (w[2 * c] >> (4 * hi)) & 0x0F0F0F0Fu, n1 = (w[2 * c + 1] >> (4 * hi)) & 0x0F0F0F0Fu;
      uint4 o;
      o.x = hfma2_bits(prmt(n0, 0x64646464u, 0x4140u), f2, nb2);
      o.y = hfma2_bits(prmt(n0, 0x64646464u, 0x4342u), f2, nb2);
      o.z = hfma2_bits(prmt(n1, 0x64646464u, 0x4140u), f2, nb2);
      o.w = hfma2_bits(prmt(n1, 0x64646464u, 0x4342u), f2, nb2);
      *reinterpret_cast<uint4*>(dst + c * 128) = o;
    }
  }
}

// Q4_K, one row of a superblock: the weight terms that multiply per-slice quantities of the activations, as a
// 16-column operand for the unit the quantiser writes per superblock (layout with sums): K chunk 0 =
// -(dmin / sigma) * m_s * 16, against half(sum x) * 2^(e - 4): the minimum term; chunk 1 = 8 * (d / sigma) * sc_s * 16
// (128 sc exactly when sigma = d), against what the fp16 rounding of the slice's products lost in total / 16: the
// quants 0..15 act on the rounding errors as 8 + (q - 8), and this gives the 8's share back, so that only the
// centred part of the weights sees them. The consumers scale the superblock's accumulator by sigma.
__device__ __forceinline__ void q4k_slice_terms(const uint8_t* raw, uint8_t* amin, int r) {
  const uint4 hdr = *reinterpret_cast<const uint4*>(raw + r * 144);
  const float sigma = q4k_sigma(hdr.x);
  const float fm = -16.0f * h2f(hdr.x >> 16) / sigma, fs = 128.0f * (h2f(hdr.x) / sigma);
  __half2 hm[4], hs[4];
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) {
    uint32_t sc, mn;
    q4k_scale_min(hdr, jj, sc, mn);
    hm[jj] = __floats2half2_rn(fm * (float)(mn & 0xFFu), fm * (float)(mn >> 8));
    hs[jj] = __floats2half2_rn(fs * (float)(sc & 0xFFu), fs * (float)(sc >> 8));
  }
  uint8_t* dst = amin + (r >> 3) * 256 + (r & 7) * 16;
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(hm);
  *reinterpret_cast<uint4*>(dst + 128) = *reinterpret_cast<const uint4*>(hs);
}

// PAIR: two CTAs (a cluster) share an item of 256 weight rows x 256 tokens. Each decodes its own 128 rows and copies
// only its half of the tokens of every activation unit; the MMAs (M = 256, cta_group::2) are issued by CTA 0 and read
// both halves, so every CTA moves half the activation bytes from L2 and through its shared memory per result. CTA 0's
// barriers collect both CTAs' "weight stage decoded" and "sums drained" arrivals; CTA 1 reports each landed unit to
// CTA 0 (b_peer); MMA completion is signalled to both CTAs at once.
template <int WK, int HU, bool PROF, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1) gemm3_acc_kernel(const Args g) {
  unsigned long long pw[4] = {0ull, 0ull, 0ull, 0ull};
  auto tick = [&]() -> unsigned long long { return PROF ? (unsigned long long)clock64() : 0ull; };
  extern __shared__ __align__(1024) uint8_t smem[];
  using S = SmemAcc<WK>;
  static_assert(WK == WK_IQ3S || !PAIR, "pairs of CTAs: IQ3_S only");
  static_assert(WK != WK_Q4K || HU == 1, "Q4_K: the rounded form only");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  constexpr int NB = PAIR ? 2 * ACC_B_SLOTS : ACC_B_SLOTS;      // activation slots (half the bytes each for a pair)
  constexpr int AHEAD = PAIR ? 2 * ACC_B_AHEAD : ACC_B_AHEAD;
  constexpr int UBC = PAIR ? UBA / 2 : UBA;                     // bytes of a unit this CTA holds
  constexpr int PL = PAIR ? HB / 2 : HB;                        // ... of one of its two planes
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = crank == 0u;
  const int group = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, n_groups = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // barriers (8 bytes each): a_full[2] a_empty[2] d_full[2] d_empty[2] b_full[NB] b_empty[NB] b_peer[NB]
  const uint32_t bar0 = saddr(smem + S::BAR);
  const uint32_t a_full = bar0, a_empty = bar0 + 16, d_full = bar0 + 32, d_empty = bar0 + 48, b_full = bar0 + 64,
                 b_empty = b_full + 8 * NB, b_peer = b_empty + 8 * NB;
  static_assert(64 + 3 * 8 * 2 * ACC_B_SLOTS + 32 <= 256, "barrier area");
  const uint32_t s_full = bar0 + 64 + 3 * 8 * 2 * ACC_B_SLOTS, s_empty = s_full + 16;   // Q4_K: units of sums
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::BAR + 260);
  const uint32_t hint = g.wait_hint;
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    if (PAIR) return mbar_wait_cluster(bar, parity, abort_flag, &g_error);
    return hint ? mbar_wait_hw(bar, parity, hint, abort_flag, &g_error) : mbar_wait(bar, parity, abort_flag, &g_error);
  };
  // arrival on a barrier of CTA 0 (the own barrier without a pair)
  auto arrive_leader = [&](uint32_t bar) {
    if (PAIR) mbar_arrive_cluster(mapa(bar, 0u));
    else mbar_arrive(bar);
  };

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(a_full + 8 * i, PROD_THREADS * (PAIR ? 2 : 1));
      mbar_init(a_empty + 8 * i, 1);          // the MMAs that read the stage have completed
      mbar_init(d_full + 8 * i, 1);
      mbar_init(d_empty + 8 * i, CONS_WARPS * (PAIR ? 2 : 1));
      mbar_init(s_full + 8 * i, 1);
      mbar_init(s_empty + 8 * i, 1);
    }
    for (int i = 0; i < NB; ++i) {
      mbar_init(b_full + 8 * i, 1);
      mbar_init(b_empty + 8 * i, 1);          // the MMAs that read the slot have completed
      mbar_init(b_peer + 8 * i, 1);           // CTA 1's half of the unit has landed
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    if (PAIR) tmem_alloc_pair(saddr(tmem_slot), TMEM_COLS);
    else tmem_alloc(saddr(tmem_slot), TMEM_COLS);
  }
  if (WK == WK_IQ3S) {
    for (int i = tid; i < 512; i += THREADS) {
      const uint32_t gv = g_iq3s_grid3[i];
      const uint32_t pos = gv ^ 0x80808080u, neg = (~gv + 0x01010101u) ^ 0x80808080u;
      uint4* dst = reinterpret_cast<uint4*>(smem + S::GRID + i * 64);
#pragma unroll
      for (int r2 = 0; r2 < 4; ++r2) dst[r2] = make_uint4(pos, neg, pos, neg);
    }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nsb = g.k >> 8;
  // items of a CTA (or pair): row tiles (pairs of them) fastest; a pair's second CTA may own a tile past the last row
  const int n_rt = PAIR ? (g.n_row_tiles + 1) / 2 : g.n_row_tiles;
  const int n_items = n_rt * g.n_tok_blocks;
  auto item_rt = [&](int item) { return PAIR ? 2 * (item % n_rt) + (int)crank : item % n_rt; };
  auto item_tb = [&](int item) { return item / n_rt; };

  if (warp < PROD_WARPS) {
    // ------------------------------------------------------------------------------------ producers
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PROD_REGS));
    const int ptid = tid;
    int f_item = group, f_sb = 0;
    auto fetch_next = [&](uint32_t n_fetch) {
      if (f_item < n_items) {
        if (WK == WK_IQ3S) fetch_raw(g, item_rt(f_item), f_sb, smem + S::RAW + (n_fetch & 1u) * S::RAWBK, ptid);
        else if (WK == WK_IQ4XS) fetch_raw_iq4xs(g, item_rt(f_item), f_sb, smem + S::RAW + (n_fetch & 1u) * S::RAWBK, ptid);
        else fetch_raw_q4k(g, item_rt(f_item), f_sb, smem + S::RAW + (n_fetch & 1u) * S::RAWBK, ptid);
        if (++f_sb == nsb) { f_sb = 0; f_item += n_groups; }
      }
      cp_async_commit();
    };
    fetch_next(0);
    uint32_t ns = 0;
    Ring ra = {0u, 0u};
    bool alive = true;
    float* sa = reinterpret_cast<float*>(smem + S::SAX);
    uint32_t tb[4] = {0u, 0u, 0u, 0u};
    if (WK == WK_IQ4XS) {
      const uint32_t* tw = reinterpret_cast<const uint32_t*>(c_iq4nl3);
#pragma unroll
      for (int e = 0; e < 4; ++e) tb[e] = tw[e] ^ 0x80808080u;
    }
    for (int item = group; item < n_items; item += n_groups) {
      const int rt = item_rt(item);
      for (int sb = 0; sb < nsb; ++sb, ++ns) {
        cp_async_wait<0>();
        asm volatile("bar.sync 1, %0;" ::"n"(PROD_THREADS) : "memory");
        fetch_next(ns + 1);
        const uint8_t* raw = smem + S::RAW + (ns & 1u) * S::RAWBK;
        int it4 = ptid;   // IQ4_XS, Q4_K: this thread's next item of the superblock, 1024 of them in half order
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const unsigned long long p0 = tick();
          alive = alive && wait(a_empty + 8 * ra.i, ra.ph ^ 1u);
          const unsigned long long p1 = tick();
          pw[0] += p1 - p0;
          if (alive) {
            uint8_t* a = smem + S::A + ra.i * STAGE_A;
            if (WK == WK_Q4K) {
              // (the minimum-term operand belongs to the first half's stage: the MMA that reads it is issued before
              // that half's, so the stage's release covers it)
              if (hf == 0 && ptid < TR) q4k_slice_terms(raw, smem + S::AMIN, ptid);
              for (; it4 < 512 * (hf + 1); it4 += PROD_THREADS) {
                if (hf == 0) decode_q4k_f16<0>(raw, a, it4);
                else decode_q4k_f16<1>(raw, a, it4 - 512);
              }
            } else if (WK == WK_IQ4XS) {
              // 512 (slice, row) items per half over 224 threads: the thread carries on where it stopped in the first
              // half, so the superblock takes 5 rounds, not 2 x 3
              for (; it4 < 512 * (hf + 1); it4 += PROD_THREADS) {
                if (hf == 0) decode_iq4xs_f16<0>(raw, a, it4, tb);
                else decode_iq4xs_f16<1>(raw, a, it4 - 512, tb);
              }
            } else if (hf == 0) {
              decode_half<0>(raw, a, sa, smem + S::GRID, g.nrows - rt * TR, warp, lane);
            } else {
              decode_half<1>(raw, a, sa, smem + S::GRID, g.nrows - rt * TR, warp, lane);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor-core reads
            arrive_leader(a_full + 8 * ra.i);
            pw[1] += tick() - p1;
          }
          ra.next(A_STAGES);
        }
      }
    }
    if (PROF && tid == 0) {
      g.prof[(size_t)blockIdx.x * 16 + 0] = pw[0];   // producer: waiting for a free stage
      g.prof[(size_t)blockIdx.x * 16 + 1] = pw[1];   // producer: decoding
    }
    cp_async_wait<0>();
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------------------------ bulk copies + MMA issue
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PROD_REGS));
    if (lane == 0) {
      const uint32_t id = PAIR ? (idesc() & ~(0x1Fu << 24)) | ((uint32_t)(2 * TR >> 4) << 24) : idesc();   // M = 256 over the pair
      const uint64_t desc_hi = desc16(0u) & 0xFFFFFFFF00000000ull;
      const uint32_t a_lo0 = (uint32_t)desc16(saddr(smem + S::A)), b_lo0 = (uint32_t)desc16(saddr(smem + S::B));
      auto desc = [&](uint32_t lo) { return desc_hi | (uint64_t)lo; };
      const uint32_t b_smem0 = saddr(smem + S::B);
      // load cursor over the stream of half-units (item, superblock, slice, hi / lo), ACC_B_AHEAD ahead of the MMAs
      int l_item = group, l_u = 0;
      const int units_item = 4 * HU * nsb;
      const uint8_t* l_base = nullptr;
      auto load_item = [&]() {
        if (l_item < n_items) l_base = g.xt + (int64_t)item_tb(l_item) * units_item * UBA;
      };
      load_item();
      Ring rl = {0u, 0u};
      uint32_t n_loaded = 0;
      bool alive = true;
      auto load_next = [&]() {
        if (l_item >= n_items || !alive) return;
        const unsigned long long l0 = tick();
        alive = wait(b_empty + 8 * rl.i, rl.ph ^ 1u);
        pw[3] += tick() - l0;
        if (!alive) return;
        mbar_expect_tx(b_full + 8 * rl.i, UBC);
        if (PAIR) {
          // this CTA's tokens of the unit's two planes: 128 of the 256 (the first or second 8 KB of each plane)
          const uint8_t* src = l_base + (int64_t)l_u * UBA + crank * PL;
          bulk_g2s(b_smem0 + rl.i * UBC, src, PL, b_full + 8 * rl.i);
          bulk_g2s(b_smem0 + rl.i * UBC + PL, src + HB, PL, b_full + 8 * rl.i);
        } else {
          bulk_g2s(b_smem0 + rl.i * UBC, l_base + (int64_t)l_u * UBA, UBA, b_full + 8 * rl.i);
        }
        rl.next(NB);
        ++n_loaded;
        if (++l_u == units_item) {
          l_u = 0;
          l_item += n_groups;
          load_item();
        }
      };
      // Q4_K: the units of sums, one per (item, superblock); one slot, refilled for the next superblock as soon as this
      // superblock's two instructions on it have completed
      int s_item = group, s_sb = 0;
      uint32_t n_sums_loaded = 0, n_sums_used = 0;
      Ring rsl = {0u, 0u}, rsu = {0u, 0u};
      const uint8_t* s_region = g.xt + (int64_t)g.n_tok_blocks * units_item * UBA;
      auto load_sums = [&]() {
        if (WK != WK_Q4K || s_item >= n_items || !alive) return;
        alive = wait(s_empty + 8 * rsl.i, rsl.ph ^ 1u);
        if (!alive) return;
        mbar_expect_tx(s_full + 8 * rsl.i, SUB);
        bulk_g2s(saddr(smem + S::BS) + rsl.i * SUB, s_region + ((int64_t)item_tb(s_item) * nsb + s_sb) * SUB, SUB, s_full + 8 * rsl.i);
        rsl.next(1);
        ++n_sums_loaded;
        if (++s_sb == nsb) { s_sb = 0; s_item += n_groups; }
      };
      load_sums();
      for (int i = 0; i < AHEAD; ++i) load_next();
      Ring ra = {0u, 0u}, rb = {0u, 0u}, rd = {0u, 0u};
      uint32_t n_used = 0;
      if (PAIR && !leader) {
        // CTA 1 issues no MMAs: it reports each landed unit to CTA 0 and keeps its own copies going
        for (int item = group; item < n_items && alive; item += n_groups) {
          for (int u = 0; u < units_item && alive; ++u) {
            alive = wait(b_full + 8 * rb.i, rb.ph);
            if (!alive) break;
            mbar_arrive_cluster(mapa(b_peer + 8 * rb.i, 0u));
            rb.next(NB);
            ++n_used;
            load_next();
          }
        }
      } else
      for (int item = group; item < n_items && alive; item += n_groups) {
        for (int st2 = 0; st2 < 2 * nsb && alive; ++st2) {
          const unsigned long long m0 = tick();
          alive = wait(a_full + 8 * ra.i, ra.ph);
          pw[0] += tick() - m0;
          if (!alive) break;
          if ((st2 & 1) == 0) {
            // a new superblock starts a new sum: the consumers have drained this half of tensor memory
            const unsigned long long m1 = tick();
            alive = wait(d_empty + 8 * rd.i, rd.ph ^ 1u);
            pw[1] += tick() - m1;
            if (!alive) break;
          }
          const uint32_t a_lo = a_lo0 + ra.i * (STAGE_A >> 4);
          const uint32_t d_addr = tmem_base + rd.i * 256;
          if (WK == WK_Q4K && (st2 & 1) == 0) {
            // the superblock's sum starts with the terms in per-slice sums (minimums, offset of the centred quants)
            alive = alive && wait(s_full + 8 * rsu.i, rsu.ph);
            if (!alive) break;
            tc_fence_after();
            mma_f16(d_addr, tc::smem_desc(saddr(smem + S::AMIN), 128, 256), tc::smem_desc(saddr(smem + S::BS) + rsu.i * SUB, 128, 256), id, 0u);
            mma_commit(s_empty + 8 * rsu.i);
            rsu.next(1);
            ++n_sums_used;
          }
#pragma unroll 1
          for (int u2 = 0; u2 < 2 * HU && alive; ++u2) {
            const unsigned long long m3 = tick();
            alive = wait(b_full + 8 * rb.i, rb.ph);
            if (PAIR) alive = alive && wait(b_peer + 8 * rb.i, rb.ph);
            pw[2] += tick() - m3;
            if (!alive) break;
            tc_fence_after();
            const uint32_t b_lo = b_lo0 + rb.i * (UBC >> 4);
            // HU = 1: slices 2 u2, 2 u2 + 1 against the unit's two planes; HU = 2: slice u2 against hi, then lo
            const uint32_t as0 = a_lo + (HU == 1 ? 2 * u2 : u2) * (SL_A >> 4), as1 = HU == 1 ? as0 + (SL_A >> 4) : as0;
            const uint32_t first = (WK != WK_Q4K && (st2 & 1) == 0 && u2 == 0) ? 0u : 1u;
            if (PAIR) {
              mma_f16_pair(d_addr, desc(as0), desc(b_lo), id, first);
              mma_f16_pair(d_addr, desc(as0 + (256 >> 4)), desc(b_lo + (256 >> 4)), id, 1u);
              mma_f16_pair(d_addr, desc(as1), desc(b_lo + (PL >> 4)), id, 1u);
              mma_f16_pair(d_addr, desc(as1 + (256 >> 4)), desc(b_lo + ((PL + 256) >> 4)), id, 1u);
              mma_commit_pair(b_empty + 8 * rb.i);
            } else {
              mma_f16(d_addr, desc(as0), desc(b_lo), id, first);
              mma_f16(d_addr, desc(as0 + (256 >> 4)), desc(b_lo + (256 >> 4)), id, 1u);
              mma_f16(d_addr, desc(as1), desc(b_lo + (PL >> 4)), id, 1u);
              mma_f16(d_addr, desc(as1 + (256 >> 4)), desc(b_lo + ((PL + 256) >> 4)), id, 1u);
              mma_commit(b_empty + 8 * rb.i);
            }
            rb.next(NB);
            ++n_used;
            load_next();
            if (WK == WK_Q4K && (st2 & 1) == 0 && u2 == 0) load_sums();   // the next superblock's sums
          }
          if (!alive) break;
          if (PAIR) mma_commit_pair(a_empty + 8 * ra.i);
          else mma_commit(a_empty + 8 * ra.i);
          ra.next(A_STAGES);
          if (st2 & 1) {
            if (PAIR) mma_commit_pair(d_full + 8 * rd.i);
            else mma_commit(d_full + 8 * rd.i);
            rd.next(2);
          }
        }
      }
      if (PROF) {
        g.prof[(size_t)blockIdx.x * 16 + 2] = pw[0];   // MMA thread: waiting for a decoded weight tile
        g.prof[(size_t)blockIdx.x * 16 + 3] = pw[1];   // MMA thread: waiting for a drained half of tensor memory
        g.prof[(size_t)blockIdx.x * 16 + 4] = pw[2];   // MMA thread: waiting for an activation half-unit to land
        g.prof[(size_t)blockIdx.x * 16 + 5] = pw[3];   // MMA thread: waiting for a free activation slot

      }
      if (!alive) {
        // a wait gave up: let the copies already issued land (bounded) before the CTA's shared memory goes away
        for (; n_used < n_loaded; ++n_used) {
          wait(b_full + 8 * rb.i, rb.ph);
          rb.next(NB);
        }
        for (; n_sums_used < n_sums_loaded; ++n_sums_used) {
          wait(s_full + 8 * rsu.i, rsu.ph);
          rsu.next(1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------------------------ consumers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(CONS_REGS));
    const int cw = warp - CONS_WARP0, q4 = warp & 3, cg = cw >> 2;
    const int r_in = 32 * q4 + lane;
    const uint32_t t_warp = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)(64 * cg);
    Ring rd = {0u, 0u};
    bool alive = true;
    for (int item = group; item < n_items && alive; item += n_groups) {
      const int rt = item_rt(item), tok0 = item_tb(item) * NT + 64 * cg;
      const int row = rt * TR + r_in;
      const bool row_ok = row < g.nrows;
      // fp16 d of this thread's row. IQ3_S: halfword (row % 16) / 8 of word row % 8 at byte 1728 of its 16-row record;
      // IQ4_XS: the first two bytes of the row's block; Q4_K: the scale worked out from its first four (d, dmin)
      const uint8_t* dwp = WK == WK_IQ3S ? g.w + (int64_t)(row & ~15) * g.row_bytes + 1728 + 4 * (row & 7) + 2 * ((row >> 3) & 1)
                                         : g.w + (int64_t)row * g.row_bytes;
      auto load_dw = [&](int sb) -> float {
        if (!row_ok) return 0.0f;
        if (WK == WK_Q4K) return q4k_sigma(*reinterpret_cast<const uint32_t*>(dwp + (int64_t)sb * 144));
        return h2f(*reinterpret_cast<const uint16_t*>(dwp + (int64_t)sb * (WK == WK_IQ3S ? 1760 : 136)));
      };
      float2 acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.0f, 0.0f);
      float dw_next = load_dw(0);
      for (int sb = 0; sb < nsb && alive; ++sb) {
        const float dw = dw_next;
        if (sb + 1 < nsb) dw_next = load_dw(sb + 1);
        const unsigned long long c2t = tick();
        alive = wait(d_full + 8 * rd.i, rd.ph);
        const unsigned long long c3t = tick();
        pw[2] += c3t - c2t;
        if (!alive) break;
        tc_fence_after();
        const uint32_t t_unit = t_warp + rd.i * 256;
        const float2 dw2 = make_float2(dw, dw);
        uint32_t c0[8], c1[8];
        tmem_ld8(t_unit, c0);
#pragma unroll
        for (int ch = 0; ch < 8; ch += 2) {
          tmem_ld_wait();
          tmem_ld8(t_unit + 8 * (ch + 1), c1);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            acc[4 * ch + j] = __ffma2_rn(make_float2(__uint_as_float(c0[2 * j]), __uint_as_float(c0[2 * j + 1])), dw2, acc[4 * ch + j]);
          tmem_ld_wait();
          if (ch < 6) tmem_ld8(t_unit + 8 * (ch + 2), c0);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            acc[4 * (ch + 1) + j] = __ffma2_rn(make_float2(__uint_as_float(c1[2 * j]), __uint_as_float(c1[2 * j + 1])), dw2, acc[4 * (ch + 1) + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_leader(d_empty + 8 * rd.i);
        pw[3] += tick() - c3t;
        rd.next(2);
      }
      if (alive && row_ok) {
        const float* inv = g.inv_scale + tok0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int tok = tok0 + 2 * i;
          const float2 is = *reinterpret_cast<const float2*>(inv + 2 * i);   // (the padded range: always readable)
          if (tok < g.m) store_out_dyn(g.y, g.y_dtype, (int64_t)tok * g.ldy + row, acc[i].x * is.x);
          if (tok + 1 < g.m) store_out_dyn(g.y, g.y_dtype, (int64_t)(tok + 1) * g.ldy + row, acc[i].y * is.y);
        }
      }
    }
  }
  if (PROF && lane == 0 && (warp == CONS_WARP0 || warp == CONS_WARP0 + 3 || warp == CONS_WARP0 + 15)) {
    const int o = warp == CONS_WARP0 ? 6 : warp == CONS_WARP0 + 3 ? 9 : 12;
    g.prof[(size_t)blockIdx.x * 16 + o + 1] = pw[2];   // consumer: waiting for a superblock's sums
    g.prof[(size_t)blockIdx.x * 16 + o + 2] = pw[3];   // consumer: reading and scaling them
  }
  tc_fence_before();
  if (PAIR) {
    cluster_sync_all();   // no arrival of a peer is still on its way to this CTA's barriers, no MMA reads its memory
    if (warp == MMA_WARP) tmem_dealloc_pair(tmem_base, TMEM_COLS);
  } else {
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int WK, int HU, bool PROF, bool PAIR>
static int launch_acc(const Args& g, int sm_count, cudaStream_t st) {
  constexpr int smem = SmemAcc<WK>::TOTAL;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static bool configured[64];
  static int max_clusters[64];
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GSQ_ERR_UNSUPPORTED;
  auto kern = gemm3_acc_kernel<WK, HU, PROF, PAIR>;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = PAIR ? 2 : 1;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (!configured[dev]) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    max_clusters[dev] = sm_count;
    if (PAIR) {
      // how many pairs the device runs at once (an SM without a free neighbour in its GPC stays out)
      cfg.gridDim = dim3(2u * (unsigned)sm_count);
      int n = 0;
      GSQ_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
      if (n < 1) return GSQ_ERR_UNSUPPORTED;
      max_clusters[dev] = n;
    }
    configured[dev] = true;
  }
  const int n_items = (PAIR ? (g.n_row_tiles + 1) / 2 : g.n_row_tiles) * g.n_tok_blocks;
  const int groups = n_items < max_clusters[dev] ? n_items : max_clusters[dev];
  cfg.gridDim = dim3((unsigned)(PAIR ? 2 * groups : groups));
  GSQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, g));
  return GSQ_OK;
}

// acc: 0 = integer slice sums; 1 / 2 = sums over a superblock on one / two planes of scaled products; pair: two CTAs per item
static int launch(const Args& g, int sm_count, int wk, int acc, int pair, cudaStream_t st) {
  if (acc) {
    if (g.dump) return GSQ_ERR_UNSUPPORTED;   // no per-slice integer sums exist in this form
    if (wk == WK_Q4K) {
      if (pair || acc != 1) return GSQ_ERR_UNSUPPORTED;
      return g.prof ? launch_acc<WK_Q4K, 1, true, false>(g, sm_count, st) : launch_acc<WK_Q4K, 1, false, false>(g, sm_count, st);
    }
    if (wk == WK_IQ4XS) {
      if (pair) return GSQ_ERR_UNSUPPORTED;
      if (acc == 1) return g.prof ? launch_acc<WK_IQ4XS, 1, true, false>(g, sm_count, st) : launch_acc<WK_IQ4XS, 1, false, false>(g, sm_count, st);
      return g.prof ? launch_acc<WK_IQ4XS, 2, true, false>(g, sm_count, st) : launch_acc<WK_IQ4XS, 2, false, false>(g, sm_count, st);
    }
    if (acc == 1) {
      if (pair) return g.prof ? launch_acc<WK_IQ3S, 1, true, true>(g, sm_count, st) : launch_acc<WK_IQ3S, 1, false, true>(g, sm_count, st);
      return g.prof ? launch_acc<WK_IQ3S, 1, true, false>(g, sm_count, st) : launch_acc<WK_IQ3S, 1, false, false>(g, sm_count, st);
    }
    if (pair) return g.prof ? launch_acc<WK_IQ3S, 2, true, true>(g, sm_count, st) : launch_acc<WK_IQ3S, 2, false, true>(g, sm_count, st);
    return g.prof ? launch_acc<WK_IQ3S, 2, true, false>(g, sm_count, st) : launch_acc<WK_IQ3S, 2, false, false>(g, sm_count, st);
  }
  if (wk != WK_IQ3S) return GSQ_ERR_UNSUPPORTED;
  static bool configured[64];
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  constexpr int smem = Smem::TOTAL;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  if (dev < 0 || dev >= 64) return GSQ_ERR_UNSUPPORTED;
  if (!configured[dev]) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm3_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm3_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    GSQ_CUDA_TRY(cudaFuncSetAttribute(gemm3_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  const int n_items = g.n_row_tiles * g.n_tok_blocks;
  const int grid = n_items < sm_count ? n_items : sm_count;
  if (g.dump) {
    gemm3_kernel<1><<<grid, THREADS, smem, st>>>(g);
  } else if (g.prof) {
    gemm3_kernel<2><<<grid, THREADS, smem, st>>>(g);
  } else {
    gemm3_kernel<0><<<grid, THREADS, smem, st>>>(g);
  }
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}

}  // namespace g3

// gsq_gemm.cu, gsq_gemm2.cu
int* gemm_dump_pointer();
unsigned long long* gemm_profile_pointer();

static int g_wait_hint = 0;

int gemm3_error_flag(int* flag) {
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(flag, g3::g_error, sizeof(int)));
  return GSQ_OK;
}

// bytes of the fp16 activation units of m tokens x k columns (tokens padded to whole blocks of 256). acc: 0 = quants
// and d per slice, 1 / 2 = scaled products in one / two fp16 planes, then one float per token
// (acc = 1 with `sums`: Q4_K's layout, one more 8 KB unit per token block and superblock)
size_t gemm3_tile_bytes(int64_t m, int64_t k, int acc, int sums) {
  const int64_t tb = (m + g3::NT - 1) / g3::NT;
  if (acc) return (size_t)(tb * (k / 256) * (8 * acc * g3::HB + (sums ? g3::SUB : 0)) + tb * g3::NT * 4);
  return (size_t)(tb * (k / 256) * 8 * g3::UB);
}

bool gemm3_applies(int ggml_type, int packed, int64_t rows) { return ggml_type == GSQ_TYPE_IQ3_S && packed && rows % 16 == 0; }
// the forms that sum over a superblock in tensor memory also serve IQ4_XS (GGUF order)
bool gemm3_acc_applies(int ggml_type, int packed, int64_t rows) {
  return gemm3_applies(ggml_type, packed, rows) || ((ggml_type == GSQ_TYPE_IQ4_XS || ggml_type == GSQ_TYPE_Q4_K) && !packed);
}

// x_tiles: the output of quantize_tiles_host in the fp16 layout that goes with acc (Q8_TILES_H16, _F16S, _F16S2)
int gemm3_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_tiles, int64_t m,
               int64_t k, void* y, int y_dtype, int64_t y_row_stride, int acc, int pair, void* stream) {
  if (m == 0 || rows == 0) return GSQ_OK;
  if (m < 0 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !x_tiles || !y) return GSQ_ERR_UNSUPPORTED;
  if (rows > INT32_MAX || k > INT32_MAX || m > INT32_MAX) return GSQ_ERR_TOO_LARGE;
  const bool iq4 = ggml_type == GSQ_TYPE_IQ4_XS, q4k = ggml_type == GSQ_TYPE_Q4_K;
  if (iq4 || q4k ? (!acc || packed || row_bytes != (k / 256) * (iq4 ? 136 : 144)) : (!gemm3_applies(ggml_type, packed, rows) || row_bytes != (k / 256) * 110))
    return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  DeviceInfo di;
  const int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  g3::Args g;
  g.w = (const uint8_t*)w;
  g.row_bytes = row_bytes;
  g.nrows = (int)rows;
  g.k = (int)k;
  g.xt = (const uint8_t*)x_tiles;
  g.m = (int)m;
  g.y = y;
  g.y_dtype = y_dtype;
  g.ldy = y_row_stride;
  g.n_row_tiles = (int)((rows + g3::TR - 1) / g3::TR);
  g.n_tok_blocks = (int)((m + g3::NT - 1) / g3::NT);
  g.dump = gemm_dump_pointer();
  g.prof = gemm_profile_pointer();
  g.wait_hint = (uint32_t)g_wait_hint;
  g.inv_scale = acc ? reinterpret_cast<const float*>((const uint8_t*)x_tiles + (size_t)g.n_tok_blocks * (k / 256) * (8 * acc * g3::HB + (q4k ? g3::SUB : 0))) : nullptr;
  if (acc < 0 || acc > 2) return GSQ_ERR_UNSUPPORTED;
  return g3::launch(g, di.sm_count, iq4 ? g3::WK_IQ4XS : q4k ? g3::WK_Q4K : g3::WK_IQ3S, acc, pair, (cudaStream_t)stream);
}

}  // namespace gsq

extern "C" int gsq_debug_gemm_wait_hint(int ns) {
  const int old = gsq::g_wait_hint;
  gsq::g_wait_hint = ns > 0 ? ns : 0;
  return old;
}
