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
#include "gsq_f1_codec.cuh"

namespace gsq {

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
