// gsq_linear: the whole product for callers that hand over X as it is (fp32 / fp16 / bf16) -- what the reference's
// ops that quantise for themselves do inside one call (lcpp_mul_mat_q, lcpp_mul_mat_mma_k, lcpp_mul_mat_iq3_packed:
// plugin/vllm_gguf_plugin/csrc/lcpp_shim.cu:626-671, 753-909). The activation quantiser and its output layout are
// chosen together with the kernel: 128-value blocks [K/128][M] for the small-batch tensor-core kernel and the
// lockstep GEMM, operand-ordered tiles for the prefill GEMM, 36-byte blocks for the dp4a kernel.
#include "gsq_common.cuh"

namespace gsq {

// gsq_mmv.cu
bool mmv_applies(int ggml_type, int packed, int64_t rows, int64_t m);
int mmv_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* xq, int x_layout,
             int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream, int* dump,
             const gsq_peer_reduce* pr = nullptr);
// gsq_gemm2.cu
bool gemm2_applies(int ggml_type, int packed, int64_t rows);
size_t gemm2_tile_bytes(int64_t m, int64_t k, int ggml_type);
int gemm2_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_tiles, int64_t m,
               int64_t k, void* y, int y_dtype, int64_t y_row_stride, void* stream);
// gsq_gemm3.cu
bool gemm3_applies(int ggml_type, int packed, int64_t rows);
bool gemm3_acc_applies(int ggml_type, int packed, int64_t rows);
size_t gemm3_tile_bytes(int64_t m, int64_t k, int acc, int sums);
int gemm3_host(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x_tiles, int64_t m,
               int64_t k, void* y, int y_dtype, int64_t y_row_stride, int acc, int pair, void* stream);
// gsq_quantize.cu
int quantize_tiles_host(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride, int layout, void* out, void* stream);
// gsq_gemm.cu
int* gemm_dump_pointer();
int gemm_variant();

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

static int g_prefill_precision = GSQ_PREFILL_ROUNDED;

}  // namespace gsq

extern "C" int gsq_prefill_precision(int mode) {
  const int old = gsq::g_prefill_precision;
  if (mode >= GSQ_PREFILL_ROUNDED && mode <= GSQ_PREFILL_INTEGER) gsq::g_prefill_precision = mode;
  return old;
}

extern "C" size_t gsq_linear_scratch_bytes(int64_t rows, int64_t m, int64_t k, int ggml_type, int packed) {
  if (m <= 0 || k <= 0) return 0;
  const size_t mmq = (size_t)(k / 128) * (size_t)m * 144, q81 = (size_t)(k / 32) * (size_t)m * 36;
  size_t tiles = gsq::gemm3_applies(ggml_type, packed, rows) ? 0 : gsq::gemm2_tile_bytes(m, k, ggml_type);
  if (gsq::gemm3_acc_applies(ggml_type, packed, rows)) {
    // the fp16-operand forms: one plane of scaled products per slice, two where the split form is selected (or forced
    // through the debug switch); and the integer-sum form's units, which the dump of those sums selects
    const int v = gsq::gemm_variant();
    const int planes = (gsq::g_prefill_precision == GSQ_PREFILL_SPLIT || v == 5 || v == 9) ? 2 : 1;
    const size_t t3 = gsq::gemm3_tile_bytes(m, k, planes, ggml_type == GSQ_TYPE_Q4_K), t0 = gsq::gemm3_tile_bytes(m, k, 0, 0);
    tiles = tiles > t3 ? tiles : t3;
    tiles = tiles > t0 ? tiles : t0;
  }
  size_t b = mmq > tiles ? mmq : tiles;
  b = b > q81 ? b : q81;
  return gsq::align256(b);
}

extern "C" int gsq_linear(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x,
                          int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* y, int y_dtype,
                          int64_t y_row_stride, void* scratch, size_t scratch_bytes, void* stream) {
  using namespace gsq;
  if (m == 0 || rows == 0) return GSQ_OK;
  if (m < 0 || rows < 0 || k <= 0 || k % 256 != 0 || !w || !x || !y) return GSQ_ERR_UNSUPPORTED;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  if (!scratch || scratch_bytes < gsq_linear_scratch_bytes(rows, m, k, ggml_type, packed)) return GSQ_ERR_SCRATCH;
  const int layout = gsq_q8_layout_for_type(ggml_type);
  int rc;
  // 1..48 rows: the small-batch tensor-core kernel on 128-value blocks, where it serves the type and the shape fits
  if (mmv_applies(ggml_type, packed, rows, m)) {
    rc = gsq_quantize_q8_1_mmq(x, x_dtype, m, k, x_row_stride, layout, scratch, stream);
    if (rc != GSQ_OK) return rc;
    rc = mmv_host(w, row_bytes, rows, ggml_type, packed, scratch, 1, m, k, y, y_dtype, y_row_stride, stream, gemm_dump_pointer());
    if (rc != 1000) return rc;  // 1000: declined, the activations of this shape do not fit its staging area
  }
  // The prefill GEMMs on operand-ordered units, where their 128-row x 256-token items can occupy the GPU. Measured
  // against the lockstep kernel (64-token tiles, K split over a cluster when tiles are few) on 17408 x 5120,
  // 5120 x 5120 and 5120 x 17408: the fp16-operand kernel wins from 256 tokens on, and from 128 where the weight
  // alone gives half an SM count of row tiles; the int8 one from 512, and from 192 on the tall weights.
  const int variant = gemm_variant();
  const bool tall = (rows + 127) / 128 >= 74;
  const bool big3 = m >= 256 || (m >= 128 && tall);
  const bool big = m >= 512 || (m >= 192 && tall);
  // repacked IQ3_S and IQ4_XS: the kernels with the sub-scales folded into fp16 operands (variant 4 keeps the int8
  // kernel for them)
  if (gemm3_acc_applies(ggml_type, packed, rows) && (variant == 3 || variant >= 5 || (variant == 0 && big3))) {
    // the form that accumulates over a superblock in tensor memory, on one or two fp16 planes of scaled products, or the
    // one with integer slice sums (also whenever the debug dump of those sums is on); variants 5 / 6 / 7 force one
    int acc = g_prefill_precision == GSQ_PREFILL_ROUNDED ? 1 : g_prefill_precision == GSQ_PREFILL_SPLIT ? 2 : 0;
    // IQ4_XS: (ls - 32) * value reaches 4064 and is not always exact in fp16, so only the rounded form is offered on
    // fp16 operands; the split setting takes the int8 kernel's integer sums instead
    // (and Q4_K, whose minimum term is folded in with one rounding of dmin / d * m)
    if ((ggml_type == GSQ_TYPE_IQ4_XS || ggml_type == GSQ_TYPE_Q4_K) && acc == 2) acc = 0;
    int pair = 0;
    if (variant == 5 || variant == 9) acc = 2;
    if (variant == 6 || variant == 8) acc = 1;
    if (variant == 8 || variant == 9) pair = gemm3_applies(ggml_type, packed, rows) ? 1 : 0;
    if (variant == 7 || gemm_dump_pointer()) acc = 0;
    if (acc || gemm3_applies(ggml_type, packed, rows)) {
      rc = quantize_tiles_host(x, x_dtype, m, k, x_row_stride,
                               acc == 2 ? Q8_TILES_F16S2 : acc == 1 ? (ggml_type == GSQ_TYPE_Q4_K ? Q8_TILES_F16SD : Q8_TILES_F16S) : Q8_TILES_H16,
                               scratch, stream);
      if (rc != GSQ_OK) return rc;
      return gemm3_host(w, row_bytes, rows, ggml_type, packed, scratch, m, k, y, y_dtype, y_row_stride, acc, pair, stream);
    }
    // (IQ4_XS with integer sums: the int8 kernel below)
  }
  if (gemm2_applies(ggml_type, packed, rows) && variant == 4) {
    rc = quantize_tiles_host(x, x_dtype, m, k, x_row_stride, layout, scratch, stream);
    if (rc != GSQ_OK) return rc;
    return gemm2_host(w, row_bytes, rows, ggml_type, packed, scratch, m, k, y, y_dtype, y_row_stride, stream);
  }
  if (gemm2_applies(ggml_type, packed, rows) && (variant == 3 || variant >= 5 || (variant == 0 && big))) {
    rc = quantize_tiles_host(x, x_dtype, m, k, x_row_stride, layout, scratch, stream);
    if (rc != GSQ_OK) return rc;
    return gemm2_host(w, row_bytes, rows, ggml_type, packed, scratch, m, k, y, y_dtype, y_row_stride, stream);
  }
  if (gemm2_applies(ggml_type, packed, rows)) {
    rc = gsq_quantize_q8_1_mmq(x, x_dtype, m, k, x_row_stride, layout, scratch, stream);
    if (rc != GSQ_OK) return rc;
    return gsq_mul_mat_q8(w, row_bytes, rows, ggml_type, packed, scratch, m, k, y, y_dtype, y_row_stride, nullptr, 0, stream);
  }
  if (ggml_type == GSQ_TYPE_Q6_K && packed) {
    // repacked Q6_K above 48 rows: the small-batch kernel, 48 rows per launch, on 36-byte blocks of the whole X
    rc = gsq_quantize_q8_1(x, x_dtype, m, k, x_row_stride, scratch, stream);
    if (rc != GSQ_OK) return rc;
    const int64_t ysz6 = y_dtype == GSQ_F32 ? 4 : 2;
    for (int64_t i = 0; i < m; i += 48) {
      const int64_t c = m - i < 48 ? m - i : 48;
      rc = mmv_host(w, row_bytes, rows, ggml_type, packed, (const uint8_t*)scratch + i * (k / 32) * 36, 0, c, k,
                    (uint8_t*)y + i * y_row_stride * ysz6, y_dtype, y_row_stride, stream, nullptr);
      if (rc != GSQ_OK) return rc == 1000 ? GSQ_ERR_TOO_LARGE : rc;
    }
    return GSQ_OK;
  }
  // Q6_K and IQ3_S in GGUF order: the dp4a kernel on 36-byte blocks, as many rows per launch as it takes
  rc = gsq_quantize_q8_1(x, x_dtype, m, k, x_row_stride, scratch, stream);
  if (rc != GSQ_OK) return rc;
  const int step = gsq_mul_mat_vec_max_rows(ggml_type, packed);
  const int64_t ysz = y_dtype == GSQ_F32 ? 4 : 2;
  for (int64_t i = 0; i < m; i += step) {
    const int64_t c = m - i < step ? m - i : step;
    rc = gsq_mul_mat_vec_q8(w, row_bytes, rows, ggml_type, packed, (const uint8_t*)scratch + i * (k / 32) * 36, c, k,
                            (uint8_t*)y + i * y_row_stride * ysz, y_dtype, y_row_stride, stream);
    if (rc != GSQ_OK) return rc;
  }
  return GSQ_OK;
}

extern "C" int gsq_linear_allreduce(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x,
                                    int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* y, int y_dtype,
                                    int64_t y_row_stride, void* scratch, size_t scratch_bytes, const gsq_peer_reduce* pr,
                                    void* stream) {
  using namespace gsq;
  if (!pr || m <= 0 || m > 48 || rows <= 0 || k <= 0 || k % 256 != 0 || !w || !x || !y) return GSQ_ERR_UNSUPPORTED;
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  if (!scratch || scratch_bytes < gsq_linear_scratch_bytes(rows, m, k, ggml_type, packed)) return GSQ_ERR_SCRATCH;
  if (!mmv_applies(ggml_type, packed, rows, m)) return GSQ_ERR_UNSUPPORTED;
  int rc = gsq_quantize_q8_1_mmq(x, x_dtype, m, k, x_row_stride, gsq_q8_layout_for_type(ggml_type), scratch, stream);
  if (rc != GSQ_OK) return rc;
  rc = mmv_host(w, row_bytes, rows, ggml_type, packed, scratch, 1, m, k, y, y_dtype, y_row_stride, stream, nullptr, pr);
  return rc == 1000 ? GSQ_ERR_UNSUPPORTED : rc;   // 1000: the shape does not fit the kernel's staging area
}
