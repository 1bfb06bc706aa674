// Tensor-core GEMM entry point (placeholder translation unit until the tcgen05 kernel lands).
#include "gsq_common.cuh"

extern "C" size_t gsq_mul_mat_scratch_bytes(int64_t rows, int64_t m, int64_t k, int ggml_type) {
  (void)rows; (void)m; (void)k; (void)ggml_type;
  return 0;
}

extern "C" int gsq_mul_mat_q8(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                              const void* x_q8_mmq, int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride,
                              void* scratch, size_t scratch_bytes, void* stream) {
  (void)w; (void)row_bytes; (void)rows; (void)ggml_type; (void)packed; (void)x_q8_mmq; (void)m; (void)k; (void)y;
  (void)y_dtype; (void)y_row_stride; (void)scratch; (void)scratch_bytes; (void)stream;
  return GSQ_ERR_UNSUPPORTED;
}
