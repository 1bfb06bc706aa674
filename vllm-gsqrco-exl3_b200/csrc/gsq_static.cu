// A product entry point for callers that cannot give the library any memory of their own.
//
// gsq_linear_vec_static runs "quantise X to q8_1, then the 1..8-row GEMV" exactly like the two-call sequence
// gsq_quantize_q8_1 + gsq_mul_mat_vec_q8, but the q8_1 blocks in between live in a fixed array that is part
// of the library image instead of a buffer the caller allocated. It is meant for hosts that must not call an
// allocator at the point where they need the product: an engine whose memory manager has already handed every
// free byte of the device to its own pools (asking the CUDA allocator there would fail or fragment), a plug-in
// that is only given input and output pointers by its host application, or a latency-critical loop where an
// allocator call is simply forbidden.
#include "gsq_common.cuh"

namespace gsq {

// Largest activation the static array holds: 8 rows of 32768 columns (36 bytes per 32 values).
constexpr int64_t STATIC_MAX_ROWS = 8;
constexpr int64_t STATIC_MAX_Q8_BYTES = STATIC_MAX_ROWS * (32768 / 32) * 36;  // 294,912 bytes

// Every GPU that loads the library carries this array until the process exits.
static __device__ __align__(256) unsigned char g_static_q8[STATIC_MAX_Q8_BYTES];

// Device address of the array per device. In host code the symbol g_static_q8 is only a handle: its address
// there is not a device address, so it is resolved once with cudaGetSymbolAddress while that device is current.
static void* g_static_q8_addr[64];

static int static_q8_address(void** out) {
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GSQ_ERR_UNSUPPORTED;
  if (g_static_q8_addr[dev] == nullptr) {
    void* p = nullptr;
    GSQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_q8));
    if (p == nullptr) return GSQ_ERR_CUDA;
    g_static_q8_addr[dev] = p;
  }
  *out = g_static_q8_addr[dev];
  return GSQ_OK;
}

}  // namespace gsq

extern "C" int64_t gsq_linear_vec_static_max_q8_bytes(void) { return gsq::STATIC_MAX_Q8_BYTES; }

extern "C" int gsq_linear_vec_static(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                                     const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* y,
                                     int y_dtype, int64_t y_row_stride, void* stream) {
  using namespace gsq;
  if (m == 0 || rows == 0) return GSQ_OK;
  if (m < 0 || k <= 0 || k % 256 != 0 || !x || !w || !y) return GSQ_ERR_UNSUPPORTED;
  // the fixed array is the limit: more rows or columns than it holds are refused, never truncated
  if (m > STATIC_MAX_ROWS || m * (k / 32) * 36 > STATIC_MAX_Q8_BYTES) return GSQ_ERR_TOO_LARGE;
  // everything the product would refuse is refused here, before the quantiser is queued
  const int bs = block_bytes(ggml_type);
  if (bs == 0 || row_bytes != (k / 256) * bs || rows < 0 || rows > INT32_MAX || k > INT32_MAX) return GSQ_ERR_UNSUPPORTED;
  if (y_dtype != GSQ_F32 && y_dtype != GSQ_F16 && y_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  if (x_dtype != GSQ_F32 && x_dtype != GSQ_F16 && x_dtype != GSQ_BF16) return GSQ_ERR_UNSUPPORTED;
  if (ggml_type == GSQ_TYPE_IQ3_S && packed && rows % 16 != 0) return GSQ_ERR_UNSUPPORTED;
  void* q8 = nullptr;
  int rc = static_q8_address(&q8);
  if (rc != GSQ_OK) return rc;
  // The quantiser writes every byte the GEMV reads (m * k/32 whole blocks), so nothing left over from the
  // previous call is ever read and nothing has to be cleared first.
  rc = gsq_quantize_q8_1(x, x_dtype, m, k, x_row_stride, q8, stream);
  if (rc != GSQ_OK) return rc;
  return gsq_mul_mat_vec_q8(w, row_bytes, rows, ggml_type, packed, q8, m, k, y, y_dtype, y_row_stride, stream);
}
