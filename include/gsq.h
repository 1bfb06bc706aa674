/*
 * gsq.h -- C ABI of the B200 (sm_100a) GGUF quantised-linear kernels.
 *
 * This is the drop-in boundary for the "Route L" path of vllm_gguf_plugin: each
 * entry point below replaces one piece of plugin/vllm_gguf_plugin/csrc/lcpp_shim.cu
 * (and the kernels it launches) of the reference. All pointers are raw device
 * pointers unless stated otherwise; sizes are plain integers; `stream` is a
 * cudaStream_t passed as void*. No function allocates device memory, synchronises
 * the device or throws: every one returns GSQ_OK (0) or a negative status, and
 * gsq_strerror() names it. The caller (the Python registration layer, which mirrors
 * the reference's torch ops `_C_gguf::lcpp_*`) owns every buffer.
 *
 * ggml type ids are those of gguf.GGMLQuantizationType: Q4_K 12, Q6_K 14,
 * IQ3_S 21, IQ4_XS 23.
 */
#ifndef GSQ_H
#define GSQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GSQ_TYPE_Q4_K 12
#define GSQ_TYPE_Q6_K 14
#define GSQ_TYPE_IQ3_S 21
#define GSQ_TYPE_IQ4_XS 23
/* the low-bit types a model file mixes with those four: served in GGUF order by the dp4a kernel, 8 rows per launch */
#define GSQ_TYPE_Q2_K 10
#define GSQ_TYPE_IQ2_XXS 16
#define GSQ_TYPE_IQ2_XS 17
#define GSQ_TYPE_IQ3_XXS 18
#define GSQ_TYPE_IQ2_S 22
#define GSQ_TYPE_IQ1_M 29

/* element types of X / Y */
#define GSQ_F32 0
#define GSQ_F16 1
#define GSQ_BF16 2
/* anything else the caller could not map (guards reject it) */
#define GSQ_DTYPE_OTHER 99

/* q8_1 scale layouts of the 128-value activation blocks (mmq.cuh:60-101 of the vendored llama.cpp) */
#define GSQ_Q8_LAYOUT_D4 0  /* 4 x fp32 d            : IQ3_S, IQ4_XS, Q6_K */
#define GSQ_Q8_LAYOUT_DS4 1 /* 4 x half2 (d, sum x)  : Q4_K */

/* status codes */
#define GSQ_OK 0
#define GSQ_ERR_GUARD -1     /* an input guard fired; message written to the caller's buffer */
#define GSQ_ERR_CUDA -2      /* a CUDA runtime call failed (see gsq_last_cuda_error) */
#define GSQ_ERR_UNSUPPORTED -3
#define GSQ_ERR_SCRATCH -4   /* scratch buffer missing or too small */
#define GSQ_ERR_TOO_LARGE -5 /* shape exceeds what the kernel (or the static buffer) can hold */
#define GSQ_ERR_DEVICE -6    /* kernel reported an internal error flag (bounded wait gave up) */

/* kernel selectors returned by gsq_route / accepted by gsq_mul_mat */
#define GSQ_KERNEL_NONE 0
#define GSQ_KERNEL_GEMV 1 /* dp4a streaming GEMV, 1..8 activation rows per launch, reads block_q8_1 */
#define GSQ_KERNEL_GEMM 2 /* tcgen05 kind::i8 GEMM, 64-token tiles in lockstep, reads 128-value q8_1 blocks */
#define GSQ_KERNEL_MMV 3  /* register-operand tensor-core kernel, 1..48 activation rows per launch */
#define GSQ_KERNEL_GEMM_PREFILL 4 /* warp-specialised tcgen05 kind::i8 GEMM, 256-token blocks, reads operand tiles */

const char* gsq_strerror(int status);
/* cudaError_t of the last failing CUDA call made by this library on this thread (0 if none). */
int gsq_last_cuda_error(void);

/* ABI version of this header; bumped when a signature changes. */
int gsq_abi_version(void);

/* Bytes per 256-value superblock of a ggml type, 0 if the type is not supported. */
int gsq_type_block_bytes(int ggml_type);

/*
 * Input guards of every product op: replaces check_inputs() and the per-kernel
 * checks at the top of run() (lcpp_shim.cu:690-732, 767-791). Nothing here touches
 * CUDA, so it also runs for CPU tensors (the reference registers its ops for the
 * CPU dispatch key for the same reason, lcpp_shim.cu:997-1008).
 *   op           name used as the message prefix ("lcpp_mul_mat_vec_q", ...)
 *   w_*          W: dim count, dtype is uint8?, sizes, strides (elements), data address
 *   x_*          X likewise; x_dtype one of GSQ_F32/F16/BF16 or GSQ_DTYPE_OTHER
 *   row          number of weight rows to use
 *   max_rows     limit on X rows (0 = none)
 *   need_iq3 / need_q4k_own / need_mma_k / is_mmq / packed : which op-specific type checks apply
 *   k_multiple   512 for the reference-compatible ops, 256 for the tensor-parallel entry points
 *   w_is_cuda, x_is_cuda, same_device : device facts, checked last
 * On failure writes a NUL-terminated message into msg[0..msg_len) and returns GSQ_ERR_GUARD.
 * On success stores the logical column count in *k_out.
 */
typedef struct gsq_guard_args {
  const char* op;
  int w_dim, w_is_uint8;
  int64_t w_size0, w_size1, w_stride0, w_stride1;
  uint64_t w_addr;
  int x_dim, x_dtype;
  int64_t x_size0, x_size1, x_stride0, x_stride1;
  int64_t row, max_rows;
  int ggml_type;
  int need_iq3, need_q4k_own, need_mma_k, is_mmq, packed;
  int k_multiple;
  int w_is_cuda, x_is_cuda, same_device;
} gsq_guard_args;
int gsq_check_inputs(const gsq_guard_args* a, int64_t* k_out, char* msg, size_t msg_len);

/*
 * One-time per-device set-up (shared-memory opt-in of the kernels, SM count cache). Call once per
 * device before the first launch and outside any stream capture; the reference needed a
 * dedicated test because its occupancy caches could be filled inside a capture
 * (tests/gpu/test_kernel_parity.py:655-698). Every launch entry point calls it lazily too.
 */
int gsq_device_init(int device);

/*
 * q8_1 quantisation, MMVQ layout: replaces quantize_q8_1_x (lcpp_shim.cu:274-294, launch 361-368).
 * x [m, k] with row stride x_row_stride elements -> out: m * k/32 blocks of 36 bytes
 * (half d, half sum, then 32 x int8: ggml's block_q8_1), rows contiguous. k % 32 == 0.
 */
int gsq_quantize_q8_1(const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* out,
                      void* stream);

/*
 * Row gather + dequantisation (the quantised embedding look-up): out[i, :] = dequantise(w[ids[i], :]) for the ten types
 * above. Replaces torch.index_select + _C_gguf::ggml_dequantize (quantization/vocal_embeds.py:79-98,
 * csrc/gguf/gguf_kernel.cu:87-103). fp32 arithmetic in the operation order of llama.cpp's C dequantiser / gguf-py
 * (bit-identical to the reference's dequantisation fixtures in fp32); fp16 / bf16 outputs are that value rounded once.
 *   w [w_rows, row_bytes] in GGUF order (not repacked); ids: n int64 row indices on the device, or NULL for rows 0..n-1;
 *   out [n, k] with row stride out_row_stride elements. An index outside [0, w_rows) writes a row of zeros and raises
 *   the flag read by gsq_dequantize_bad_index_flag (nothing out of bounds is read).
 */
int gsq_dequantize_rows(const void* w, int64_t row_bytes, int64_t w_rows, int ggml_type, const int64_t* ids, int64_t n,
                        int64_t k, void* out, int out_dtype, int64_t out_row_stride, void* stream);
int gsq_dequantize_bad_index_flag(int* flag);

/*
 * The element-wise step in front of a quantised linear fused with its q8_1 quantiser (block_q8_1 layout, as
 * gsq_quantize_q8_1 writes it). Not in the reference, whose layers run vLLM's rms_norm / silu_and_mul kernels and
 * then quantise inside apply(); the arithmetic here is theirs (every intermediate rounded to X's type where the
 * separate kernels store it), so the q8_1 bytes equal gsq_quantize_q8_1 of the y_out of the same call bit for bit.
 *
 * gsq_rmsnorm_quantize_q8_1: x [m, k] (row stride x_row_stride); residual: NULL, or [m, k] contiguous, read and
 *   overwritten with x + residual (the "fused add" form); gamma [k] in X's type; out_q8: m * k/32 blocks; y_out: NULL or
 *   [m, k] contiguous, receives the normalised activations in X's type. k % 32 == 0, k <= 40960.
 * gsq_silu_mul_quantize_q8_1: gate_up [m, 2 * inter] (gate columns first; row stride row_stride) -> q8_1 of
 *   silu(gate) * up over the `inter` columns; y_out: NULL or [m, inter] contiguous. inter % 32 == 0.
 */
int gsq_rmsnorm_quantize_q8_1(const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* residual,
                              const void* gamma, float eps, void* out_q8, void* y_out, void* stream);
int gsq_silu_mul_quantize_q8_1(const void* gate_up, int x_dtype, int64_t m, int64_t inter, int64_t row_stride,
                               void* out_q8, void* y_out, void* stream);

/*
 * q8_1 quantisation, 128-value blocks: replaces quantize_mmq_q8_1_x (lcpp_shim.cu:298-355).
 * out: k/128 * m blocks of 144 bytes (16 scale bytes in `layout`, then 128 x int8); block (kb, row)
 * sits at (kb * m + row) * 144. k % 128 == 0.
 */
int gsq_quantize_q8_1_mmq(const void* x, int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, int layout,
                          void* out, void* stream);

/*
 * Product with block_q8_1 activations, 1 .. gsq_mul_mat_vec_max_rows(type, packed) activation rows (8, or 48
 * for Q4_K, IQ4_XS and packed IQ3_S): replaces the vendored MMVQ (ggml_cuda_op_mul_mat_vec_q, mmvq.cu:1538) and
 * the owned small-batch kernels iq3_mul_mat_vec (lcpp_shim.cu:498-572), own_mul_mat_vec
 * (lcpp_owned_k4.cu:116-234), iq3_mma / iq3_mma_packed (lcpp_owned_iq3_mma.cu:179-328, 483-600).
 * Runs the dp4a GEMV or the register-operand tensor-core kernel, whichever is faster for the type and count.
 *   w            uint8 [rows, row_bytes] GGUF blocks (packed != 0: IQ3_S in gsq_iq3s_repack's layout)
 *   x_q8         m * k/32 block_q8_1 (36 bytes each)
 *   y            [m, rows] in y_dtype, row stride y_row_stride elements
 */
int gsq_mul_mat_vec_q8(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                       const void* x_q8, int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride,
                       void* stream);

/*
 * No counterpart in the reference (its shim always takes scratch from torch's allocator, lcpp_shim.cu:250-263).
 * Quantise X and run the 1..8-row GEMV in one call without any buffer from the caller besides X, W and Y:
 * the q8_1 blocks in between are kept in a fixed device array inside the library. For hosts that cannot
 * allocate where they need the product -- their memory manager owns the whole device, they are a plug-in that
 * is handed only input and output pointers, or an allocator call is not allowed on that code path.
 *   - Limit: m <= 8 and m * k/32 * 36 <= gsq_linear_vec_static_max_q8_bytes() (294,912 bytes, i.e. 8 rows of
 *     32768 columns); anything larger returns GSQ_ERR_TOO_LARGE ("shape too large ...") and launches nothing.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call, and gsq_device_init for the device, before starting a stream
 *     capture. On every call the device of `stream` must be the current device: the address used is the
 *     current device's.
 *   - All calls on a device share the one array, which keeps what the last call wrote. Every call overwrites
 *     all the bytes it reads, so nothing needs clearing; but two calls that overlap on the GPU (different
 *     streams, no ordering) race on it. Order them, or use the two-call sequence with your own buffers.
 * Arguments as gsq_quantize_q8_1 (x, x_dtype, m, k, x_row_stride) and gsq_mul_mat_vec_q8 (the rest).
 */
int64_t gsq_linear_vec_static_max_q8_bytes(void);
int gsq_linear_vec_static(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x,
                          int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* y, int y_dtype,
                          int64_t y_row_stride, void* stream);


/*
 * Every wait on a bulk copy inside a kernel is bounded; a wait that gave up sets a sticky per-device flag
 * instead of hanging. Copies the flag (0 = never happened) to *flag. Synchronises the device.
 */
int gsq_device_error_flag(int* flag);


/*
 * Product with block_q8_1_mmq activations, any number of activation rows (the register-operand tensor-core
 * kernel up to 48 rows where it fits, the tcgen05 kind::i8 GEMM with TMEM accumulators above): replaces
 * the vendored MMQ (mul_mat_q, mmq.cuh:961-1385 + shim host side lcpp_shim.cu:626-671) and the owned
 * mma_k (lcpp_owned_mma_k.cu:353-539) and iq3_packed_mmq (lcpp_owned_iq3_mma.cu:768-970).
 *   x_q8_mmq     k/128 * m blocks of 144 bytes in the type's layout (gsq_q8_layout_for_type)
 *   scratch      gsq_mul_mat_scratch_bytes(...) bytes, 256-byte aligned; contents need not be
 *                initialised and are not preserved
 */
int gsq_q8_layout_for_type(int ggml_type);
/* Most activation rows one gsq_mul_mat_vec_q8 call takes for this type (8, or 48 where the kernel above serves it). */
int gsq_mul_mat_vec_max_rows(int ggml_type, int packed);
size_t gsq_mul_mat_scratch_bytes(int64_t rows, int64_t m, int64_t k, int ggml_type);
int gsq_mul_mat_q8(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                   const void* x_q8_mmq, int64_t m, int64_t k, void* y, int y_dtype, int64_t y_row_stride,
                   void* scratch, size_t scratch_bytes, void* stream);

/*
 * The whole product from X as it is, any number of activation rows: quantises X into `scratch` in the layout of
 * the kernel it then runs (the small-batch tensor-core kernel up to 48 rows, the warp-specialised tcgen05 GEMM
 * above, the dp4a kernel for Q6_K and IQ3_S in GGUF order). Replaces what the reference's self-quantising ops do
 * in one call: lcpp_mul_mat_q, lcpp_mul_mat_mma_k, lcpp_mul_mat_iq3_packed (lcpp_shim.cu:626-671, 753-909, whose
 * scratch comes from torch's allocator, :250-263).
 *   x            [m, k] in x_dtype, row stride x_row_stride elements
 *   scratch      gsq_linear_scratch_bytes(...) bytes, 256-byte aligned; need not be initialised, not preserved
 */
size_t gsq_linear_scratch_bytes(int64_t rows, int64_t m, int64_t k, int ggml_type, int packed);
int gsq_linear(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x, int x_dtype,
               int64_t m, int64_t k, int64_t x_row_stride, void* y, int y_dtype, int64_t y_row_stride, void* scratch,
               size_t scratch_bytes, void* stream);

/*
 * How gsq_linear forms the prefill product of repacked IQ3_S, of IQ4_XS and of Q4_K (256 tokens and up; the other
 * routes are not affected).
 * The reference's kernels keep an exact int32 sum per 32-value slice and scale it in fp32
 * (lcpp_owned_iq3_mma.cu:768-970, mmq.cuh:961-1385). Sets the mode, returns the previous one:
 *   GSQ_PREFILL_ROUNDED (default)  d_x * q goes into the tensor-core operand as one fp16 number and tensor memory
 *                                  accumulates over a superblock: a result differs from the reference kernels' by
 *                                  2e-4 .. 4e-4 of its row's norm (bound of the parity tests: 1e-3); fastest
 *   GSQ_PREFILL_SPLIT              d_x * q as a pair of fp16 numbers (22 bits): differs by about 1e-6 (IQ4_XS and Q4_K,
 *                                  whose weight operands carry a rounding of their own: as GSQ_PREFILL_INTEGER)
 *   GSQ_PREFILL_INTEGER            exact integer slice sums, scaled per slice as the reference does
 * A process-wide setting; not to be changed while products are in flight on another thread.
 */
#define GSQ_PREFILL_ROUNDED 0
#define GSQ_PREFILL_SPLIT 1
#define GSQ_PREFILL_INTEGER 2
int gsq_prefill_precision(int mode);

/*
 * IQ3_S load-time repack, in place, bijective: replaces iq3_pack.pack_ / unpack
 * (plugin/vllm_gguf_plugin/quantization/iq3_pack.py:73-181). w uint8 [rows, row_bytes], rows % 16 == 0,
 * 16-byte aligned. direction 0: GGUF blocks -> streaming layout; 1: back. One thread block stages one
 * 16-row tile in shared memory, so 16 * row_bytes must fit (GSQ_ERR_TOO_LARGE otherwise).
 */
int gsq_iq3s_repack(void* w, int64_t rows, int64_t row_bytes, int direction, void* stream);

/*
 * Q6_K load-time repack, in place, bijective; no counterpart in the reference, which reads Q6_K in GGUF order
 * with its vendored kernels. GGUF's 210-byte blocks are only 2-byte aligned; the repack is a byte permutation
 * inside each 16-row tile into 3360-byte records (one per superblock) in which a lane's share of the int8
 * tensor-core fragments is six 128-bit loads (layout in csrc/gsq_repack.cu). Arguments as gsq_iq3s_repack
 * (row_bytes a multiple of 210). Repacked Q6_K is passed to the product entry points with packed != 0 and is
 * served by the small-batch tensor-core kernel at every row count (48 rows per launch).
 */
int gsq_q6k_repack(void* w, int64_t rows, int64_t row_bytes, int direction, void* stream);

/*
 * Sum of the partial results of K-sharded products (o_proj / down style, one [m, rows] partial per GPU) over peer
 * memory, one kernel per rank, no NCCL call and no host involvement (so it replays inside a CUDA graph). No
 * counterpart in the reference, which leaves the reduction to vLLM's row-parallel layer (an NCCL all-reduce after
 * apply()). Every rank must make the same sequence of calls.
 *   peer_bufs    device array of `world` pointers: each rank's partial buffer of `count` elements, mapped into this
 *                process (symmetric memory / CUDA IPC; entry `rank` is this rank's own); 16-byte aligned
 *   peer_flags   device array of `world` pointers: each rank's flag pad of `world` uint32, zero before the first call
 *   out          [count] in `dtype`, this rank's memory; receives the sum (fp32 accumulation, rank order: all
 *                ranks get bit-identical results)
 *   state        2 uint32 of this rank's device memory, zero before the first call (call counter, block ticket)
 * Consecutive calls must use different partial buffers (alternate between two): a partial buffer may be rewritten
 * once the call after the one that read it has returned. Waits on the peers are bounded (a fraction of a second):
 * a wait that gives up leaves `out` unwritten and raises the flag read by gsq_allreduce_error_flag.
 * count * element size must be a multiple of 16.
 */
int gsq_allreduce_sum(const void* const* peer_bufs, uint32_t* const* peer_flags, int rank, int world, int64_t count,
                      int dtype, void* out, uint32_t* state, void* stream);
int gsq_allreduce_error_flag(int* flag);

/*
 * The same sum fused into the product: gsq_linear whose kernel, after forming this rank's partial [m, rows] of a
 * K-sharded product, stores it into a slot on every GPU, signals, waits (bounded) for the other ranks' partials and
 * writes their sum to y -- one kernel per rank for product + all-reduce, no collective call, replayable in a CUDA
 * graph. Served by the small-batch tensor-core kernel only (1..48 rows of the types and shapes it takes; any other
 * call returns GSQ_ERR_UNSUPPORTED with only the activation quantiser queued, and the caller uses gsq_linear +
 * gsq_allreduce_sum). Every rank must make the same sequence of calls with the same shapes.
 *   slots   device array of `world` pointers: each rank's slot area of 2 * world * slot_bytes bytes (symmetric memory /
 *           CUDA IPC; entry `rank` is this rank's own), 16-byte aligned
 *   flags   device array of `world` pointers: each rank's flag area of `world` uint32, zero before the first call
 *   state   3 uint32 of this rank's device memory, zero before the first call
 *   slot_bytes  >= ((m - 1) * y_row_stride + rows) * element size of y, a multiple of 16
 * y is written in y_dtype with fp32 accumulation of the ranks' partials (rounded to y_dtype) in rank order: all ranks
 * get bit-identical results. A wait that gives up leaves y unwritten and raises gsq_peer_reduce_error_flag.
 */
typedef struct gsq_peer_reduce {
  void* const* slots;
  uint32_t* const* flags;
  uint32_t* state;
  int rank, world;
  int64_t slot_bytes;
} gsq_peer_reduce;
int gsq_linear_allreduce(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed, const void* x,
                         int x_dtype, int64_t m, int64_t k, int64_t x_row_stride, void* y, int y_dtype,
                         int64_t y_row_stride, void* scratch, size_t scratch_bytes, const gsq_peer_reduce* pr, void* stream);
int gsq_peer_reduce_error_flag(int* flag);

/*
 * Kernel family that serves (activation rows m, type, weight rows, k, packed) on B200: GSQ_KERNEL_*, the choice
 * gsq_mul_mat_vec_q8 and gsq_linear make. The op-level routing table of the reference (_lcpp_op,
 * quantization/linear.py:85-114) stays in the Python layer because its op names are API; this is the choice made
 * underneath those names.
 */
int gsq_route(int64_t m, int ggml_type, int64_t rows, int64_t k, int packed);

#ifdef __cplusplus
}
#endif
#endif /* GSQ_H */
