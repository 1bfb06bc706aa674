/*
 * gsq_debug.h -- test and experiment hooks of libgsq.so. Not part of the product boundary (include/gsq.h): they
 * switch kernel variants or expose kernel internals for the parity tests and for A/B measurements, and they change
 * process-global state, so a host application has no reason to call them. Each setter returns the previous value.
 */
#ifndef GSQ_DEBUG_H
#define GSQ_DEBUG_H

#include "gsq.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * The GEMV has two weight-streaming variants: bulk copies (cp.async.bulk + mbarrier) into a per-warp
 * shared-memory ring, used wherever row segments are 16-byte aligned, and direct 128-bit loads otherwise.
 * Test hook: on != 0 forces the direct variant everywhere; returns the previous setting.
 */
int gsq_debug_force_direct_loads(int on);
int gsq_debug_force_cluster_size(int cs); /* dp4a GEMV: 0 = choose; 1, 2, 4 = CTAs per cluster */


/*
 * Test hook: the raw int32 dot product of every weight group with the matching activation quants, taken
 * from inside the GEMV kernel itself (a debug instantiation of the same code, one activation row per
 * launch). These are the `sumi` of the reference's vec_dot_*_q8_1 (vecdotq.cuh:1233-1243 and siblings)
 * before any scale is applied; no reference op exposes them.
 *   sums       int32 [m, rows, k/g], g = 32 (16 for Q6_K); MUST be zeroed by the caller (lanes add into it)
 *   y_scratch  rows floats, overwritten
 */
int gsq_debug_block_sums(const void* w, int64_t row_bytes, int64_t rows, int ggml_type, int packed,
                         const void* x_q8, int64_t m, int64_t k, int32_t* sums, float* y_scratch, void* stream);

/* Test hooks of the GEMM: exchange the two stride fields of its shared-memory matrix descriptors (returns
 * the previous setting); make every following gsq_mul_mat_q8 call also store its raw int32 slice sums to
 * sums[m][rows][k/32] (NULL switches it off). */
int gsq_debug_swap_descriptor_strides(int on);
int gsq_debug_gemm_dump_sums(int32_t* sums);
int gsq_debug_gemm_wait_hint(int ns); /* fp16-operand prefill GEMM: 0 = poll the mbarriers with short sleeps, else the nanoseconds a waiting thread is suspended per try; returns previous */
int gsq_debug_gemm_variant(int v); /* kernel behind gsq_linear above the small-batch row counts: 0 = by shape (default), 3 = always a prefill GEMM (fp16 operands for repacked IQ3_S in the form gsq_prefill_precision selects, int8 otherwise), 5 / 6 / 7 = the same with the split / rounded / integer form forced, 9 / 8 = the split / rounded form on pairs of CTAs (cta_group::2), 4 = always the int8 prefill GEMM, 1 / 2 = the warp-specialised / lockstep kernels of gsq_mul_mat_q8; returns previous */
/* device buffer of 16 uint64 per CTA that the prefill GEMM fills with clock counts of its roles' waits and work (a
 * separate instantiation; NULL switches it off): [0] producer waits for a free stage, [1] decodes; MMA thread waits
 * for [2] a weight tile, [3] a drained half of tensor memory, [4] an activation unit; consumer warp 4: [5] waits for
 * the unit, [6] for the MMA, [7] scales, [8] waits for the scale planes; warps 7 and 19 likewise at [9..11], [12..14] */
int gsq_debug_gemm_profile(unsigned long long* clocks);
int gsq_debug_gemm_ksplit(int ks); /* 0 = choose; 1, 2, 4 = CTAs per cluster that split K (experiments) */
/* The register-operand tensor-core kernel that serves 1..48 activation rows behind gsq_mul_mat_vec_q8 and
 * gsq_mul_mat_q8 (experiments and tests; each returns the previous value). */
int gsq_debug_mmv_mode(int mode);        /* 0 = wherever it applies (default), 1 = never: dp4a GEMV / tcgen05 GEMM */
int gsq_debug_mmv_min_rows(int n);       /* fewest activation rows it serves; 0 = per type (default) */
int gsq_debug_mmv_max_rows(int n);       /* most activation rows it serves (default and at most 48) */
int gsq_debug_mmv_cluster_size(int cs);  /* 0 = choose; 1, 2, 4, 8 = CTAs per cluster */
int gsq_debug_mmv_prefetch_first(int n); /* records a warp requests from L2 before the staging (default 2) */
int gsq_debug_mmv_chunking(int mode);    /* records per warp: -1 = choose (default), 0 = equal chunks, 1 = whole tiles */
int gsq_debug_mmv_trace(int on);         /* one line per launch plan on stderr */
int gsq_debug_mmv_pdl(int on);           /* programmatic dependent launch: 0 = off, 1 = on, 2 = and the kernel lets the next one start early where that measured faster (default), 3 = everywhere */
/* device buffer of 8 uint64 per CTA that receives time stamps (ns) at the kernel's phase boundaries, or NULL */
int gsq_debug_mmv_profile(unsigned long long* stamps);

#ifdef __cplusplus
}
#endif
#endif /* GSQ_DEBUG_H */
