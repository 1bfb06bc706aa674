// Load-time repacks (in place, bijective) into the layouts the sm_100a kernels read: IQ3_S, and Q6_K further down.
//
// Takes the place of the reference's iq3_pack (plugin/vllm_gguf_plugin/quantization/iq3_pack.py:73-181).
// As there, rows are grouped in tiles of 16 and tile t keeps the bytes rows 16t..16t+15 had, as one
// 1760-byte record per superblock j at  t * 16 * row_bytes + j * 1760. Inside a record the bytes are ordered
// for 128-bit coalesced loads by a warp whose lanes hold the int8 tensor-core A fragment of the 16 rows:
// lane l = 4 g + t (g = 0..7, t = 0..3) owns rows g and g + 8 and, of every 32-value slice s, the two 4-value
// groups 2t and 2t + 1. Its 32 "fields" are numbered f = 4 s + 2 h + e (h: row g + 8 h, e: group 2t + e):
//   [   0,  512)  16 bytes per lane: words 0..3 of the lane's 9-word index stream
//   [ 512, 1024)  16 bytes per lane: words 4..7
//   [1024, 1152)   4 bytes per lane: word 8
//                 the stream holds the 32 nine-bit codebook indices, field f at bit 9 f: qs byte | qh bit << 8
//   [1152, 1664)  16 bytes per lane: word f / 8 holds the 4 sign bits of fields 8 (f / 8) .. + 7, the sign of
//                 value p of field f at bit 16 ((f % 8) / 4) + 4 p + f % 4: a shift and one AND/OR turn them
//                 into the byte-permute selector that picks +g or -g
//   [1664, 1728)   8 bytes per g: u32 of row g (nibble s = 4-bit sub-scale of slice s), then u32 of row g + 8
//   [1728, 1760)   4 bytes per g: fp16 d of row g, then of row g + 8
#include "gsq_common.cuh"

namespace gsq {

__device__ __forceinline__ uint32_t stream_get(const uint32_t (&idx)[10], int f) {
  const int bit = 9 * f, word = bit >> 5, off = bit & 31;
  uint32_t v = idx[word] >> off;
  if (off + 9 > 32) v |= idx[word + 1] << (32 - off);
  return v & 0x1FFu;
}

// direction 0: GGUF blocks -> records, one thread per (superblock, lane). direction 1: records -> GGUF blocks,
// one thread per (superblock, row, slice). Both read the tile from its copy in shared memory and write W.
__global__ void __launch_bounds__(256) iq3s_repack_kernel(uint8_t* __restrict__ w, int64_t row_bytes, int nb,
                                                         int direction) {
  extern __shared__ __align__(16) uint8_t tile[];
  uint8_t* base = w + (int64_t)blockIdx.x * 16 * row_bytes;
  const int tile_bytes = (int)(16 * row_bytes);
  for (int i = threadIdx.x; i < tile_bytes / 16; i += blockDim.x) {
    reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(base)[i];
  }
  __syncthreads();
  if (direction == 0) {
    for (int it = threadIdx.x; it < nb * 32; it += blockDim.x) {
      const int j = it >> 5, l = it & 31, g = l >> 2, t = l & 3;
      uint32_t idx[10];
#pragma unroll
      for (int q = 0; q < 10; ++q) idx[q] = 0;
      uint32_t sg[4] = {0, 0, 0, 0};
      for (int s = 0; s < 8; ++s) {
        for (int h = 0; h < 2; ++h) {
          const uint8_t* b = tile + (size_t)(g + 8 * h) * row_bytes + (size_t)j * 110;
          const uint32_t qh = b[66 + s];
          const uint8_t* sp = b + 74 + 4 * s;
          const uint32_t sbits = (uint32_t)sp[0] | ((uint32_t)sp[1] << 8) | ((uint32_t)sp[2] << 16) | ((uint32_t)sp[3] << 24);
          for (int e = 0; e < 2; ++e) {
            const int f = 4 * s + 2 * h + e, e8 = 2 * t + e;
            const uint32_t v = (uint32_t)b[2 + 8 * s + e8] | (((qh >> e8) & 1u) << 8);
            const int bit = 9 * f, word = bit >> 5, off = bit & 31;
            idx[word] |= v << off;
            if (off + 9 > 32) idx[word + 1] |= v >> (32 - off);
            const int fl = f & 7;
            for (int p = 0; p < 4; ++p) {
              sg[f >> 3] |= ((sbits >> (4 * e8 + p)) & 1u) << (16 * (fl >> 2) + 4 * p + (fl & 3));
            }
          }
        }
      }
      uint8_t* o = base + (size_t)j * 1760;
      *reinterpret_cast<uint4*>(o + 16 * l) = make_uint4(idx[0], idx[1], idx[2], idx[3]);
      *reinterpret_cast<uint4*>(o + 512 + 16 * l) = make_uint4(idx[4], idx[5], idx[6], idx[7]);
      *reinterpret_cast<uint32_t*>(o + 1024 + 4 * l) = idx[8];
      *reinterpret_cast<uint4*>(o + 1152 + 16 * l) = make_uint4(sg[0], sg[1], sg[2], sg[3]);
      if (t < 2) {  // lane (g, t = h): the sub-scales of row g + 8 h; lanes t = 2: the two d
        const uint8_t* b = tile + (size_t)(g + 8 * t) * row_bytes + (size_t)j * 110;
        *reinterpret_cast<uint32_t*>(o + 1664 + 8 * g + 4 * t) =
            (uint32_t)b[106] | ((uint32_t)b[107] << 8) | ((uint32_t)b[108] << 16) | ((uint32_t)b[109] << 24);
      } else if (t == 2) {
        const uint8_t* b0 = tile + (size_t)g * row_bytes + (size_t)j * 110;
        const uint8_t* b1 = tile + (size_t)(g + 8) * row_bytes + (size_t)j * 110;
        *reinterpret_cast<uint32_t*>(o + 1728 + 4 * g) =
            (uint32_t)b0[0] | ((uint32_t)b0[1] << 8) | ((uint32_t)b1[0] << 16) | ((uint32_t)b1[1] << 24);
      }
    }
  } else {
    for (int it = threadIdx.x; it < nb * 128; it += blockDim.x) {
      const int j = it >> 7, r = (it >> 3) & 15, s = it & 7, g = r & 7, h = r >> 3;
      const uint8_t* o = tile + (size_t)j * 1760;
      uint8_t* b = base + (size_t)r * row_bytes + (size_t)j * 110;
      uint32_t qh = 0, sbits = 0;
      uint32_t qs[8];
      for (int t = 0; t < 4; ++t) {
        const int l = 4 * g + t;
        uint32_t idx[10];
        const uint4 ia = *reinterpret_cast<const uint4*>(o + 16 * l);
        const uint4 ib = *reinterpret_cast<const uint4*>(o + 512 + 16 * l);
        idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
        idx[4] = ib.x; idx[5] = ib.y; idx[6] = ib.z; idx[7] = ib.w;
        idx[8] = *reinterpret_cast<const uint32_t*>(o + 1024 + 4 * l);
        idx[9] = 0;
        for (int e = 0; e < 2; ++e) {
          const int f = 4 * s + 2 * h + e, e8 = 2 * t + e, fl = f & 7;
          const uint32_t v = stream_get(idx, f);
          qs[e8] = v & 0xFFu;
          qh |= (v >> 8) << e8;
          const uint32_t sgw = *reinterpret_cast<const uint32_t*>(o + 1152 + 16 * l + 4 * (f >> 3));
          for (int p = 0; p < 4; ++p) {
            sbits |= ((sgw >> (16 * (fl >> 2) + 4 * p + (fl & 3))) & 1u) << (4 * e8 + p);
          }
        }
      }
      // blocks are 2-byte aligned: write halfwords
      for (int e = 0; e < 8; e += 2) {
        *reinterpret_cast<uint16_t*>(b + 2 + 8 * s + e) = (uint16_t)(qs[e] | (qs[e + 1] << 8));
      }
      b[66 + s] = (uint8_t)qh;
      *reinterpret_cast<uint16_t*>(b + 74 + 4 * s) = (uint16_t)(sbits & 0xFFFFu);
      *reinterpret_cast<uint16_t*>(b + 76 + 4 * s) = (uint16_t)(sbits >> 16);
      if (s < 2) {  // the four scale bytes, two per thread
        const uint32_t sc = *reinterpret_cast<const uint32_t*>(o + 1664 + 8 * g + 4 * h);
        *reinterpret_cast<uint16_t*>(b + 106 + 2 * s) = (uint16_t)(sc >> (16 * s));
      } else if (s == 2) {
        const uint32_t dd = *reinterpret_cast<const uint32_t*>(o + 1728 + 4 * g);
        *reinterpret_cast<uint16_t*>(b) = (uint16_t)(dd >> (16 * h));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Q6_K: 210-byte blocks are only 2-byte aligned in GGUF order (128 bytes of low nibbles, 64 bytes of 2-bit high
// parts, 16 int8 sub-scales, fp16 d), which would force 16-bit loads. The repack is a pure byte permutation inside
// each 16-row tile, one 3360-byte record per superblock j at  t * 16 * row_bytes + j * 3360  (a multiple of 16):
//   [   0, 2048)  64 bytes per lane 4 g + t: row g, then row g + 8; per row the eight 4-byte words
//                 (n, qb, is) = ql[64 n + 32 qb + 16 is + 4 t .. + 3]: the lane's 4 values of the 16-value groups
//                 8 n + 2 qb + is (low nibbles) and 8 n + 2 (qb + 2) + is (high nibbles)
//   [2048, 3072)  32 bytes per lane: row g, then row g + 8; per row the four words (n, is) =
//                 qh[32 n + 16 is + 4 t .. + 3]: two bits for each of the four groups 8 n + 2 q + is, q = 0..3
//   [3072, 3328)  32 bytes per g: the 16 sub-scales of row g, then of row g + 8
//   [3328, 3360)   4 bytes per g: fp16 d of row g, then of row g + 8
// With that a lane's share of the int8 tensor-core fragments (rows g, g + 8; values 4 t .. 4 t + 3 of every group) is
// six 128-bit loads. No kernel reads GGUF-order bytes from a repacked tensor: direction 1 restores them.

// byte o of a record comes from (row of the tile, byte of that row's 210-byte block)
__host__ __device__ inline void q6k_source(int o, int* row, int* src) {
  if (o < 2048) {
    const int lane = o >> 6, w = (o & 63) >> 2, b = o & 3, g = lane >> 2, t = lane & 3, h = w >> 3, wi = w & 7;
    *row = g + 8 * h;
    *src = 64 * (wi >> 2) + 32 * ((wi >> 1) & 1) + 16 * (wi & 1) + 4 * t + b;
  } else if (o < 3072) {
    const int q = o - 2048, lane = q >> 5, w = (q & 31) >> 2, b = q & 3, g = lane >> 2, t = lane & 3, h = w >> 2, wi = w & 3;
    *row = g + 8 * h;
    *src = 128 + 32 * (wi >> 1) + 16 * (wi & 1) + 4 * t + b;
  } else if (o < 3328) {
    const int q = o - 3072;
    *row = (q >> 5) + 8 * ((q >> 4) & 1);
    *src = 192 + (q & 15);
  } else {
    const int q = o - 3328;
    *row = (q >> 2) + 8 * ((q >> 1) & 1);
    *src = 208 + (q & 1);
  }
}

__global__ void __launch_bounds__(256) q6k_repack_kernel(uint8_t* __restrict__ w, int64_t row_bytes, int nb, int direction) {
  extern __shared__ __align__(16) uint8_t tile[];
  uint8_t* base = w + (int64_t)blockIdx.x * 16 * row_bytes;
  const int tile_bytes = (int)(16 * row_bytes);
  for (int i = threadIdx.x; i < tile_bytes / 16; i += blockDim.x) {
    reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(base)[i];
  }
  __syncthreads();
  // two bytes per step: sources and destinations of even offsets are even and their partners follow them
  for (int it = threadIdx.x; it < nb * 1680; it += blockDim.x) {
    const int j = it / 1680, o = 2 * (it - j * 1680);
    int row, src;
    q6k_source(o, &row, &src);
    const size_t raw = (size_t)row * row_bytes + (size_t)j * 210 + src, rec = (size_t)j * 3360 + o;
    if (direction == 0) {
      *reinterpret_cast<uint16_t*>(base + rec) = *reinterpret_cast<const uint16_t*>(tile + raw);
    } else {
      *reinterpret_cast<uint16_t*>(base + raw) = *reinterpret_cast<const uint16_t*>(tile + rec);
    }
  }
}

}  // namespace gsq

extern "C" int gsq_q6k_repack(void* w, int64_t rows, int64_t row_bytes, int direction, void* stream) {
  using namespace gsq;
  if (rows == 0) return GSQ_OK;
  if (!w || rows < 0 || rows % 16 != 0 || row_bytes <= 0 || row_bytes % 210 != 0 || (uintptr_t)w % 16 != 0 ||
      (direction != 0 && direction != 1)) {
    return GSQ_ERR_UNSUPPORTED;
  }
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  const size_t smem = (size_t)16 * row_bytes;
  if (smem > (size_t)di.max_smem_optin) return GSQ_ERR_TOO_LARGE;
  static int configured_mask = 0;
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 32 || !((configured_mask >> dev) & 1)) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(q6k_repack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev < 32) configured_mask |= 1 << dev;
  }
  q6k_repack_kernel<<<(unsigned)(rows / 16), 256, smem, (cudaStream_t)stream>>>((uint8_t*)w, row_bytes,
                                                                               (int)(row_bytes / 210), direction);
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}

extern "C" int gsq_iq3s_repack(void* w, int64_t rows, int64_t row_bytes, int direction, void* stream) {
  using namespace gsq;
  if (rows == 0) return GSQ_OK;
  if (!w || rows < 0 || rows % 16 != 0 || row_bytes <= 0 || row_bytes % 110 != 0 || (uintptr_t)w % 16 != 0 ||
      (direction != 0 && direction != 1)) {
    return GSQ_ERR_UNSUPPORTED;
  }
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  const size_t smem = (size_t)16 * row_bytes;
  if (smem > (size_t)di.max_smem_optin) return GSQ_ERR_TOO_LARGE;
  static int configured_mask = 0;
  int dev = 0;
  GSQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 32 || !((configured_mask >> dev) & 1)) {
    GSQ_CUDA_TRY(cudaFuncSetAttribute(iq3s_repack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev < 32) configured_mask |= 1 << dev;
  }
  iq3s_repack_kernel<<<(unsigned)(rows / 16), 256, smem, (cudaStream_t)stream>>>((uint8_t*)w, row_bytes,
                                                                                (int)(row_bytes / 110), direction);
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}
