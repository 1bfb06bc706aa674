// IQ3_S load-time repack into the streaming layout the sm_100a kernels read (in place, bijective).
//
// Takes the place of the reference's iq3_pack (plugin/vllm_gguf_plugin/quantization/iq3_pack.py:73-181),
// whose layout is cut for mma.sync fragments; this one is cut for 128-bit coalesced loads and a cheap
// in-register decode. As there, rows are grouped in tiles of 16 and tile t keeps the bytes rows
// 16t..16t+15 had, as one 1760-byte record per superblock j at  t * 16 * row_bytes + j * 1760.
//
// Inside a record, lane l = 8 a + s (a = 0..3, s = 0..7) owns slice s (values 32 s .. 32 s + 31) of rows
// r_i = a + 4 i (i = 0..3):
//   [   0,  512)  16 bytes per lane: words 0..3 of the lane's 9-word index stream
//   [ 512, 1024)  16 bytes per lane: words 4..7
//   [1024, 1152)   4 bytes per lane: word 8
//                 the stream holds 32 nine-bit codebook indices, row i group e (values 4e..4e+3 of the
//                 slice) at bit 9 * (8 i + e): qs byte | qh bit << 8
//   [1152, 1664)  16 bytes per lane: word i = the slice's 32 sign bits of row r_i, transposed so that
//                 bit 16 (e / 4) + 4 p + e % 4 is the sign of value p of group e (GGUF order: bit 4 e + p):
//                 a shift and one AND/OR turn them into the byte-permute selector that picks +g or -g
//   [1664, 1728)   2 bytes per lane: nibble i = 4-bit sub-scale of (row r_i, slice s)
//   [1728, 1760)  fp16 d of row a + 4 i at halfword 4 a + i
#include "gsq_common.cuh"

namespace gsq {

__device__ __forceinline__ uint32_t sign_spread(uint32_t g) {  // GGUF bit 4e+p -> bit 16(e/4) + 4p + e%4
  uint32_t o = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e)
#pragma unroll
    for (int p = 0; p < 4; ++p) o |= ((g >> (4 * e + p)) & 1u) << (16 * (e >> 2) + 4 * p + (e & 3));
  return o;
}
__device__ __forceinline__ uint32_t sign_gather(uint32_t o) {  // inverse of sign_spread
  uint32_t g = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e)
#pragma unroll
    for (int p = 0; p < 4; ++p) g |= ((o >> (16 * (e >> 2) + 4 * p + (e & 3))) & 1u) << (4 * e + p);
  return g;
}

__global__ void __launch_bounds__(256) iq3s_repack_kernel(uint8_t* __restrict__ w, int64_t row_bytes, int nb,
                                                         int direction) {
  extern __shared__ __align__(16) uint8_t tile[];
  uint8_t* base = w + (int64_t)blockIdx.x * 16 * row_bytes;
  const int tile_bytes = (int)(16 * row_bytes);
  for (int i = threadIdx.x; i < tile_bytes / 16; i += blockDim.x) {
    reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(base)[i];
  }
  __syncthreads();
  for (int t = threadIdx.x; t < nb * 32; t += blockDim.x) {
    const int j = t >> 5, l = t & 31, a = l >> 3, s = l & 7;
    if (direction == 0) {
      uint32_t idx[10];
#pragma unroll
      for (int q = 0; q < 10; ++q) idx[q] = 0;
      uint32_t sg[4], sc = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint8_t* b = tile + (size_t)(a + 4 * i) * row_bytes + (size_t)j * 110;
        const uint32_t qh = b[66 + s];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t f = (uint32_t)b[2 + 8 * s + e] | (((qh >> e) & 1u) << 8);
          const int bit = 9 * (8 * i + e), word = bit >> 5, off = bit & 31;
          idx[word] |= f << off;
          if (off + 9 > 32) idx[word + 1] |= f >> (32 - off);
        }
        const uint8_t* g = b + 74 + 4 * s;
        sg[i] = sign_spread((uint32_t)g[0] | ((uint32_t)g[1] << 8) | ((uint32_t)g[2] << 16) | ((uint32_t)g[3] << 24));
        sc |= (((uint32_t)b[106 + (s >> 1)] >> (4 * (s & 1))) & 0xFu) << (4 * i);
      }
      uint8_t* o = base + (size_t)j * 1760;
      *reinterpret_cast<uint4*>(o + 16 * l) = make_uint4(idx[0], idx[1], idx[2], idx[3]);
      *reinterpret_cast<uint4*>(o + 512 + 16 * l) = make_uint4(idx[4], idx[5], idx[6], idx[7]);
      *reinterpret_cast<uint32_t*>(o + 1024 + 4 * l) = idx[8];
      *reinterpret_cast<uint4*>(o + 1152 + 16 * l) = make_uint4(sg[0], sg[1], sg[2], sg[3]);
      *reinterpret_cast<uint16_t*>(o + 1664 + 2 * l) = (uint16_t)sc;
      if (s < 4) {  // lane (a, s = i) stores d of row a + 4 i
        const uint8_t* b = tile + (size_t)(a + 4 * s) * row_bytes + (size_t)j * 110;
        *reinterpret_cast<uint16_t*>(o + 1728 + 2 * (4 * a + s)) = (uint16_t)(b[0] | (b[1] << 8));
      }
    } else {
      const uint8_t* o = tile + (size_t)j * 1760;
      uint32_t idx[10];
      const uint4 ia = *reinterpret_cast<const uint4*>(o + 16 * l);
      const uint4 ib = *reinterpret_cast<const uint4*>(o + 512 + 16 * l);
      idx[0] = ia.x; idx[1] = ia.y; idx[2] = ia.z; idx[3] = ia.w;
      idx[4] = ib.x; idx[5] = ib.y; idx[6] = ib.z; idx[7] = ib.w;
      idx[8] = *reinterpret_cast<const uint32_t*>(o + 1024 + 4 * l);
      idx[9] = 0;
      const uint4 sgv = *reinterpret_cast<const uint4*>(o + 1152 + 16 * l);
      const uint32_t sg[4] = {sgv.x, sgv.y, sgv.z, sgv.w};
      const uint32_t sc = *reinterpret_cast<const uint16_t*>(o + 1664 + 2 * l);
      const uint32_t sc_next = *reinterpret_cast<const uint16_t*>(o + 1664 + 2 * (l | 1));  // slice s | 1, same rows
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint8_t* b = base + (size_t)(a + 4 * i) * row_bytes + (size_t)j * 110;
        uint32_t qh = 0;
        uint32_t qs[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int bit = 9 * (8 * i + e), word = bit >> 5, off = bit & 31;
          uint32_t f = idx[word] >> off;
          if (off + 9 > 32) f |= idx[word + 1] << (32 - off);
          f &= 0x1FFu;
          qs[e] = f & 0xFFu;
          qh |= (f >> 8) << e;
        }
        // blocks are 2-byte aligned: write halfwords
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          *reinterpret_cast<uint16_t*>(b + 2 + 8 * s + e) = (uint16_t)(qs[e] | (qs[e + 1] << 8));
        }
        const uint32_t g = sign_gather(sg[i]);
        *reinterpret_cast<uint16_t*>(b + 74 + 4 * s) = (uint16_t)(g & 0xFFFFu);
        *reinterpret_cast<uint16_t*>(b + 76 + 4 * s) = (uint16_t)(g >> 16);
        if ((s & 1) == 0) {
          // slices s and s + 1 share a scale byte: the even one writes both nibbles
          const uint32_t nib0 = (sc >> (4 * i)) & 0xFu, nib1 = (sc_next >> (4 * i)) & 0xFu;
          b[106 + (s >> 1)] = (uint8_t)(nib0 | (nib1 << 4));
        }
        b[66 + s] = (uint8_t)qh;
      }
      if (s < 4) {
        uint8_t* b = base + (size_t)(a + 4 * s) * row_bytes + (size_t)j * 110;
        *reinterpret_cast<uint16_t*>(b) = *reinterpret_cast<const uint16_t*>(o + 1728 + 2 * (4 * a + s));
      }
    }
  }
}

}  // namespace gsq

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
