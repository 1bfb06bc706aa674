// One-shot sum of the partial results of K-sharded products over peer memory (NVLink / NVSwitch), sm_100a.
//
// The reference has no collective of its own (vLLM's row-parallel layers call NCCL after apply()); at decode row
// counts the partial results are a few hundred KB, and an NCCL all-reduce costs a fixed ~15-25 us whatever the size.
// Here every rank keeps its partial result in a buffer its peers can read (symmetric memory set up by the host:
// the same offset on every GPU), and one small kernel per rank
//   1. tells every peer "my partial of epoch e is complete" (one 32-bit store into the peer's flag pad),
//   2. waits until every peer has said the same (bounded spin on its own pad), and
//   3. adds all ranks' partials in rank order (plain peer loads, 16 bytes each) and writes the sum locally.
// No TMA, no multicast load, no multimem: plain loads and stores over peer pointers. The sum is formed in fp32 in the
// same order on every rank, so all ranks hold bit-identical results and a run repeats bit for bit.
//
// Buffer reuse: the caller alternates between (at least) two partial buffers from one call to the next. A rank can
// only pass step 2 of call n + 1 once every peer has started call n + 1, hence finished reading the buffer of call n;
// so the buffer of call n may be rewritten after call n + 1 returns -- which an alternating pair guarantees.
#include "gsq_common.cuh"

namespace gsq {

__device__ int g_ar_error = 0;

struct ArArgs {
  const void* const* bufs;      // device array [world]: every rank's partial buffer (peer pointers, own included)
  uint32_t* const* flags;       // device array [world]: every rank's flag pad, `world` uint32 each
  int rank, world;
  int64_t nvec;                 // 16-byte vectors per buffer
  int dtype;
  void* out;
  uint32_t* epoch;              // this rank's call counter (device memory, starts at 0)
  uint32_t* done;               // this rank's block ticket (device memory, starts at 0)
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__device__ __forceinline__ void acc8(float (&s)[8], const uint4& v);
template <>
__device__ __forceinline__ void acc8<__nv_bfloat16>(float (&s)[8], const uint4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    s[2 * i] += f.x;
    s[2 * i + 1] += f.y;
  }
}
template <>
__device__ __forceinline__ void acc8<__half>(float (&s)[8], const uint4& v) {
  const __half2* p = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(p[i]);
    s[2 * i] += f.x;
    s[2 * i + 1] += f.y;
  }
}

template <int DT>
__global__ void __launch_bounds__(256) allreduce_kernel(const ArArgs a) {
  __shared__ int s_ok;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;   // this call's epoch: same in every block
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // 1. block 0: this rank's partial (written by the kernels before this one in the stream) is complete
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.flags[threadIdx.x] + a.rank, e);
  }
  // 2. every block: wait for every rank's flag in this rank's pad (bounded: gives up, raises the error flag)
  if (threadIdx.x < a.world) {
    const uint32_t* f = a.flags[a.rank] + threadIdx.x;
    bool ok = false;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (int spin = 0; spin < (1 << 24); ++spin) {       // bounded twice: by polls and by time (0.2 s)
      if ((int32_t)(ld_acquire_sys(f) - e) >= 0) { ok = true; break; }
      __nanosleep(20);
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 200000000ull) break;
    }
    if (!ok) {
      s_ok = 0;
      atomicExch(&g_ar_error, 1);
    }
  }
  __syncthreads();
  // 3. the sum, in rank order, 16 bytes per thread and step
  if (s_ok) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.nvec; i += (int64_t)gridDim.x * blockDim.x) {
      if (DT == GSQ_F32) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < a.world; ++r) {
          const uint4 v = __ldcv(reinterpret_cast<const uint4*>(a.bufs[r]) + i);
          s.x += __uint_as_float(v.x); s.y += __uint_as_float(v.y); s.z += __uint_as_float(v.z); s.w += __uint_as_float(v.w);
        }
        reinterpret_cast<float4*>(a.out)[i] = s;
      } else {
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < a.world; ++r) {
          const uint4 v = __ldcv(reinterpret_cast<const uint4*>(a.bufs[r]) + i);
          if (DT == GSQ_BF16) acc8<__nv_bfloat16>(s, v); else acc8<__half>(s, v);
        }
        uint4 o;
        if (DT == GSQ_BF16) {
          __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) p[q] = __floats2bfloat162_rn(s[2 * q], s[2 * q + 1]);
        } else {
          __half2* p = reinterpret_cast<__half2*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) p[q] = __floats2half2_rn(s[2 * q], s[2 * q + 1]);
        }
        reinterpret_cast<uint4*>(a.out)[i] = o;
      }
    }
  }
  // the last block to finish publishes the epoch for the next call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
      *a.done = 0u;
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = e;
    }
  }
}

}  // namespace gsq

extern "C" int gsq_allreduce_error_flag(int* flag) {
  if (!flag) return GSQ_ERR_UNSUPPORTED;
  GSQ_CUDA_TRY(cudaMemcpyFromSymbol(flag, gsq::g_ar_error, sizeof(int)));
  return GSQ_OK;
}

extern "C" int gsq_allreduce_sum(const void* const* peer_bufs, uint32_t* const* peer_flags, int rank, int world,
                                 int64_t count, int dtype, void* out, uint32_t* state, void* stream) {
  using namespace gsq;
  if (count == 0) return GSQ_OK;
  if (!peer_bufs || !peer_flags || !out || !state || world < 1 || world > 16 || rank < 0 || rank >= world || count < 0)
    return GSQ_ERR_UNSUPPORTED;
  const int64_t esz = dtype == GSQ_F32 ? 4 : (dtype == GSQ_F16 || dtype == GSQ_BF16) ? 2 : 0;
  if (esz == 0 || (count * esz) % 16 != 0 || (uintptr_t)out % 16 != 0) return GSQ_ERR_UNSUPPORTED;
  DeviceInfo di;
  const int rc = device_info(&di);
  if (rc != GSQ_OK) return rc;
  ArArgs a;
  a.bufs = peer_bufs;
  a.flags = peer_flags;
  a.rank = rank;
  a.world = world;
  a.nvec = count * esz / 16;
  a.dtype = dtype;
  a.out = out;
  a.epoch = state;
  a.done = state + 1;
  int64_t blocks = (a.nvec + 255) / 256;
  if (blocks > di.sm_count) blocks = di.sm_count;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case GSQ_F32: allreduce_kernel<GSQ_F32><<<(unsigned)blocks, 256, 0, st>>>(a); break;
    case GSQ_F16: allreduce_kernel<GSQ_F16><<<(unsigned)blocks, 256, 0, st>>>(a); break;
    default: allreduce_kernel<GSQ_BF16><<<(unsigned)blocks, 256, 0, st>>>(a); break;
  }
  GSQ_CUDA_TRY(cudaGetLastError());
  return GSQ_OK;
}
