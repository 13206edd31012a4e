// Small device helpers shared by the tcgen05 recurrence kernels: packed 16-bit <-> fp32
// conversion, 16-byte global accesses, tensor-memory column loads.
#pragma once

#include "sm100_common.cuh"

namespace blstm {
namespace sm100 {

template <typename T16> __device__ __forceinline__ float2 cvt2(uint32_t v);
template <> __device__ __forceinline__ float2 cvt2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <> __device__ __forceinline__ float2 cvt2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}
template <typename T16> __device__ __forceinline__ uint32_t pk2(float a, float b);
template <> __device__ __forceinline__ uint32_t pk2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pk2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void stg16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

template <typename T16>
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int u = 0; u < 4; ++u) { const float2 t = cvt2<T16>(w[u]); f[2 * u] = t.x; f[2 * u + 1] = t.y; }
}
template <typename T16>
__device__ __forceinline__ void store8(T16* dst, const float* f) {
  stg16(dst, make_uint4(pk2<T16>(f[0], f[1]), pk2<T16>(f[2], f[3]), pk2<T16>(f[4], f[5]), pk2<T16>(f[6], f[7])));
}
template <int NCOL>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[NCOL]) {
  if constexpr (NCOL == 16) tmem_ld_32x16(taddr, r); else tmem_ld_32x8(taddr, r);
}

}  // namespace sm100
}  // namespace blstm
