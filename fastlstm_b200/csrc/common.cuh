// Shared device/host helpers: element-type traits, gate math, the workspace
// control block and bounded cross-CTA waits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fastlstm_b200.h"

namespace blstm {

// ---------------------------------------------------------------------------
// Workspace control block (first 256 bytes of every workspace).  Zeroed by the
// host entry point with a stream-ordered memset before each launch.
// ---------------------------------------------------------------------------
struct Control {
  int abort;        // set by the first CTA whose wait ran out; polled by all spinners
  int status;       // BLSTM_OK or BLSTM_E_WAIT_TIMEOUT
  int detail[2];    // step index, batch tile of the wait that gave up
  int pad[60];
};
static_assert(sizeof(Control) == 256, "control block is 256 bytes");

constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // 2 s

// ---------------------------------------------------------------------------
// Element types
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float ld_f(const T* p) { return Elem<T>::to_f(*p); }
// load that bypasses the (non-coherent) L1: for data written by other SMs during this kernel
template <typename T> __device__ __forceinline__ float ld_cg_f(const T* p);
template <> __device__ __forceinline__ float ld_cg_f<float>(const float* p) { return __ldcg(p); }
template <> __device__ __forceinline__ float ld_cg_f<__half>(const __half* p) {
  unsigned short r = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __half2float(__ushort_as_half(r));
}
template <> __device__ __forceinline__ float ld_cg_f<__nv_bfloat16>(const __nv_bfloat16* p) {
  unsigned short r = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __bfloat162float(__ushort_as_bfloat16(r));
}

// ---------------------------------------------------------------------------
// Gate math.  Accurate forms (expf/tanhf) for the fp32 path, MUFU forms for
// the 16-bit tensor-core path whose storage rounding (2^-9 / 2^-12) dwarfs the
// approximation error (about 2^-11 relative for tanh.approx).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_acc(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float tanh_acc(float x) { return tanhf(x); }
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_fast(float x) { return fmaf(tanh_fast(0.5f * x), 0.5f, 0.5f); }

// ---------------------------------------------------------------------------
// Bounded waits on global flags
// ---------------------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Spin until *flag >= target.  Gives up (returns false) when another CTA has
// raised ctl->abort or when limit_ns elapsed; in the latter case it records
// BLSTM_E_WAIT_TIMEOUT with (d0, d1) and raises abort so every other spinner
// leaves promptly.  Never traps, never spins unbounded.
static __device__ __noinline__ bool wait_flag_ge(const int* flag, int target, Control* ctl,
                                          unsigned long long limit_ns, int d0, int d1) {
  if (ld_acquire_gpu(flag) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    if (ld_acquire_gpu(flag) >= target) return true;
    if ((++spins & 31u) == 0u) {
      if (ld_relaxed_gpu(&ctl->abort) != 0) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        if (atomicCAS(&ctl->status, 0, BLSTM_E_WAIT_TIMEOUT) == 0) {
          ctl->detail[0] = d0;
          ctl->detail[1] = d1;
        }
        atomicExch(&ctl->abort, 1);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host-side error plumbing
// ---------------------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);
void count_launch(int n = 1);  // bump the per-process kernel-launch counter

#define BLSTM_CUDA_OK(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      ::blstm::set_cuda_error(_e, #expr);                    \
      return BLSTM_E_CUDA;                                   \
    }                                                        \
  } while (0)

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }

struct DeviceInfo {
  int device;
  int sm_count;
  int cc_major, cc_minor;
  int coop;
  size_t smem_optin;
};
int get_device_info(DeviceInfo* out);  // current device, cached per device
// SM count the launch plans are sized for: the current device's, or 148 (a full B200) when no
// device can be queried (workspace sizes asked for on a host without a GPU).
int plan_sm_count();

}  // namespace blstm
