// blstm_fwd_recurrence_static: the forward recurrence for callers that cannot give the
// library a workspace because they cannot allocate device memory at all - for example a
// serving process that has handed every free byte of HBM to its own arena at start-up, or a
// plug-in running under a host that forbids cudaMalloc after initialisation (it would
// serialise the device and break the host's latency budget).  They still own the inputs and
// outputs; only the kernel's scratch (control block + per-(step, batch tile) arrival
// counters) comes from a fixed array that lives in this library's device image.
#include <mutex>

#include "generic.cuh"
#include "sm100.cuh"

namespace blstm {

// Scratch of the no-allocation entry point.  Every GPU that loads the library holds these
// bytes until the process exits.  In HOST code `g_static_scratch` is only a stand-in for the
// symbol, never a device address: the address is obtained with cudaGetSymbolAddress below.
constexpr size_t kStaticScratchBytes = 1u << 20;   // 1 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array on the CURRENT device; looked up once per device.
static int static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* ptrs[64] = {};
  int dev = 0;
  BLSTM_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return BLSTM_E_INVALID_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    BLSTM_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));   // device `dev` is current here
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return BLSTM_OK;
}

}  // namespace blstm

using namespace blstm;

extern "C" {

size_t blstm_static_scratch_capacity(void) { return kStaticScratchBytes; }

int blstm_fwd_recurrence_static(const blstm_desc* d, void* ifgo, const void* Wh, void* out, void* cell,
                                void* stream) {
  if (!d || !ifgo || !Wh || !out || !cell) return BLSTM_E_INVALID_ARG;
  const size_t need = blstm_workspace_bytes(d, BLSTM_PHASE_FWD);
  if (need == 0) return BLSTM_E_INVALID_ARG;            // bad descriptor
  if (d->dtype != BLSTM_F32 &&
      ((reinterpret_cast<uintptr_t>(ifgo) | reinterpret_cast<uintptr_t>(Wh) | reinterpret_cast<uintptr_t>(out) |
        reinterpret_cast<uintptr_t>(cell)) & 15u) != 0)
    return BLSTM_E_INVALID_ARG;                           // 16-bit tensors move in 16-byte pieces
  if (need > kStaticScratchBytes) return BLSTM_E_TOO_LARGE;
  void* ws = nullptr;
  int rc = static_scratch_ptr(&ws);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // The launchers below clear the control block and every counter they use with a
  // stream-ordered memset before the kernel, so the previous call's contents never leak in.
  if (sm100_recurrence_supported(*d, BLSTM_PHASE_FWD))
    return sm100_fwd_recurrence(*d, ifgo, Wh, out, cell, ws, kStaticScratchBytes, st);
  return generic_fwd_recurrence(*d, ifgo, Wh, out, cell, ws, kStaticScratchBytes, st);
}

int blstm_static_scratch_status(int32_t* detail, void* stream) {
  void* ws = nullptr;
  int rc = static_scratch_ptr(&ws);
  if (rc) return rc;
  return blstm_read_status(ws, detail, stream);
}

}  // extern "C"
