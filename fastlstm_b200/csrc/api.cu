// extern "C" entry points (declared in include/fastlstm_b200.h): argument
// validation, kernel-family choice, workspace carving.  No allocation, no
// host synchronisation except blstm_read_status.
#include <atomic>
#include <mutex>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "generic.cuh"
#include "sm100.cuh"

namespace blstm {

static thread_local char g_cuda_err[256] = "";

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e), where);
  (void)cudaGetLastError();  // clear the sticky-free error so later calls start clean
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int get_device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  static bool have[64] = {};
  int dev = 0;
  BLSTM_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return BLSTM_E_INVALID_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo di;
    di.device = dev;
    int v = 0;
    BLSTM_CUDA_OK(cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev));
    BLSTM_CUDA_OK(cudaDeviceGetAttribute(&di.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    BLSTM_CUDA_OK(cudaDeviceGetAttribute(&di.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    BLSTM_CUDA_OK(cudaDeviceGetAttribute(&di.coop, cudaDevAttrCooperativeLaunch, dev));
    BLSTM_CUDA_OK(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    di.smem_optin = (size_t)v;
    cache[dev] = di;
    have[dev] = true;
  }
  *out = cache[dev];
  return BLSTM_OK;
}

int plan_sm_count() {
  DeviceInfo di;
  if (get_device_info(&di) != BLSTM_OK || di.sm_count <= 0) return 148;
  return di.sm_count;
}

static int check_desc(const blstm_desc* d) {
  if (!d) return BLSTM_E_INVALID_ARG;
  if (d->dtype != BLSTM_F32 && d->dtype != BLSTM_F16 && d->dtype != BLSTM_BF16) return BLSTM_E_INVALID_ARG;
  if (d->seq_len <= 0 || d->batch <= 0 || d->input_size <= 0 || d->hidden_size <= 0) return BLSTM_E_INVALID_ARG;
  if (d->wait_limit_us < 0) return BLSTM_E_INVALID_ARG;
  return BLSTM_OK;
}

static size_t esize(int dtype) { return dtype == BLSTM_F32 ? 4 : 2; }

// The 16-bit kernels move every tensor in 16-byte pieces (vector loads and stores, TMA): all tensor
// base pointers must be 16-byte aligned there (null pointers, where allowed, pass).
template <typename... P>
static bool aligned16(int dtype, P... ptrs) {
  if (dtype == BLSTM_F32) return true;
  uintptr_t m = 0;
  ((m |= reinterpret_cast<uintptr_t>(ptrs)), ...);
  return (m & 15u) == 0;
}

static bool ws_ok(const void* ws, size_t have, size_t need) {
  return ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0 && have >= need;
}

// Workspace of the backward operator = [recurrence part | GEMM scratch part].
struct BwdLayout {
  size_t rec_bytes, gemm_off, gemm_bytes, total;
};
static BwdLayout bwd_layout(const blstm_desc& d) {
  BwdLayout L;
  if (sm100_recurrence_supported(d, BLSTM_PHASE_BWD)) {
    L.rec_bytes = sm100_recurrence_workspace(d, BLSTM_PHASE_BWD);
  } else {
    GenericPlan pl;
    pl.make(d, BLSTM_PHASE_BWD);
    L.rec_bytes = pl.ws_bytes;
  }
  L.gemm_off = round_up(L.rec_bytes, 256);
  L.gemm_bytes = sm100_gemm_supported(d) ? sm100_bwd_gemm_workspace(d) : 0;
  L.total = round_up(L.gemm_off + L.gemm_bytes, 256);
  return L;
}

}  // namespace blstm

using namespace blstm;

extern "C" {

int blstm_abi_version(void) { return BLSTM_ABI_VERSION; }

const char* blstm_strerror(int code) {
  switch (code) {
    case BLSTM_OK: return "ok";
    case BLSTM_E_INVALID_ARG: return "invalid argument (null pointer, non-positive size, unknown dtype, or a 16-bit tensor not 16-byte aligned)";
    case BLSTM_E_UNSUPPORTED: return "shape/dtype combination not supported";
    case BLSTM_E_WORKSPACE: return "workspace missing, not 256-byte aligned, or too small";
    case BLSTM_E_CUDA: return "CUDA call failed (see blstm_last_cuda_error)";
    case BLSTM_E_NOT_CORESIDENT: return "persistent grid cannot be co-resident on this device";
    case BLSTM_E_WAIT_TIMEOUT: return "device-side wait ran out (peer CTA never arrived)";
    case BLSTM_E_ARCH: return "device is not sm_100 (B200)";
    case BLSTM_E_TOO_LARGE: return "request exceeds the fixed capacity of this entry point";
  }
  return "unknown status code";
}

const char* blstm_last_cuda_error(void) { return g_cuda_err; }

int blstm_device_check(int device) {
  int n = 0;
  BLSTM_CUDA_OK(cudaGetDeviceCount(&n));
  if (device < 0 || device >= n) return BLSTM_E_INVALID_ARG;
  int major = 0, coop = 0;
  BLSTM_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  BLSTM_CUDA_OK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
  if (major != 10) return BLSTM_E_ARCH;
  if (!coop) return BLSTM_E_NOT_CORESIDENT;
  return BLSTM_OK;
}

size_t blstm_workspace_bytes(const blstm_desc* d, int phase) {
  if (check_desc(d)) return 0;
  if (phase == BLSTM_PHASE_FWD) {
    if (sm100_recurrence_supported(*d, phase)) return round_up(sm100_recurrence_workspace(*d, phase), 256);
    GenericPlan pl;
    pl.make(*d, phase);
    return round_up(pl.ws_bytes, 256);
  }
  if (phase == BLSTM_PHASE_BWD) return bwd_layout(*d).total;
  return 0;
}

const char* blstm_plan_name(const blstm_desc* d, int phase) {
  if (check_desc(d)) return "invalid";
  if (phase == BLSTM_PHASE_FWD_OP) {
    if (generic_fused_fwd_supported(*d)) return "fused";
    phase = BLSTM_PHASE_FWD;
  }
  return sm100_recurrence_supported(*d, phase) ? "sm100" : "generic";
}

int blstm_plan_detail(const blstm_desc* d, int phase, char* buf, size_t buf_bytes) {
  if (!buf || buf_bytes == 0) return BLSTM_E_INVALID_ARG;
  buf[0] = 0;
  int rc = check_desc(d);
  if (rc) return rc;
  if (phase == BLSTM_PHASE_FWD_OP) {
    if (generic_fused_fwd_supported(*d)) {
      snprintf(buf, buf_bytes, "fused fwd (projection inside the time loop) rows_per_cta=4 grid=%d threads=%d",
               (d->batch + 3) / 4, 4 * d->hidden_size);
      return BLSTM_OK;
    }
    phase = BLSTM_PHASE_FWD;
  }
  if (sm100_recurrence_supported(*d, phase)) {
    sm100_plan_detail(*d, phase, buf, buf_bytes);
  } else {
    GenericPlan pl;
    pl.make(*d, phase);
    snprintf(buf, buf_bytes, "generic %s rows_per_cta=%d units_per_cta=%d batch_tiles=%d hidden_tiles=%d wh=%s",
             phase == BLSTM_PHASE_BWD ? "bwd" : "fwd", GenericPlan::kBT, GenericPlan::kUH, pl.nbt, pl.nh,
             pl.w_in_smem ? "resident" : "global");
  }
  return BLSTM_OK;
}

int blstm_input_projection(const blstm_desc* d, const void* x, const void* Wx, const void* bx,
                           const void* bh, void* ifgo, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!x || !Wx || !ifgo) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, x, Wx, ifgo)) return BLSTM_E_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int M = d->seq_len * d->batch, N = 4 * d->hidden_size, K = d->input_size;
  if (sm100_gemm_supported(*d)) return sm100_input_projection(*d, x, Wx, bx, bh, ifgo, st);
  return generic_gemm(d->dtype, false, M, N, K, x, K, 1, Wx, 1, K, ifgo, N, bx, bh, st);
}

int blstm_fwd_recurrence(const blstm_desc* d, void* ifgo, const void* Wh, void* out, void* cell,
                         void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!ifgo || !Wh || !out || !cell) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, ifgo, Wh, out, cell)) return BLSTM_E_INVALID_ARG;
  if (!ws_ok(workspace, workspace_bytes, blstm_workspace_bytes(d, BLSTM_PHASE_FWD))) return BLSTM_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (sm100_recurrence_supported(*d, BLSTM_PHASE_FWD))
    return sm100_fwd_recurrence(*d, ifgo, Wh, out, cell, workspace, workspace_bytes, st);
  return generic_fwd_recurrence(*d, ifgo, Wh, out, cell, workspace, workspace_bytes, st);
}

int blstm_fwd(const blstm_desc* d, const void* x, const void* h0, const void* c0, const void* Wx,
              const void* Wh, const void* bx, const void* bh, void* out, void* cell, void* ifgo,
              void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!x || !Wx || !Wh || !out || !cell || !ifgo) return BLSTM_E_INVALID_ARG;
  if ((h0 == nullptr) != (c0 == nullptr)) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, x, h0, c0, Wx, Wh, bx, bh, out, cell, ifgo)) return BLSTM_E_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t slot = (size_t)d->batch * d->hidden_size * esize(d->dtype);
  if (h0) {
    BLSTM_CUDA_OK(cudaMemcpyAsync(out, h0, slot, cudaMemcpyDeviceToDevice, st));
    BLSTM_CUDA_OK(cudaMemcpyAsync(cell, c0, slot, cudaMemcpyDeviceToDevice, st));
  } else {
    BLSTM_CUDA_OK(cudaMemsetAsync(out, 0, slot, st));
    BLSTM_CUDA_OK(cudaMemsetAsync(cell, 0, slot, st));
  }
  if (generic_fused_fwd_supported(*d)) {
    // the kernel records nothing on the device, but callers read the control block afterwards
    if (workspace && workspace_bytes >= sizeof(Control)) BLSTM_CUDA_OK(cudaMemsetAsync(workspace, 0, sizeof(Control), st));
    return generic_fused_fwd(*d, x, Wx, Wh, bx, bh, ifgo, out, cell, st);
  }
  rc = blstm_input_projection(d, x, Wx, bx, bh, ifgo, stream);
  if (rc) return rc;
  return blstm_fwd_recurrence(d, ifgo, Wh, out, cell, workspace, workspace_bytes, stream);
}

int blstm_bwd_recurrence(const blstm_desc* d, const void* dout, const void* dh_n, const void* dc_n,
                         const void* ifgo, const void* cell, const void* Wh, void* d_ifgo, void* dh0,
                         void* dc0, float* db, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!dout || !ifgo || !cell || !Wh || !d_ifgo || !dh0 || !dc0) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, db)) return BLSTM_E_INVALID_ARG;
  const BwdLayout L = bwd_layout(*d);
  if (!ws_ok(workspace, workspace_bytes, L.rec_bytes)) return BLSTM_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (sm100_recurrence_supported(*d, BLSTM_PHASE_BWD))
    return sm100_bwd_recurrence(*d, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, db, workspace,
                                L.rec_bytes, st);
  return generic_bwd_recurrence(*d, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, db, workspace,
                                L.rec_bytes, st);
}

int blstm_dgrad_input(const blstm_desc* d, const void* d_ifgo, const void* Wx, void* dx,
                      void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!d_ifgo || !Wx || !dx) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, d_ifgo, Wx, dx)) return BLSTM_E_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int M = d->seq_len * d->batch, N = d->input_size, K = 4 * d->hidden_size;
  if (sm100_gemm_supported(*d)) {
    const BwdLayout L = bwd_layout(*d);
    if (!ws_ok(workspace, workspace_bytes, L.total)) return BLSTM_E_WORKSPACE;
    return sm100_dgrad_input(*d, d_ifgo, Wx, dx, static_cast<char*>(workspace) + L.gemm_off, L.gemm_bytes, st);
  }
  return generic_gemm(d->dtype, false, M, N, K, d_ifgo, K, 1, Wx, N, 1, dx, N, nullptr, nullptr, st);
}

int blstm_wgrad(const blstm_desc* d, const void* d_ifgo, const void* x, const void* out, float* dWx,
                float* dWh, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!d_ifgo || !x || !out || !dWx || !dWh) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, d_ifgo, x, out, dWx, dWh)) return BLSTM_E_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int TB = d->seq_len * d->batch, G = 4 * d->hidden_size, I = d->input_size, H = d->hidden_size;
  if (sm100_gemm_supported(*d)) {
    const BwdLayout L = bwd_layout(*d);
    if (!ws_ok(workspace, workspace_bytes, L.total)) return BLSTM_E_WORKSPACE;
    return sm100_wgrad(*d, d_ifgo, x, out, dWx, dWh, static_cast<char*>(workspace) + L.gemm_off, L.gemm_bytes, st);
  }
  rc = generic_gemm(d->dtype, true, G, I, TB, d_ifgo, 1, G, x, I, 1, dWx, I, nullptr, nullptr, st);
  if (rc) return rc;
  return generic_gemm(d->dtype, true, G, H, TB, d_ifgo, 1, G, out, H, 1, dWh, H, nullptr, nullptr, st);
}

int blstm_bias_grad(const blstm_desc* d, const void* d_ifgo, float* db, void* workspace,
                    size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!d_ifgo || !db) return BLSTM_E_INVALID_ARG;
  if (!aligned16(d->dtype, d_ifgo, db)) return BLSTM_E_INVALID_ARG;
  const BwdLayout L = bwd_layout(*d);
  if (!ws_ok(workspace, workspace_bytes, L.rec_bytes)) return BLSTM_E_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (sm100_recurrence_supported(*d, BLSTM_PHASE_BWD)) return sm100_bias_grad(*d, d_ifgo, db, workspace, L.rec_bytes, st);
  return generic_bias_grad(*d, d_ifgo, db, workspace, L.rec_bytes, st);
}

int blstm_bwd(const blstm_desc* d, const void* dout, const void* dh_n, const void* dc_n, const void* x,
              const void* out, const void* cell, const void* ifgo, const void* Wx, const void* Wh,
              void* d_ifgo, void* dx, void* dh0, void* dc0, float* dWx, float* dWh, float* db,
              void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_desc(d);
  if (rc) return rc;
  if (!x || !out || !Wx) return BLSTM_E_INVALID_ARG;
  if (!ws_ok(workspace, workspace_bytes, blstm_workspace_bytes(d, BLSTM_PHASE_BWD))) return BLSTM_E_WORKSPACE;
  rc = blstm_bwd_recurrence(d, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, db, workspace,
                            workspace_bytes, stream);
  if (rc) return rc;
  if (dx) {
    rc = blstm_dgrad_input(d, d_ifgo, Wx, dx, workspace, workspace_bytes, stream);
    if (rc) return rc;
  }
  if (dWx && dWh) rc = blstm_wgrad(d, d_ifgo, x, out, dWx, dWh, workspace, workspace_bytes, stream);
  return rc;
}

unsigned long long blstm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int blstm_read_status(const void* workspace, int32_t* detail, void* stream) {
  if (!workspace) return BLSTM_E_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  int host[4] = {0, 0, 0, 0};
  BLSTM_CUDA_OK(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, st));
  BLSTM_CUDA_OK(cudaStreamSynchronize(st));
  if (detail) {
    detail[0] = host[2];
    detail[1] = host[3];
  }
  return host[1];
}

}  // extern "C"
