/*
 * fastlstm_b200 — C ABI of the B200 (sm_100a) LSTM layer kernels.
 *
 * The reference project (oleicht/FastLSTM) has no C/FFI boundary: its hot path
 * is reached through Python "operator" functions that launch Triton kernels and
 * cuBLAS GEMMs.  Each entry point below replaces one of those operator
 * functions (or one launch inside it); the citation names the reference code it
 * stands in for (paths are relative to the reference checkout).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; the library
 *     allocates nothing, callers own every buffer (workspace included);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and
 *     no entry point synchronises the host unless its comment says so;
 *   - tensors are dense row-major.  x [T,B,I], out/cell [T+1,B,H] (slot 0 holds
 *     the initial state), ifgo/d_ifgo [T,B,4H] with gate order i|f|g|o along 4H,
 *     Wx [4H,I], Wh [4H,H], biases [4H]; activations, states and weights share
 *     the element type `dtype`; weight/bias GRADIENTS are always fp32;
 *   - return value: 0 on success, a BLSTM_E_* code otherwise (see
 *     blstm_strerror).  Conditions found on the device (a bounded wait that ran
 *     out) are recorded in the workspace control block and read back with
 *     blstm_read_status.
 */
#ifndef FASTLSTM_B200_H_
#define FASTLSTM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BLSTM_ABI_VERSION 1

enum { BLSTM_F32 = 0, BLSTM_F16 = 1, BLSTM_BF16 = 2 };

/* status codes */
enum {
  BLSTM_OK = 0,
  BLSTM_E_INVALID_ARG = 1,     /* null pointer, non-positive size, unknown dtype, or a
                                  16-bit tensor pointer that is not 16-byte aligned     */
  BLSTM_E_UNSUPPORTED = 2,     /* shape/dtype combination no kernel covers               */
  BLSTM_E_WORKSPACE = 3,       /* workspace pointer null/misaligned or too small         */
  BLSTM_E_CUDA = 4,            /* a CUDA runtime/driver call failed (see blstm_last_cuda_error) */
  BLSTM_E_NOT_CORESIDENT = 5,  /* persistent grid cannot be made co-resident on this GPU */
  BLSTM_E_WAIT_TIMEOUT = 6,    /* device: a bounded cross-CTA wait ran out               */
  BLSTM_E_ARCH = 7,            /* device is not sm_100                                    */
  BLSTM_E_TOO_LARGE = 8        /* request exceeds a fixed capacity (no-allocation entry) */
};

/* blstm_desc.flags */
enum {
  BLSTM_FLAG_FORCE_GENERIC = 1, /* use the CUDA-core kernels even where a tcgen05 kernel exists */
  BLSTM_FLAG_RESERVED = 2,
  BLSTM_FLAG_INFERENCE = 8,     /* forward only: the recurrence does not write back the final
                                   pre-activations nor cell[1..T-1] (nothing is saved for backward);
                                   out[1..T] and cell[T] are still produced.  Halves the bytes a
                                   step moves (5*B*H*e instead of 10*B*H*e). */
  BLSTM_FLAG_NO_FUSED = 32,     /* blstm_fwd: do not use the single-kernel forward (projection inside the
                                   time loop) that tiny sizes (max(H, I) <= 32 in fp32, <= 64 in 16 bit)
                                   otherwise get; for comparisons and tests */
  BLSTM_FLAG_HALF_DEVICE = 128, /* recurrences: plan for half of the SMs, so that two persistent kernels (two
                                   layers of a stack working on neighbouring time chunks) fit side by side */
  BLSTM_FLAG_NO_CLUSTER = 16,   /* forward: do not use the cluster hand-off kernel that small hidden
                                   sizes (H = 64, 128, 256 with at most 7 batch tiles) otherwise get;
                                   for comparisons and tests */
  BLSTM_FLAG_TEST_NO_ARRIVE = 4 /* test hook: CTAs never signal step completion, so every
                                   cross-CTA wait runs into wait_limit_us and the launch ends
                                   with BLSTM_E_WAIT_TIMEOUT in the control block (no fault) */
};

typedef struct blstm_desc {
  int32_t dtype;        /* BLSTM_F32 / BLSTM_F16 / BLSTM_BF16                            */
  int32_t seq_len;      /* T                                                             */
  int32_t batch;        /* B                                                             */
  int32_t input_size;   /* I                                                             */
  int32_t hidden_size;  /* H                                                             */
  int32_t flags;        /* BLSTM_FLAG_*                                                  */
  int32_t wait_limit_us;/* cap on any single device-side wait; 0 = default (2 s)         */
  int32_t reserved;
} blstm_desc;

/* BLSTM_PHASE_FWD_OP (plan queries only): the whole forward operator blstm_fwd, which for tiny sizes
 * is one fused kernel ("fused") and otherwise projection + BLSTM_PHASE_FWD recurrence. */
enum { BLSTM_PHASE_FWD = 0, BLSTM_PHASE_BWD = 1, BLSTM_PHASE_FWD_OP = 2 };

/* ABI version of the loaded library (compare with BLSTM_ABI_VERSION). */
int blstm_abi_version(void);

/* Human-readable text for a status code.  Replaces the reference's Python
 * assert/ValueError messages (fastlstm/lstm.py:49-50,77-80,531,683). */
const char* blstm_strerror(int code);

/* Text of the last CUDA error this library saw on the calling thread (HOST string). */
const char* blstm_last_cuda_error(void);

/* 0 if `device` can run these kernels (sm_100, cooperative launch); replaces the
 * import-time device query of fastlstm/configs.py:5-6. */
int blstm_device_check(int device);

/* Bytes of workspace the phase needs for this problem (>= 256, multiple of 256).
 * Replaces the per-call `global_sync`/`sync` allocations of
 * fastlstm/lstm.py:96-100 and :249. */
size_t blstm_workspace_bytes(const blstm_desc* d, int phase);

/* Name of the kernel family the phase will use for this problem ("generic",
 * "sm100"); HOST string.  Stands in for the reference's launch-geometry
 * choice, fastlstm/configs.py:146-276 (prune_persistent_configs) and :29-58. */
const char* blstm_plan_name(const blstm_desc* d, int phase);

/* Writes a one-line, human-readable description of the launch geometry the phase will use
 * (tile sizes, interleaved batch tiles, grid, ring depth) into the HOST buffer `buf`.
 * Read-only; stands in for inspecting the reference's chosen autotune config
 * (fastlstm/configs.py:146-276). */
int blstm_plan_detail(const blstm_desc* d, int phase, char* buf, size_t buf_bytes);

/* ifgo[T*B,4H] = x[T*B,I] * Wx^T + (bx + bh); bx/bh may be NULL.
 * Replaces torch.addmm at fastlstm/lstm.py:66-68. */
int blstm_input_projection(const blstm_desc* d, const void* x, const void* Wx,
                           const void* bx, const void* bh, void* ifgo, void* stream);

/* Persistent forward recurrence over all T steps: reads the projected
 * pre-activations in `ifgo`, overwrites them with the final pre-activations,
 * fills out[1..T], cell[1..T]; out[0]/cell[0] must already hold h0/c0.
 * Replaces the persistent_fwd_kernel launch, fastlstm/lstm.py:131-142
 * (kernel: fastlstm/kernels.py:414-663). */
int blstm_fwd_recurrence(const blstm_desc* d, void* ifgo, const void* Wh, void* out,
                         void* cell, void* workspace, size_t workspace_bytes, void* stream);

/* Whole forward operator: initial-state slots, projection, recurrence.
 * h0/c0 [B,H] may both be NULL (zeros).  Replaces lstm_persistent_fwd,
 * fastlstm/lstm.py:31-146, including its dispatch of tiny sizes to the fully fused kernel
 * (fastlstm/lstm.py:40-47, fastlstm/kernels.py:672-819): one launch, no projected
 * pre-activations in memory, no workspace use. */
int blstm_fwd(const blstm_desc* d, const void* x, const void* h0, const void* c0,
              const void* Wx, const void* Wh, const void* bx, const void* bh,
              void* out, void* cell, void* ifgo,
              void* workspace, size_t workspace_bytes, void* stream);

/* Persistent reverse-time recurrence: d_ifgo[T,B,4H], final carries dh0/dc0
 * [B,H], db[4H] (fp32, = sum over t,b of d_ifgo).  dout [T,B,H] is the gradient
 * of out[1..T]; dh_n/dc_n [B,H] (NULL = zeros) are gradients of the final
 * states and may alias dh0/dc0.  Replaces the lstm_persistent_seq_bwd launch,
 * fastlstm/lstm.py:277-290 (kernel: fastlstm/kernels.py:1201-1409) and the
 * bias reduction of fastlstm/lstm.py:497. */
int blstm_bwd_recurrence(const blstm_desc* d, const void* dout, const void* dh_n,
                         const void* dc_n, const void* ifgo, const void* cell,
                         const void* Wh, void* d_ifgo, void* dh0, void* dc0, float* db,
                         void* workspace, size_t workspace_bytes, void* stream);

/* dx[T*B,I] = d_ifgo[T*B,4H] * Wx.  Replaces `d_ifgo @ Wx`, fastlstm/lstm.py:294. */
int blstm_dgrad_input(const blstm_desc* d, const void* d_ifgo, const void* Wx, void* dx,
                      void* workspace, size_t workspace_bytes, void* stream);

/* dWx[4H,I] = d_ifgo^T * x, dWh[4H,H] = d_ifgo^T * out[0..T-1]; fp32 outputs.
 * Replaces Wgrad, fastlstm/lstm.py:494-501 (without its transpose copy). */
int blstm_wgrad(const blstm_desc* d, const void* d_ifgo, const void* x, const void* out,
                float* dWx, float* dWh, void* workspace, size_t workspace_bytes, void* stream);

/* db[4H] (fp32) = sum over t,b of d_ifgo[T*B,4H]; `workspace` as for BLSTM_PHASE_BWD.
 * Replaces `d_ifgo.sum(0)` of Wgrad, fastlstm/lstm.py:497 (blstm_bwd_recurrence already
 * returns db; this entry serves callers that hold only d_ifgo). */
int blstm_bias_grad(const blstm_desc* d, const void* d_ifgo, float* db, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Whole backward operator = bwd recurrence + dgrad + wgrad.  dx may be NULL
 * (input needs no gradient).  Replaces lstm_persistent_bwd, fastlstm/lstm.py:236-334. */
int blstm_bwd(const blstm_desc* d, const void* dout, const void* dh_n, const void* dc_n,
              const void* x, const void* out, const void* cell, const void* ifgo,
              const void* Wx, const void* Wh,
              void* d_ifgo, void* dx, void* dh0, void* dc0,
              float* dWx, float* dWh, float* db,
              void* workspace, size_t workspace_bytes, void* stream);

/* Copies the workspace control block to the host and WAITS for `stream`;
 * returns the device-recorded status (0, or BLSTM_E_WAIT_TIMEOUT with
 * detail[0] = step index, detail[1] = batch tile).  detail may be NULL.
 * The reference has no counterpart: its spin-waits are unbounded
 * (fastlstm/kernels.py:546-548,1358-1359). */
int blstm_read_status(const void* workspace, int32_t* detail, void* stream);

/* Forward recurrence WITHOUT a caller-provided workspace.  It has no counterpart in the
 * reference.  Same contract as blstm_fwd_recurrence (ifgo in/out, out[0]/cell[0] preset,
 * out[1..T]/cell[1..T] written), but the kernel's scratch - control block and arrival
 * counters - is a fixed 1 MiB array inside the library's device image, so the call performs
 * no device allocation of any kind.  It is meant for callers that cannot allocate: a server
 * whose own arena already owns all free HBM, or a plug-in whose host forbids cudaMalloc once
 * it is initialised.
 *   - Limit: blstm_workspace_bytes(d, BLSTM_PHASE_FWD) must be <= blstm_static_scratch_capacity()
 *     (1 MiB: e.g. T = 1024 with up to 255 batch tiles); larger problems return BLSTM_E_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (the device must be
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array: two calls that overlap on the GPU (different
 *     streams, or a second process-wide caller) race on it.  Serialise them.
 *   - Device-side status of the last call: blstm_static_scratch_status (waits for `stream`). */
int blstm_fwd_recurrence_static(const blstm_desc* d, void* ifgo, const void* Wh, void* out,
                                void* cell, void* stream);
size_t blstm_static_scratch_capacity(void);
int blstm_static_scratch_status(int32_t* detail, void* stream);

/* Number of kernels this library has launched in this process so far (HOST
 * counter; memsets and copies are not counted).  Benchmarks report the
 * difference across their timed region.  No reference counterpart. */
unsigned long long blstm_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FASTLSTM_B200_H_ */
