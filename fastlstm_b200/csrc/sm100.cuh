// Host launchers of the tcgen05/TMEM + TMA kernels (16-bit element types).
#pragma once
#include "common.cuh"

namespace blstm {

// true when the tcgen05 GEMMs cover this problem (projection, dgrad, wgrad)
bool sm100_gemm_supported(const blstm_desc& d);
// scratch the backward GEMMs need (bytes)
size_t sm100_bwd_gemm_workspace(const blstm_desc& d);

int sm100_input_projection(const blstm_desc& d, const void* x, const void* Wx, const void* bx,
                           const void* bh, void* ifgo, cudaStream_t st);
int sm100_dgrad_input(const blstm_desc& d, const void* d_ifgo, const void* Wx, void* dx, void* ws,
                      size_t ws_bytes, cudaStream_t st);
int sm100_wgrad(const blstm_desc& d, const void* d_ifgo, const void* x, const void* out, float* dWx,
                float* dWh, void* ws, size_t ws_bytes, cudaStream_t st);

// true when the tcgen05 persistent recurrence covers this problem
bool sm100_recurrence_supported(const blstm_desc& d, int phase);
size_t sm100_recurrence_workspace(const blstm_desc& d, int phase);
int sm100_fwd_recurrence(const blstm_desc& d, void* ifgo, const void* Wh, void* out, void* cell,
                         void* ws, size_t ws_bytes, cudaStream_t st);
int sm100_bwd_recurrence(const blstm_desc& d, const void* dout, const void* dh_n, const void* dc_n,
                         const void* ifgo, const void* cell, const void* Wh, void* d_ifgo, void* dh0,
                         void* dc0, float* db, void* ws, size_t ws_bytes, cudaStream_t st);

// Small hidden sizes (H = 64, 128, 256) with few batch tiles: the forward recurrence whose CTAs hand
// h over inside one cluster per batch tile.  *taken = false when the shape (or the device's cluster
// capacity) does not allow it and the general kernel has to run.  `ws` = zeroed control block.
bool sm100_fwd_cluster_shape(const blstm_desc& d);
int sm100_fwd_cluster(const blstm_desc& d, void* ifgo, const void* Wh, void* out, void* cell, void* ws,
                      cudaStream_t st, bool* taken);

// one-line description of the launch plan of a phase ("" when the tcgen05 kernels do not cover it)
int sm100_plan_detail(const blstm_desc& d, int phase, char* buf, size_t n);

// db[4H] = column sums of d_ifgo [T*B,4H] (16-bit); scratch = the backward recurrence workspace
int sm100_bias_grad(const blstm_desc& d, const void* d_ifgo, float* db, void* ws, size_t ws_bytes,
                    cudaStream_t st);

}  // namespace blstm
