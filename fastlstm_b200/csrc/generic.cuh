// Declarations of the CUDA-core kernels' host launchers and their launch plan.
#pragma once
#include "common.cuh"

namespace blstm {

struct GenericPlan {
  static constexpr int kBT = 16;   // batch rows per CTA
  static constexpr int kUH = 8;    // hidden units per CTA
  static constexpr int kKC = 512;  // reduction chunk staged in shared memory
  int T, B, H;
  int nbt, nh;          // batch tiles, hidden tiles
  int nb_par, grid;     // batch tiles resident at once, CTAs (filled at launch)
  bool w_in_smem;
  size_t smem_bytes;
  size_t n_flags, off_flags, off_db, ws_bytes;
  void make(const blstm_desc& d, int phase);
};

// C[M,N] = A*B (+bias0+bias1); A(m,k) = A[m*sam + k*sak], B(k,n) = B[k*sbk + n*sbn].
// dtype selects the element type of A, B and the biases; C is fp32 when out_f32.
int generic_gemm(int dtype, bool out_f32, int M, int N, int K, const void* A, long long sam,
                 long long sak, const void* B, long long sbk, long long sbn, void* C, long long ldc,
                 const void* bias0, const void* bias1, cudaStream_t st);

int generic_fwd_recurrence(const blstm_desc& d, void* ifgo, const void* Wh, void* out, void* cell,
                           void* ws, size_t ws_bytes, cudaStream_t st);

int generic_bwd_recurrence(const blstm_desc& d, const void* dout, const void* dh_n, const void* dc_n,
                           const void* ifgo, const void* cell, const void* Wh, void* d_ifgo,
                           void* dh0, void* dc0, float* db, void* ws, size_t ws_bytes,
                           cudaStream_t st);

// Whole forward operator in one kernel for tiny hidden sizes (max(H, I) <= 32 in fp32, <= 64 in 16 bit):
// the input projection is computed inside the time loop.  out[0]/cell[0] must hold the initial state.
bool generic_fused_fwd_supported(const blstm_desc& d);
int generic_fused_fwd(const blstm_desc& d, const void* x, const void* Wx, const void* Wh, const void* bx,
                      const void* bh, void* ifgo, void* out, void* cell, cudaStream_t st);

int reduce_db(const float* part, int n_part, int n, float* db, cudaStream_t st);

// db[4H] = column sums of d_ifgo [T*B,4H]; scratch = the backward recurrence workspace of this plan
int generic_bias_grad(const blstm_desc& d, const void* d_ifgo, float* db, void* ws, size_t ws_bytes,
                      cudaStream_t st);

}  // namespace blstm
