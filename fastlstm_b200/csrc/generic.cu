// CUDA-core (FFMA) kernels: the fp32 path (tolerance 1e-5 forbids TF32) and the
// path for shapes the tcgen05 kernels do not cover (ragged H/I/B).
//
//   gemm_generic_kernel   C = A*B (+bias), fp32 accumulate, arbitrary strides
//   gen_fwd_kernel        persistent forward recurrence   (reference: fastlstm/kernels.py:414-663)
//   gen_bwd_kernel        persistent reverse recurrence   (reference: fastlstm/kernels.py:1201-1409)
//   reduce_db_kernel      db = sum of per-batch-tile partial bias gradients
//
// Both recurrences are single cooperative launches: CTAs own (batch tile x
// hidden tile), carry c / dc / dh in fp32 registers over the time loop and
// hand h[t] (or d_ifgo[t]) to their peers through global memory, one int32
// arrival counter per (step, batch tile), every wait bounded.
#include "generic.cuh"

namespace blstm {

// ---------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------
constexpr int GM = 64, GN = 64, GK = 16;

template <typename TA, typename TB, typename TC, typename TBias>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(int M, int N, int K, const TA* __restrict__ A, long long sam, long long sak,
                    const TB* __restrict__ B, long long sbk, long long sbn, TC* __restrict__ C,
                    long long ldc, const TBias* __restrict__ bias0, const TBias* __restrict__ bias1) {
  __shared__ float As[GK][GM + 4];
  __shared__ float Bs[GK][GN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int idx = tid + r * 256;
      int m, k;
      if (sak == 1) { k = idx % GK; m = idx / GK; } else { m = idx % GM; k = idx / GM; }
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? Elem<TA>::to_f(A[gm * sam + gk * sak]) : 0.f;
      int n, kb;
      if (sbk == 1) { kb = idx % GK; n = idx / GK; } else { n = idx % GN; kb = idx / GN; }
      const int gn = n0 + n, gkb = k0 + kb;
      Bs[kb][n] = (gn < N && gkb < K) ? Elem<TB>::to_f(B[gkb * sbk + gn * sbn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias0) v += Elem<TBias>::to_f(bias0[gn]);
      if (bias1) v += Elem<TBias>::to_f(bias1[gn]);
      C[gm * ldc + gn] = Elem<TC>::from_f(v);
    }
  }
}

template <typename TA, typename TB, typename TC, typename TBias>
static int launch_gemm(int M, int N, int K, const void* A, long long sam, long long sak,
                       const void* B, long long sbk, long long sbn, void* C, long long ldc,
                       const void* bias0, const void* bias1, cudaStream_t st) {
  dim3 grid(cdiv(N, GN), cdiv(M, GM));
  gemm_generic_kernel<TA, TB, TC, TBias><<<grid, 256, 0, st>>>(
      M, N, K, (const TA*)A, sam, sak, (const TB*)B, sbk, sbn, (TC*)C, ldc, (const TBias*)bias0,
      (const TBias*)bias1);
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return BLSTM_OK;
}

int generic_gemm(int dtype, bool out_f32, int M, int N, int K, const void* A, long long sam,
                 long long sak, const void* B, long long sbk, long long sbn, void* C, long long ldc,
                 const void* bias0, const void* bias1, cudaStream_t st) {
  if (M <= 0 || N <= 0) return BLSTM_OK;
  switch (dtype) {
    case BLSTM_F32:
      return launch_gemm<float, float, float, float>(M, N, K, A, sam, sak, B, sbk, sbn, C, ldc, bias0, bias1, st);
    case BLSTM_F16:
      return out_f32 ? launch_gemm<__half, __half, float, __half>(M, N, K, A, sam, sak, B, sbk, sbn, C, ldc, bias0, bias1, st)
                     : launch_gemm<__half, __half, __half, __half>(M, N, K, A, sam, sak, B, sbk, sbn, C, ldc, bias0, bias1, st);
    case BLSTM_BF16:
      return out_f32 ? launch_gemm<__nv_bfloat16, __nv_bfloat16, float, __nv_bfloat16>(M, N, K, A, sam, sak, B, sbk, sbn, C, ldc, bias0, bias1, st)
                     : launch_gemm<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(M, N, K, A, sam, sak, B, sbk, sbn, C, ldc, bias0, bias1, st);
  }
  return BLSTM_E_INVALID_ARG;
}

// ---------------------------------------------------------------------------
// Recurrence kernels
// ---------------------------------------------------------------------------
constexpr int BT = GenericPlan::kBT;   // batch rows per CTA
constexpr int UH = GenericPlan::kUH;   // hidden units per CTA
constexpr int KC = GenericPlan::kKC;   // K chunk staged in shared memory
constexpr int NT = BT * UH;            // threads

struct GenParams {
  int T, B, H;
  int nbt, nh, nb_par;
  int w_in_smem;
  int no_arrive;  // test hook: skip the arrival so waits run out
  int inference;  // forward only: skip the stores that only backward needs
  unsigned long long limit_ns;
  Control* ctl;
  int* flags;
  float* db_part;  // bwd only: [nbt][4H]
};

template <typename T>
__global__ void __launch_bounds__(NT)
gen_fwd_kernel(GenParams p, T* __restrict__ ifgo, const T* __restrict__ Wh, T* __restrict__ out,
               T* __restrict__ cell) {
  extern __shared__ float smem[];
  __shared__ int s_alive;
  const int H = p.H, B = p.B, Tn = p.T;
  const int Hp = H | 1;
  float* h_s = smem;                    // [BT][KC+1]
  float* w_s = smem + BT * (KC + 1);    // [4*UH][Hp]   (only when p.w_in_smem)
  const int tid = threadIdx.x;
  const int u = tid % UH, b = tid / UH;
  const int ph = blockIdx.x % p.nh, pb0 = blockIdx.x / p.nh;
  const int unit = ph * UH + u;
  const bool unit_ok = unit < H;
  const size_t H4 = 4 * (size_t)H;

  if (p.w_in_smem) {
    for (int idx = tid; idx < 4 * UH * H; idx += NT) {
      const int r = idx / H, k = idx % H;
      const int g = r / UH, uu = ph * UH + (r % UH);
      w_s[r * Hp + k] = (uu < H) ? ld_f(&Wh[((size_t)g * H + uu) * H + k]) : 0.f;
    }
  }
  if (tid == 0) s_alive = 1;
  __syncthreads();

  for (int bt = pb0; bt < p.nbt; bt += p.nb_par) {
    const int brow = bt * BT + b;
    const bool ok = unit_ok && brow < B;
    float c = ok ? ld_f(&cell[(size_t)brow * H + unit]) : 0.f;
    for (int t = 0; t < Tn; ++t) {
      float a[4] = {0.f, 0.f, 0.f, 0.f};
      const size_t grow = ((size_t)t * B + brow) * H4 + unit;
      if (ok) {
#pragma unroll
        for (int g = 0; g < 4; ++g) a[g] = ld_f(&ifgo[grow + (size_t)g * H]);
      }
      if (t > 0) {  // h[t] of this batch tile must be complete (all nh hidden tiles arrived)
        if (tid == 0 && !wait_flag_ge(&p.flags[(size_t)t * p.nbt + bt], p.nh, p.ctl, p.limit_ns, t, bt))
          s_alive = 0;
        __syncthreads();
        if (!s_alive) return;
      }
      for (int k0 = 0; k0 < H; k0 += KC) {
        const int kc = min(KC, H - k0);
        for (int idx = tid; idx < BT * kc; idx += NT) {
          const int bb = idx / kc, k = idx % kc;
          const int row = bt * BT + bb;
          h_s[bb * (KC + 1) + k] =
              (row < B) ? ld_cg_f(&out[((size_t)t * B + row) * H + k0 + k]) : 0.f;
        }
        __syncthreads();
        if (unit_ok) {
          const float* hb = h_s + b * (KC + 1);
          if (p.w_in_smem) {
            const float* w0 = w_s + (0 * UH + u) * Hp + k0;
            const float* w1 = w_s + (1 * UH + u) * Hp + k0;
            const float* w2 = w_s + (2 * UH + u) * Hp + k0;
            const float* w3 = w_s + (3 * UH + u) * Hp + k0;
            for (int k = 0; k < kc; ++k) {
              const float hk = hb[k];
              a[0] = fmaf(hk, w0[k], a[0]);
              a[1] = fmaf(hk, w1[k], a[1]);
              a[2] = fmaf(hk, w2[k], a[2]);
              a[3] = fmaf(hk, w3[k], a[3]);
            }
          } else {
            const T* w0 = Wh + ((size_t)0 * H + unit) * H + k0;
            const T* w1 = Wh + ((size_t)1 * H + unit) * H + k0;
            const T* w2 = Wh + ((size_t)2 * H + unit) * H + k0;
            const T* w3 = Wh + ((size_t)3 * H + unit) * H + k0;
            for (int k = 0; k < kc; ++k) {
              const float hk = hb[k];
              a[0] = fmaf(hk, ld_f(w0 + k), a[0]);
              a[1] = fmaf(hk, ld_f(w1 + k), a[1]);
              a[2] = fmaf(hk, ld_f(w2 + k), a[2]);
              a[3] = fmaf(hk, ld_f(w3 + k), a[3]);
            }
          }
        }
        __syncthreads();
      }
      if (ok) {
        if (!p.inference) {
#pragma unroll
          for (int g = 0; g < 4; ++g) ifgo[grow + (size_t)g * H] = Elem<T>::from_f(a[g]);
        }
        c = sigmoid_acc(a[1]) * c + sigmoid_acc(a[0]) * tanh_acc(a[2]);
        const float h = sigmoid_acc(a[3]) * tanh_acc(c);
        const size_t o1 = ((size_t)(t + 1) * B + brow) * H + unit;
        if (!p.inference || t == Tn - 1) cell[o1] = Elem<T>::from_f(c);
        out[o1] = Elem<T>::from_f(h);
      }
      __syncthreads();  // every store of this CTA for step t is issued
      if (tid == 0 && !p.no_arrive) {
        __threadfence();
        red_release_gpu_add(&p.flags[(size_t)(t + 1) * p.nbt + bt], 1);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
gen_bwd_kernel(GenParams p, const T* __restrict__ dout, const T* __restrict__ dh_n,
               const T* __restrict__ dc_n, const T* __restrict__ ifgo, const T* __restrict__ cell,
               const T* __restrict__ Wh, T* __restrict__ d_ifgo, T* __restrict__ dh0,
               T* __restrict__ dc0) {
  extern __shared__ float smem[];
  __shared__ int s_alive;
  const int H = p.H, B = p.B, Tn = p.T;
  float* dg_s = smem;                    // [BT][KC+1]
  float* w_s = smem + BT * (KC + 1);     // [4H][UH]   (only when p.w_in_smem)
  const int tid = threadIdx.x;
  const int u = tid % UH, b = tid / UH;
  const int ph = blockIdx.x % p.nh, pb0 = blockIdx.x / p.nh;
  const int unit = ph * UH + u;
  const bool unit_ok = unit < H;
  const int K4 = 4 * H;
  const size_t H4 = 4 * (size_t)H;

  if (p.w_in_smem) {
    for (int idx = tid; idx < K4 * UH; idx += NT) {
      const int k = idx / UH, uu = ph * UH + (idx % UH);
      w_s[idx] = (uu < H) ? ld_f(&Wh[(size_t)k * H + uu]) : 0.f;
    }
  }
  if (tid == 0) s_alive = 1;
  __syncthreads();

  for (int bt = pb0; bt < p.nbt; bt += p.nb_par) {
    const int brow = bt * BT + b;
    const bool ok = unit_ok && brow < B;
    float dh_carry = (ok && dh_n) ? ld_f(&dh_n[(size_t)brow * H + unit]) : 0.f;
    float dc = (ok && dc_n) ? ld_f(&dc_n[(size_t)brow * H + unit]) : 0.f;
    float dbacc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = Tn - 1; t >= 0; --t) {
      const int step = Tn - 1 - t;
      if (ok) {
        const size_t grow = ((size_t)t * B + brow) * H4 + unit;
        const float pi = ld_f(&ifgo[grow]), pf = ld_f(&ifgo[grow + H]);
        const float pg = ld_f(&ifgo[grow + 2 * (size_t)H]), po = ld_f(&ifgo[grow + 3 * (size_t)H]);
        const float c0 = ld_f(&cell[((size_t)t * B + brow) * H + unit]);
        const float c1 = ld_f(&cell[((size_t)(t + 1) * B + brow) * H + unit]);
        const float dh = ld_f(&dout[((size_t)t * B + brow) * H + unit]) + dh_carry;
        const float si = sigmoid_acc(pi), sf = sigmoid_acc(pf), so = sigmoid_acc(po);
        const float tg = tanh_acc(pg), tc = tanh_acc(c1);
        dc = fmaf(dh * so, 1.f - tc * tc, dc);
        const T qi = Elem<T>::from_f(dc * tg * si * (1.f - si));
        const T qf = Elem<T>::from_f(dc * c0 * sf * (1.f - sf));
        const T qg = Elem<T>::from_f(dc * si * (1.f - tg * tg));
        const T qo = Elem<T>::from_f(dh * tc * so * (1.f - so));
        d_ifgo[grow] = qi;
        d_ifgo[grow + H] = qf;
        d_ifgo[grow + 2 * (size_t)H] = qg;
        d_ifgo[grow + 3 * (size_t)H] = qo;
        dbacc[0] += Elem<T>::to_f(qi);
        dbacc[1] += Elem<T>::to_f(qf);
        dbacc[2] += Elem<T>::to_f(qg);
        dbacc[3] += Elem<T>::to_f(qo);
        dc *= sf;
      }
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        int* f = &p.flags[(size_t)step * p.nbt + bt];
        if (!p.no_arrive) red_release_gpu_add(f, 1);
        if (!wait_flag_ge(f, p.nh, p.ctl, p.limit_ns, t, bt)) s_alive = 0;
      }
      __syncthreads();
      if (!s_alive) return;
      // dh_{t-1}[b, unit] = sum_k d_ifgo[t][b, k] * Wh[k, unit]
      float acc = 0.f;
      for (int k0 = 0; k0 < K4; k0 += KC) {
        const int kc = min(KC, K4 - k0);
        for (int idx = tid; idx < BT * kc; idx += NT) {
          const int bb = idx / kc, k = idx % kc;
          const int row = bt * BT + bb;
          dg_s[bb * (KC + 1) + k] =
              (row < B) ? ld_cg_f(&d_ifgo[((size_t)t * B + row) * H4 + k0 + k]) : 0.f;
        }
        __syncthreads();
        if (unit_ok) {
          const float* db_ = dg_s + b * (KC + 1);
          if (p.w_in_smem) {
            const float* w = w_s + (size_t)k0 * UH + u;
            for (int k = 0; k < kc; ++k) acc = fmaf(db_[k], w[k * UH], acc);
          } else {
            const T* w = Wh + (size_t)k0 * H + unit;
            for (int k = 0; k < kc; ++k) acc = fmaf(db_[k], ld_f(w + (size_t)k * H), acc);
          }
        }
        __syncthreads();
      }
      dh_carry = acc;
    }
    if (ok) {
      dh0[(size_t)brow * H + unit] = Elem<T>::from_f(dh_carry);
      dc0[(size_t)brow * H + unit] = Elem<T>::from_f(dc);
    }
    // bias-gradient partial of this batch tile: sum over the CTA's batch rows
    float* red = dg_s;  // [BT][4*UH]
    __syncthreads();
#pragma unroll
    for (int g = 0; g < 4; ++g) red[b * (4 * UH) + g * UH + u] = ok ? dbacc[g] : 0.f;
    __syncthreads();
    if (tid < 4 * UH) {
      float s = 0.f;
      for (int bb = 0; bb < BT; ++bb) s += red[bb * (4 * UH) + tid];
      const int g = tid / UH, uu = ph * UH + (tid % UH);
      if (uu < H) p.db_part[(size_t)bt * H4 + (size_t)g * H + uu] = s;
    }
    __syncthreads();
  }
}

__global__ void reduce_db_kernel(const float* __restrict__ part, int n_part, int n, float* __restrict__ db) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float s = 0.f;
  for (int i = 0; i < n_part; ++i) s += part[(size_t)i * n + j];
  db[j] = s;
}

int reduce_db(const float* part, int n_part, int n, float* db, cudaStream_t st) {
  reduce_db_kernel<<<cdiv(n, 256), 256, 0, st>>>(part, n_part, n, db);
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return BLSTM_OK;
}

// ---------------------------------------------------------------------------
// Planning and launch
// ---------------------------------------------------------------------------
void GenericPlan::make(const blstm_desc& d, int phase) {
  T = d.seq_len; B = d.batch; H = d.hidden_size;
  nbt = cdiv(B, kBT);
  nh = cdiv(H, kUH);
  const size_t stage = (size_t)kBT * (kKC + 1) * sizeof(float);
  const size_t wbytes = (phase == BLSTM_PHASE_FWD) ? (size_t)4 * kUH * (H | 1) * sizeof(float)
                                                   : (size_t)4 * H * kUH * sizeof(float);
  w_in_smem = wbytes <= 64 * 1024;
  smem_bytes = stage + (w_in_smem ? wbytes : 0);
  n_flags = (size_t)(T + 1) * nbt;
  off_flags = sizeof(Control);
  off_db = off_flags + round_up(n_flags * sizeof(int), 256);
  ws_bytes = off_db + (phase == BLSTM_PHASE_BWD ? round_up((size_t)nbt * 4 * H * sizeof(float), 256) : 0);
}

template <typename Kern>
static int coresident_grid(Kern kern, GenericPlan& pl) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc) return rc;
  if (!di.coop) return BLSTM_E_NOT_CORESIDENT;
  BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes));
  int per_sm = 0;
  BLSTM_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, pl.smem_bytes));
  const int cap = per_sm * di.sm_count;
  if (cap < pl.nh) return BLSTM_E_NOT_CORESIDENT;
  pl.nb_par = cap / pl.nh;
  if (pl.nb_par > pl.nbt) pl.nb_par = pl.nbt;
  pl.grid = pl.nb_par * pl.nh;
  return BLSTM_OK;
}

static GenParams make_params(const blstm_desc& d, const GenericPlan& pl, void* ws) {
  GenParams p;
  p.T = pl.T; p.B = pl.B; p.H = pl.H;
  p.nbt = pl.nbt; p.nh = pl.nh; p.nb_par = pl.nb_par;
  p.w_in_smem = pl.w_in_smem ? 1 : 0;
  p.no_arrive = (d.flags & BLSTM_FLAG_TEST_NO_ARRIVE) ? 1 : 0;
  p.inference = (d.flags & BLSTM_FLAG_INFERENCE) ? 1 : 0;
  p.limit_ns = d.wait_limit_us > 0 ? (unsigned long long)d.wait_limit_us * 1000ull : kDefaultWaitNs;
  p.ctl = reinterpret_cast<Control*>(ws);
  p.flags = reinterpret_cast<int*>(static_cast<char*>(ws) + pl.off_flags);
  p.db_part = reinterpret_cast<float*>(static_cast<char*>(ws) + pl.off_db);
  return p;
}

template <typename T>
static int launch_fwd(const blstm_desc& d, GenericPlan& pl, void* ifgo, const void* Wh, void* out,
                      void* cell, void* ws, cudaStream_t st) {
  int rc = coresident_grid(gen_fwd_kernel<T>, pl);
  if (rc) return rc;
  GenParams p = make_params(d, pl, ws);
  T* a0 = (T*)ifgo; const T* a1 = (const T*)Wh; T* a2 = (T*)out; T* a3 = (T*)cell;
  void* args[] = {&p, &a0, &a1, &a2, &a3};
  BLSTM_CUDA_OK(cudaLaunchCooperativeKernel((void*)gen_fwd_kernel<T>, dim3(pl.grid), dim3(NT), args,
                                            pl.smem_bytes, st));
  count_launch();
  return BLSTM_OK;
}

int generic_fwd_recurrence(const blstm_desc& d, void* ifgo, const void* Wh, void* out, void* cell,
                           void* ws, size_t ws_bytes, cudaStream_t st) {
  GenericPlan pl;
  pl.make(d, BLSTM_PHASE_FWD);
  if (ws_bytes < pl.ws_bytes) return BLSTM_E_WORKSPACE;
  BLSTM_CUDA_OK(cudaMemsetAsync(ws, 0, pl.off_db, st));
  switch (d.dtype) {
    case BLSTM_F32: return launch_fwd<float>(d, pl, ifgo, Wh, out, cell, ws, st);
    case BLSTM_F16: return launch_fwd<__half>(d, pl, ifgo, Wh, out, cell, ws, st);
    case BLSTM_BF16: return launch_fwd<__nv_bfloat16>(d, pl, ifgo, Wh, out, cell, ws, st);
  }
  return BLSTM_E_INVALID_ARG;
}

template <typename T>
static int launch_bwd(const blstm_desc& d, GenericPlan& pl, const void* dout, const void* dh_n,
                      const void* dc_n, const void* ifgo, const void* cell, const void* Wh,
                      void* d_ifgo, void* dh0, void* dc0, void* ws, cudaStream_t st) {
  int rc = coresident_grid(gen_bwd_kernel<T>, pl);
  if (rc) return rc;
  GenParams p = make_params(d, pl, ws);
  const T* a0 = (const T*)dout; const T* a1 = (const T*)dh_n; const T* a2 = (const T*)dc_n;
  const T* a3 = (const T*)ifgo; const T* a4 = (const T*)cell; const T* a5 = (const T*)Wh;
  T* a6 = (T*)d_ifgo; T* a7 = (T*)dh0; T* a8 = (T*)dc0;
  void* args[] = {&p, &a0, &a1, &a2, &a3, &a4, &a5, &a6, &a7, &a8};
  BLSTM_CUDA_OK(cudaLaunchCooperativeKernel((void*)gen_bwd_kernel<T>, dim3(pl.grid), dim3(NT), args,
                                            pl.smem_bytes, st));
  count_launch();
  return BLSTM_OK;
}

int generic_bwd_recurrence(const blstm_desc& d, const void* dout, const void* dh_n, const void* dc_n,
                           const void* ifgo, const void* cell, const void* Wh, void* d_ifgo,
                           void* dh0, void* dc0, float* db, void* ws, size_t ws_bytes,
                           cudaStream_t st) {
  GenericPlan pl;
  pl.make(d, BLSTM_PHASE_BWD);
  if (ws_bytes < pl.ws_bytes) return BLSTM_E_WORKSPACE;
  BLSTM_CUDA_OK(cudaMemsetAsync(ws, 0, pl.off_db, st));
  int rc = BLSTM_E_INVALID_ARG;
  switch (d.dtype) {
    case BLSTM_F32: rc = launch_bwd<float>(d, pl, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, ws, st); break;
    case BLSTM_F16: rc = launch_bwd<__half>(d, pl, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, ws, st); break;
    case BLSTM_BF16: rc = launch_bwd<__nv_bfloat16>(d, pl, dout, dh_n, dc_n, ifgo, cell, Wh, d_ifgo, dh0, dc0, ws, st); break;
  }
  if (rc) return rc;
  if (db) {
    const float* part = reinterpret_cast<const float*>(static_cast<char*>(ws) + pl.off_db);
    return reduce_db(part, pl.nbt, 4 * d.hidden_size, db, st);
  }
  return BLSTM_OK;
}

// ---------------------------------------------------------------------------
// Tiny hidden sizes: the whole forward operator in ONE kernel (replaces
// fully_fused_persistent_fwd_kernel, fastlstm/kernels.py:672-819, dispatch fastlstm/lstm.py:40-47).
// With max(H, I) <= 32 (fp32) or <= 64 (16-bit) the input projection is as memory-bound as the
// recurrence, so it is computed inside the time loop and the projected pre-activations never make a
// round trip through memory.  A CTA owns FB batch rows and ALL 4H gate columns, so no CTA ever waits
// for another: a plain launch, any batch size.  Thread n keeps row n of [Wx | Wh] (its gate column's
// weights) in registers; per step the CTA stages [x_t | h_t] of its rows in shared memory, every
// thread forms its column's pre-activation for the FB rows, and thread (row, unit) applies the gates
// with c carried in a register.
// ---------------------------------------------------------------------------
constexpr int FB = 4;                   // batch rows per CTA

template <typename T, int KMAX>         // KMAX >= I + H
__global__ void __launch_bounds__(256)
fused_fwd_kernel(int Tn, int B, int I, int H, int inference, const T* __restrict__ x, const T* __restrict__ Wx,
                 const T* __restrict__ Wh, const T* __restrict__ bx, const T* __restrict__ bh,
                 T* __restrict__ ifgo, T* __restrict__ out, T* __restrict__ cell) {
  __shared__ __align__(16) float xh[FB][KMAX];          // [x_t | h_t] of the CTA's rows
  __shared__ float pre[FB][256];                        // pre-activations, gate-major like ifgo
  const int n = threadIdx.x, G = 4 * H, K = I + H;
  const int row0 = blockIdx.x * FB;
  float w[KMAX];
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    float v = 0.f;
    if (n < G) {
      if (k < I) v = ld_f(Wx + (size_t)n * I + k);
      else if (k < K) v = ld_f(Wh + (size_t)n * H + (k - I));
    }
    w[k] = v;
  }
  // the bias as the unfused path forms it: bx + bh rounded to the storage type
  float bias = 0.f;
  if (n < G) bias = Elem<T>::to_f(Elem<T>::from_f((bx ? ld_f(bx + n) : 0.f) + (bh ? ld_f(bh + n) : 0.f)));
  for (int i = n; i < FB * KMAX; i += blockDim.x) (&xh[0][0])[i] = 0.f;   // columns past K stay zero
  __syncthreads();
  // thread (rb, u) of the first FB*H threads owns one cell state
  const int rb = n / H, u = n % H;
  const bool owner = n < FB * H && row0 + rb < B;
  float c = 0.f;
  if (owner) {
    c = ld_f(cell + (size_t)(row0 + rb) * H + u);
    xh[rb][I + u] = ld_f(out + (size_t)(row0 + rb) * H + u);
  } else if (n < FB * H) {
    xh[rb][I + u] = 0.f;
  }
  for (int t = 0; t < Tn; ++t) {
    for (int i = n; i < FB * I; i += blockDim.x) {
      const int b = i / I, k = i % I;
      xh[b][k] = (row0 + b < B) ? ld_f(x + ((size_t)t * B + row0 + b) * I + k) : 0.f;
    }
    __syncthreads();
    float acc[FB];
#pragma unroll
    for (int b = 0; b < FB; ++b) acc[b] = bias;
#pragma unroll
    for (int k = 0; k < KMAX; k += 4) {
      if (k < K) {
#pragma unroll
        for (int b = 0; b < FB; ++b) {
          const float4 v = *reinterpret_cast<const float4*>(&xh[b][k]);
          acc[b] = fmaf(w[k], v.x, acc[b]);
          acc[b] = fmaf(w[k + 1], v.y, acc[b]);
          acc[b] = fmaf(w[k + 2], v.z, acc[b]);
          acc[b] = fmaf(w[k + 3], v.w, acc[b]);
        }
      }
    }
    if (n < G) {
#pragma unroll
      for (int b = 0; b < FB; ++b) {
        pre[b][n] = acc[b];
        if (!inference && row0 + b < B) ifgo[((size_t)t * B + row0 + b) * G + n] = Elem<T>::from_f(acc[b]);
      }
    }
    __syncthreads();
    if (owner) {
      const float pi = pre[rb][u], pf = pre[rb][H + u], pg = pre[rb][2 * H + u], po = pre[rb][3 * H + u];
      c = sigmoid_acc(pf) * c + sigmoid_acc(pi) * tanh_acc(pg);
      const T h = Elem<T>::from_f(sigmoid_acc(po) * tanh_acc(c));
      const size_t o1 = ((size_t)(t + 1) * B + row0 + rb) * H + u;
      out[o1] = h;
      if (!inference || t == Tn - 1) cell[o1] = Elem<T>::from_f(c);
      xh[rb][I + u] = Elem<T>::to_f(h);                  // fed back at storage precision
    }
    // (the barrier at the top of the next step orders these writes before the next reads, and the x
    //  columns written before it were last read before the barrier above)
  }
}

bool generic_fused_fwd_supported(const blstm_desc& d) {
  if (d.flags & BLSTM_FLAG_NO_FUSED) return false;
  const int size = d.hidden_size > d.input_size ? d.hidden_size : d.input_size;
  return size <= (d.dtype == BLSTM_F32 ? 32 : 64);
}

template <typename T>
static int launch_fused(const blstm_desc& d, const void* x, const void* Wx, const void* Wh, const void* bx,
                        const void* bh, void* ifgo, void* out, void* cell, cudaStream_t st) {
  const int H = d.hidden_size, I = d.input_size;
  const int threads = (int)round_up((size_t)(4 * H > FB * H ? 4 * H : FB * H), 32);
  const int grid = cdiv(d.batch, FB);
  const int inf = (d.flags & BLSTM_FLAG_INFERENCE) ? 1 : 0;
  if (I + H <= 64)
    fused_fwd_kernel<T, 64><<<grid, threads, 0, st>>>(d.seq_len, d.batch, I, H, inf, (const T*)x, (const T*)Wx, (const T*)Wh,
                                                      (const T*)bx, (const T*)bh, (T*)ifgo, (T*)out, (T*)cell);
  else
    fused_fwd_kernel<T, 128><<<grid, threads, 0, st>>>(d.seq_len, d.batch, I, H, inf, (const T*)x, (const T*)Wx, (const T*)Wh,
                                                       (const T*)bx, (const T*)bh, (T*)ifgo, (T*)out, (T*)cell);
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return BLSTM_OK;
}

int generic_fused_fwd(const blstm_desc& d, const void* x, const void* Wx, const void* Wh, const void* bx,
                      const void* bh, void* ifgo, void* out, void* cell, cudaStream_t st) {
  switch (d.dtype) {
    case BLSTM_F32: return launch_fused<float>(d, x, Wx, Wh, bx, bh, ifgo, out, cell, st);
    case BLSTM_F16: return launch_fused<__half>(d, x, Wx, Wh, bx, bh, ifgo, out, cell, st);
    case BLSTM_BF16: return launch_fused<__nv_bfloat16>(d, x, Wx, Wh, bx, bh, ifgo, out, cell, st);
  }
  return BLSTM_E_INVALID_ARG;
}

// Column sums of d_ifgo [rows, cols]: part p adds the rows congruent to p modulo n_part, then
// reduce_db adds the parts in a fixed order (deterministic).
template <typename T>
__global__ void gen_colsum_kernel(const T* __restrict__ g, int rows, int cols, int n_part, float* __restrict__ part) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float s = 0.f;
  for (int r = blockIdx.y; r < rows; r += n_part) s += ld_f(g + (size_t)r * cols + col);
  part[(size_t)blockIdx.y * cols + col] = s;
}

int generic_bias_grad(const blstm_desc& d, const void* d_ifgo, float* db, void* ws, size_t ws_bytes,
                      cudaStream_t st) {
  GenericPlan pl;
  pl.make(d, BLSTM_PHASE_BWD);
  if (ws_bytes < pl.ws_bytes) return BLSTM_E_WORKSPACE;
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + pl.off_db);
  const int rows = d.seq_len * d.batch, cols = 4 * d.hidden_size;
  dim3 grid(cdiv(cols, 128), pl.nbt);
  switch (d.dtype) {
    case BLSTM_F32: gen_colsum_kernel<float><<<grid, 128, 0, st>>>((const float*)d_ifgo, rows, cols, pl.nbt, part); break;
    case BLSTM_F16: gen_colsum_kernel<__half><<<grid, 128, 0, st>>>((const __half*)d_ifgo, rows, cols, pl.nbt, part); break;
    case BLSTM_BF16: gen_colsum_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)d_ifgo, rows, cols, pl.nbt, part); break;
    default: return BLSTM_E_INVALID_ARG;
  }
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return reduce_db(part, pl.nbt, cols, db, st);
}

}  // namespace blstm
