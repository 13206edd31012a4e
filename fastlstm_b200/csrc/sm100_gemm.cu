// tcgen05/TMEM + TMA GEMM for the dense contractions of the LSTM layer
// (16-bit operands, fp32 accumulation in tensor memory):
//
//   input projection  ifgo = x * Wx^T + (bx+bh)     A K-major,  B K-major,  16-bit out
//   input gradient    dx   = d_ifgo * Wx            A K-major,  B N-major,  16-bit out
//   weight gradients  dW   = d_ifgo^T * [x | h]     A M-major,  B N-major,  fp32 out, split-K
//
// They replace the cuBLAS calls of the reference (fastlstm/lstm.py:66-68, :294,
// :494-501); the M/N-major operand forms remove the reference's transpose copy
// of d_ifgo (lstm.py:495).
//
// One persistent CTA per SM walks 128x256 output tiles.  Warp 0 feeds a 4-stage
// shared-memory ring with TMA tile loads, warp 1 issues tcgen05.mma into one of
// two 256-column TMEM accumulators, warps 2-5 drain the other accumulator
// (tcgen05.ld -> registers -> bias/convert -> global), so the epilogue of tile
// i overlaps the main loop of tile i+1.  No TMA multicast is used.
#include <stdlib.h>

#include "sm100.cuh"
#include "sm100_common.cuh"

namespace blstm {
namespace sm100 {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int STG_BYTES = 4096;        // one epilogue staging box: 32 rows x 128 B
constexpr int STG_TOTAL = 4 * 2 * STG_BYTES;   // 4 epilogue warps, double-buffered
constexpr size_t GEMM_SMEM = 1024 /*align slack*/ + (size_t)STAGES * STAGE_BYTES + STG_TOTAL + 128 + BN * 4;
static_assert(GEMM_SMEM <= 232448, "exceeds the 227 KB shared-memory limit per CTA");

struct GemmParams {
  int M, N, K;
  int m_tiles, n_tiles, splits;
  int kb_total, kb_per_split;
  int fmt;                 // 0 f16, 1 bf16
  void* out;               // 16-bit [M,ldc] or fp32 [splits][M,ldc]
  long long ldc;
  const void* bias0;       // 16-bit [N] or null
  const void* bias1;
  Control* ctl;            // may be null
  unsigned long long limit_ns;
};

template <typename T16>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T16> __device__ __forceinline__ float2 unpack2(uint32_t v);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}

// A_MN / B_MN: operand is M/N-major in global memory (and therefore in shared memory).
// OUT_F32: fp32 output (weight gradients), else 16-bit output with optional bias.
template <int A_MN, int B_MN, bool OUT_F32, typename T16>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + (size_t)STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + STG_TOTAL);
  uint64_t* full = bars;                   // [STAGES]
  uint64_t* empty = bars + STAGES;         // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  T16* bias_s = reinterpret_cast<T16*>(reinterpret_cast<uint8_t*>(bars) + 128);   // [2][BN], 128 B past the barriers

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    *dead = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.m_tiles * p.n_tiles * p.splits;
  WaitCtx wc{dead, p.ctl, p.limit_ns, -1, (int)blockIdx.x};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // A thread needs ~150-300 clocks per cp.async.bulk.tensor issue, and the M/N-major operand forms
    // need one box per 64-element chunk (up to six boxes per k-block, more than the k-block's MMAs
    // take), so every box has its own lane: the lanes walk the stages in lockstep, lane 0 arms the
    // stage's barrier, each lane issues one load.
    constexpr int NA = A_MN ? 2 : 1, NB = B_MN ? 4 : 1;
    if (lane < NA + NB) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int nt = tile % p.n_tiles, mt = (tile / p.n_tiles) % p.m_tiles, z = tile / (p.n_tiles * p.m_tiles);
        const int m0 = mt * BM, n0 = nt * BN;
        const int kb0 = z * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, wc)) { ok = false; break; }
          uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (lane == 0) mbar_expect_tx(&full[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (lane < NA) {
            if (A_MN) tma_load_2d(sa + lane * 8192, &tmA, &full[s], m0 + 64 * lane, k0);
            else      tma_load_2d(sa, &tmA, &full[s], k0, m0);
          } else {
            const int j = lane - NA;
            if (B_MN) tma_load_2d(sb + j * 8192, &tmB, &full[s], n0 + 64 * j, k0);
            else      tma_load_2d(sb, &tmB, &full[s], k0, n0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint64_t descA = A_MN ? smem_desc_base(8192, 1024) : smem_desc_base(16, 1024);
      constexpr uint64_t descB = B_MN ? smem_desc_base(8192, 1024) : smem_desc_base(16, 1024);
      constexpr uint32_t stepA = A_MN ? 2048 : 32, stepB = B_MN ? 2048 : 32;  // bytes per K=16
      const uint32_t idesc = instr_desc(p.fmt, A_MN, B_MN, BM, BN);
      int s = 0;
      uint32_t ph = 0;
      uint32_t acc_ph[2] = {0, 0};
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
        const int z = tile / (p.n_tiles * p.m_tiles);
        const int kb0 = z * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
        const int a = it & 1;
        if (!mbar_wait(&acc_empty[a], acc_ph[a] ^ 1, wc)) { ok = false; break; }
        acc_ph[a] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, wc)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16(d_tmem, smem_desc(descA, sa + k * stepA), smem_desc(descB, sb + k * stepB), idesc,
                     (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);   // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&acc_full[a]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                  // TMEM lane quarter this warp may access
    uint32_t acc_ph[2] = {0, 0};
    uint32_t stg_toggle = 0;
    const bool has_bias = !OUT_F32 && (p.bias0 != nullptr || p.bias1 != nullptr);
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
      const int nt = tile % p.n_tiles, mt = (tile / p.n_tiles) % p.m_tiles, z = tile / (p.n_tiles * p.m_tiles);
      const int m0 = mt * BM, n0 = nt * BN;
      const int a = it & 1;
      if (!mbar_wait(&acc_full[a], acc_ph[a], wc)) { ok = false; break; }
      acc_ph[a] ^= 1;
      tc_fence_after();
      if (has_bias) {
        // bx + bh for this tile's 256 columns, rounded to the storage type (as the reference forms
        // its bias, fastlstm/lstm.py:67) and zero past N.  EVERY epilogue warp writes the whole
        // (identical) table into the buffer of this tile's parity and then only needs a warp-level
        // sync: no cross-warp barrier can strand a warp.  Warps are never more than one tile apart
        // (a TMEM buffer is re-issued only after all four released it), so two buffers suffice.
        T16* bdst = bias_s + (it & 1) * BN;
        const int cc = n0 + lane * 8;
        uint32_t w[4] = {0, 0, 0, 0};
        if (cc < p.N) {
          uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
          if (p.bias0) v0 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T16*>(p.bias0) + cc);
          if (p.bias1) v1 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T16*>(p.bias1) + cc);
          const uint32_t a0[4] = {v0.x, v0.y, v0.z, v0.w}, a1[4] = {v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f0 = unpack2<T16>(a0[j]), f1 = unpack2<T16>(a1[j]);
            w[j] = pack2<T16>(f0.x + f1.x, f0.y + f1.y);
          }
        }
        *reinterpret_cast<uint4*>(bdst + lane * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        __syncwarp();
      }
      const uint32_t taddr = tmem_base + a * BN + (uint32_t(q * 32) << 16);
      constexpr int CW = OUT_F32 ? 32 : 64;      // output columns per staged box (128 B per row)
      uint8_t* my_stage = staging + (warp - 2) * 2 * STG_BYTES;
#pragma unroll 1
      for (int c = 0; c < BN; c += CW) {
        const int col = n0 + c;
        if (col >= p.N) break;
        uint32_t v[32];
        if (OUT_F32) {
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
        } else {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c, r0);
          tmem_ld_32x32(taddr + c + 32, r1);
          tmem_ld_wait();
          if (has_bias) {
            const uint32_t* bs = reinterpret_cast<const uint32_t*>(bias_s + (it & 1) * BN + c);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float2 b0 = unpack2<T16>(bs[j]), b1 = unpack2<T16>(bs[16 + j]);
              v[j] = pack2<T16>(__uint_as_float(r0[2 * j]) + b0.x, __uint_as_float(r0[2 * j + 1]) + b0.y);
              v[16 + j] = pack2<T16>(__uint_as_float(r1[2 * j]) + b1.x, __uint_as_float(r1[2 * j + 1]) + b1.y);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] = pack2<T16>(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
              v[16 + j] = pack2<T16>(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
            }
          }
        }
        // stage the 32x128-byte box with the 128-byte swizzle the output tensor map expects,
        // then one lane hands it to TMA (rows/columns past M/N are clipped by the hardware)
        uint8_t* buf = my_stage + (stg_toggle & 1) * STG_BYTES;
        ++stg_toggle;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* rowp = buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmC, buf, col, m0 + q * 32, z);
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
    }
    if (lane == 0) tma_store_wait<0>();
  }
  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- CTA-pair variant
// The single-CTA kernel above needs (128 + 256) x 64 x 2 B = 48 KB of operands per k-block of 504 tensor
// clocks, 97 B/clk per SM - more than an SM takes in through TMA (about 70 B/clk), so it tops out near
// 70 % of the tensor peak.  Here two CTAs of a cluster share a 256x256 tile: each loads 128 rows of A and
// 128 columns of B per k-block (32 KB, 65 B/clk), one thread of the even CTA issues M=256 MMAs that read
// both CTAs' shared memory, and each CTA ends up with its 128 rows x 256 columns in its own tensor
// memory.  Six 32 KB stages per CTA.  Both producers count their bytes on the EVEN CTA's stage
// barrier; the issuer's commits arrive on both CTAs' barriers; the odd CTA's epilogue warps hand
// accumulators back with remote arrivals.  No multicast load.
constexpr int P_STAGES = 6;
constexpr int P_STAGE_BYTES = 2 * A_BYTES;                 // A 128x64 + B 128x64
constexpr size_t GEMM_P_SMEM = 1024 + (size_t)P_STAGES * P_STAGE_BYTES + STG_TOTAL + 256 + BN * 4;
static_assert(GEMM_P_SMEM <= 232448, "exceeds the 227 KB shared-memory limit per CTA");

template <int A_MN, int B_MN, bool OUT_F32, typename T16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + (size_t)P_STAGES * P_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + STG_TOTAL);
  uint64_t* full = bars;                     // [P_STAGES] (the even CTA's are used)
  uint64_t* empty = bars + P_STAGES;         // [P_STAGES]
  uint64_t* acc_full = bars + 2 * P_STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2] (the even CTA's are used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  T16* bias_s = reinterpret_cast<T16*>(reinterpret_cast<uint8_t*>(bars) + 256);   // [2][BN]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    *dead = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                        // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.m_tiles * p.n_tiles * p.splits;     // 256x256 tiles
  WaitCtx wc{dead, p.ctl, p.limit_ns, -1, (int)blockIdx.x};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    constexpr int NA = A_MN ? 2 : 1, NB = B_MN ? 2 : 1;
    if (lane < NA + NB) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += npairs) {
        const int nt = tile % p.n_tiles, mt = (tile / p.n_tiles) % p.m_tiles, z = tile / (p.n_tiles * p.m_tiles);
        const int m0 = mt * 256 + (int)rank * 128, n0 = nt * 256 + (int)rank * 128;
        const int kb0 = z * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, wc)) { ok = false; break; }
          uint8_t* sa = smem + (size_t)s * P_STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // the stage's bytes of BOTH CTAs are counted on the even CTA's barrier
          if (rank == 0 && lane == 0) mbar_expect_tx(&full[s], 2 * P_STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
          const int k0 = kb * BK;
          if (lane < NA) {
            if (A_MN) tma_load_2d_pair(sa + lane * 8192, &tmA, bar, m0 + 64 * lane, k0);
            else      tma_load_2d_pair(sa, &tmA, bar, k0, m0);
          } else {
            const int j = lane - NA;
            if (B_MN) tma_load_2d_pair(sb + j * 8192, &tmB, bar, n0 + 64 * j, k0);
            else      tma_load_2d_pair(sb, &tmB, bar, k0, n0);
          }
          if (++s == P_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint64_t descA = A_MN ? smem_desc_base(8192, 1024) : smem_desc_base(16, 1024);
      constexpr uint64_t descB = B_MN ? smem_desc_base(8192, 1024) : smem_desc_base(16, 1024);
      constexpr uint32_t stepA = A_MN ? 2048 : 32, stepB = B_MN ? 2048 : 32;  // bytes per K=16
      const uint32_t idesc = instr_desc(p.fmt, A_MN, B_MN, 256, BN);
      int s = 0;
      uint32_t ph = 0;
      uint32_t acc_ph[2] = {0, 0};
      bool ok = true;
      int it = 0;
      for (int tile = pair; tile < tiles && ok; tile += npairs, ++it) {
        const int z = tile / (p.n_tiles * p.m_tiles);
        const int kb0 = z * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
        const int a = it & 1;
        if (!mbar_wait_cluster(&acc_empty[a], acc_ph[a] ^ 1, wc)) { ok = false; break; }
        acc_ph[a] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, wc)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)s * P_STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16_pair(d_tmem, smem_desc(descA, sa + k * stepA), smem_desc(descB, sb + k * stepB), idesc,
                          (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // frees the stage in both CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&empty[s]));
          umma_commit_pair(mapa_shared(smem_u32(&empty[s]), 1));
          if (++s == P_STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) {
          umma_commit_pair(smem_u32(&acc_full[a]));
          umma_commit_pair(mapa_shared(smem_u32(&acc_full[a]), 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;                  // TMEM lane quarter this warp may access
    uint32_t acc_ph[2] = {0, 0};
    uint32_t stg_toggle = 0;
    const bool has_bias = !OUT_F32 && (p.bias0 != nullptr || p.bias1 != nullptr);
    bool ok = true;
    int it = 0;
    for (int tile = pair; tile < tiles && ok; tile += npairs, ++it) {
      const int nt = tile % p.n_tiles, mt = (tile / p.n_tiles) % p.m_tiles, z = tile / (p.n_tiles * p.m_tiles);
      const int m0 = mt * 256 + (int)rank * 128, n0 = nt * BN;
      const int a = it & 1;
      if (!mbar_wait(&acc_full[a], acc_ph[a], wc)) { ok = false; break; }
      acc_ph[a] ^= 1;
      tc_fence_after();
      if (has_bias) {
        T16* bdst = bias_s + (it & 1) * BN;
        const int cc = n0 + lane * 8;
        uint32_t w[4] = {0, 0, 0, 0};
        if (cc < p.N) {
          uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
          if (p.bias0) v0 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T16*>(p.bias0) + cc);
          if (p.bias1) v1 = *reinterpret_cast<const uint4*>(reinterpret_cast<const T16*>(p.bias1) + cc);
          const uint32_t a0[4] = {v0.x, v0.y, v0.z, v0.w}, a1[4] = {v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f0 = unpack2<T16>(a0[j]), f1 = unpack2<T16>(a1[j]);
            w[j] = pack2<T16>(f0.x + f1.x, f0.y + f1.y);
          }
        }
        *reinterpret_cast<uint4*>(bdst + lane * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        __syncwarp();
      }
      const uint32_t taddr = tmem_base + a * BN + (uint32_t(q * 32) << 16);
      constexpr int CW = OUT_F32 ? 32 : 64;      // output columns per staged box (128 B per row)
      uint8_t* my_stage = staging + (warp - 2) * 2 * STG_BYTES;
#pragma unroll 1
      for (int c = 0; c < BN; c += CW) {
        const int col = n0 + c;
        if (col >= p.N) break;
        uint32_t v[32];
        if (OUT_F32) {
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
        } else {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c, r0);
          tmem_ld_32x32(taddr + c + 32, r1);
          tmem_ld_wait();
          if (has_bias) {
            const uint32_t* bs = reinterpret_cast<const uint32_t*>(bias_s + (it & 1) * BN + c);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float2 b0 = unpack2<T16>(bs[j]), b1 = unpack2<T16>(bs[16 + j]);
              v[j] = pack2<T16>(__uint_as_float(r0[2 * j]) + b0.x, __uint_as_float(r0[2 * j + 1]) + b0.y);
              v[16 + j] = pack2<T16>(__uint_as_float(r1[2 * j]) + b1.x, __uint_as_float(r1[2 * j + 1]) + b1.y);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] = pack2<T16>(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
              v[16 + j] = pack2<T16>(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
            }
          }
        }
        uint8_t* buf = my_stage + (stg_toggle & 1) * STG_BYTES;
        ++stg_toggle;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* rowp = buf + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmC, buf, col, m0 + q * 32, z);
          tma_store_commit();
        }
      }
      // hand the accumulator back to the issuer (in the even CTA)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&acc_empty[a]), 0));
    }
    if (lane == 0) tma_store_wait<0>();
  }
  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // no MMA reads the peer's shared memory, no remote arrival is under way
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// fp32 [splits][n] partials -> out[n] (deterministic order)
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, size_t n, float* __restrict__ out) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 s = *reinterpret_cast<const float4*>(part + i);
  for (int z = 1; z < splits; ++z) {
    const float4 v = *reinterpret_cast<const float4*>(part + (size_t)z * n + i);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  *reinterpret_cast<float4*>(out + i) = s;
}

// ---------------------------------------------------------------- host
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

int encode_tensor_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int elem_bytes, int swizzle_bytes) {
  EncodeFn fn = get_encode_fn();
  if (!fn) {
    set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point unavailable");
    return BLSTM_E_CUDA;
  }
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  const CUtensorMapSwizzle swz = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                               : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                               : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx,
                  es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled rejected the tensor map");
    return BLSTM_E_CUDA;
  }
  return BLSTM_OK;
}

// Operand description: row-major 16-bit matrix [rows, cols] with leading dimension ld (elements).
// K-major operand: rows = M or N, cols = K.  MN-major operand: rows = K, cols = M or N.
static int make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                            bool mn_major, int tile_mn) {
  uint64_t dims[2] = {cols, rows};
  uint64_t str[1] = {ld * 2};
  uint32_t box[2];
  if (mn_major) { box[0] = 64; box[1] = BK; }            // 64 M/N elements x 64 k rows per box
  else          { box[0] = BK; box[1] = (uint32_t)tile_mn; }
  return encode_tensor_map(map, base, 2, dims, str, box);
}

// CTA pairs (256x256 tiles) need whole 256-column tiles to pay, and a reduction long enough to hide a
// tile's epilogue behind the next tile's main loop: with K = 512 (8 k-blocks, 4 k tensor clocks per tile)
// the pair kernel is bound by its epilogue and measured 0.68x cuBLAS against 0.95x for the single-CTA
// kernel, from K = 1024 on it is the faster one (0.91-1.07x cuBLAS against 0.79-1.07x).
// BLSTM_GEMM_NO_PAIRS=1 keeps the single-CTA kernel (for comparisons).
static bool gemm_uses_pairs(int M, int N, int K) {
  static const bool off = [] { const char* e = getenv("BLSTM_GEMM_NO_PAIRS"); return e && e[0] == '1'; }();
  return !off && M >= 256 && N % 256 == 0 && K >= 1024;
}

template <int A_MN, int B_MN, bool OUT_F32, typename T16>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                  int sm_count, cudaStream_t st) {
  auto kern = gemm_kernel<A_MN, B_MN, OUT_F32, T16>;
  BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM));
  const int tiles = p.m_tiles * p.n_tiles * p.splits;
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(ta, tb, tc, p);
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return BLSTM_OK;
}

template <int A_MN, int B_MN, bool OUT_F32, typename T16>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                       int sm_count, cudaStream_t st) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT_F32, T16>;
  BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_P_SMEM));
  const int tiles = p.m_tiles * p.n_tiles * p.splits;
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  kern<<<2 * pairs, GEMM_THREADS, GEMM_P_SMEM, st>>>(ta, tb, tc, p);
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return BLSTM_OK;
}

// C[M,N] = op(A) * op(B).  A: K-major [M,K] (lda) or M-major [K,M] (lda); B: K-major [N,K] or
// N-major [K,N].  out: 16-bit [M,ldc] (+bias) or fp32.  splits > 1 needs `partials`
// (fp32 [splits][M][ldc]) and writes the reduced result to out.
int gemm(int dtype, int M, int N, int K, const void* A, long long lda, bool a_mn, const void* B, long long ldb,
         bool b_mn, void* out, long long ldc, bool out_f32, const void* bias0, const void* bias1, int splits,
         float* partials, Control* ctl, cudaStream_t st) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc) return rc;
  // CTA pairs on 256x256 tiles when the output has whole tile columns and at least one full tile row
  const bool pair = gemm_uses_pairs(M, N, K);
  CUtensorMap ta, tb;
  rc = a_mn ? make_operand_map(&ta, A, K, M, lda, true, BM) : make_operand_map(&ta, A, M, K, lda, false, BM);
  if (rc) return rc;
  rc = b_mn ? make_operand_map(&tb, B, K, N, ldb, true, BN)
            : make_operand_map(&tb, B, N, K, ldb, false, pair ? 128 : BN);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = cdiv(M, pair ? 256 : BM); p.n_tiles = cdiv(N, BN);
  p.kb_total = cdiv(K, BK);
  if (splits < 1) splits = 1;
  if (splits > p.kb_total) splits = p.kb_total;
  p.kb_per_split = cdiv(p.kb_total, splits);
  p.splits = cdiv(p.kb_total, p.kb_per_split);
  p.fmt = dtype == BLSTM_BF16 ? 1 : 0;
  p.out = (p.splits > 1) ? (void*)partials : out;
  p.ldc = ldc;
  p.bias0 = bias0; p.bias1 = bias1;
  p.ctl = ctl;
  p.limit_ns = kDefaultWaitNs;
  if (p.splits > 1 && (!out_f32 || !partials)) return BLSTM_E_INVALID_ARG;
  CUtensorMap tc;
  {
    const int eb = out_f32 ? 4 : 2;
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)p.splits};
    uint64_t str[2] = {(uint64_t)ldc * eb, (uint64_t)M * ldc * eb};
    uint32_t box[3] = {out_f32 ? 32u : 64u, 32u, 1u};
    rc = encode_tensor_map(&tc, p.out, 3, dims, str, box, eb);
    if (rc) return rc;
  }
#define BLSTM_GEMM_CASE(AM, BMN, F32)                                                              \
  if (a_mn == (AM != 0) && b_mn == (BMN != 0) && out_f32 == F32) {                                 \
    if (pair)                                                                                      \
      rc = (dtype == BLSTM_BF16) ? launch_pair<AM, BMN, F32, __nv_bfloat16>(ta, tb, tc, p, di.sm_count, st) \
                                 : launch_pair<AM, BMN, F32, __half>(ta, tb, tc, p, di.sm_count, st);       \
    else                                                                                           \
      rc = (dtype == BLSTM_BF16) ? launch<AM, BMN, F32, __nv_bfloat16>(ta, tb, tc, p, di.sm_count, st)   \
                                 : launch<AM, BMN, F32, __half>(ta, tb, tc, p, di.sm_count, st);         \
  } else
  BLSTM_GEMM_CASE(0, 0, false)
  BLSTM_GEMM_CASE(0, 1, false)
  BLSTM_GEMM_CASE(1, 1, true)
  { return BLSTM_E_UNSUPPORTED; }
#undef BLSTM_GEMM_CASE
  if (rc) return rc;
  if (p.splits > 1) {
    const size_t n = (size_t)M * ldc;
    splitk_reduce_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(partials, p.splits, n, (float*)out);
    BLSTM_CUDA_OK(cudaGetLastError());
    count_launch();
  }
  return BLSTM_OK;
}

// ---------------------------------------------------------------- LSTM-level wrappers
// Split-K factor of the weight-gradient GEMMs (K = T*B is long, the output has few tiles).  The grid is
// persistent over tiles x splits work items, so what counts is how full the last wave of `sm_count`
// CTAs is: take the smallest factor within 3 % of the best wave efficiency (every extra split adds an
// fp32 partial of the output to write and reduce), with at least 8 k-blocks per split.
static int pick_splits(int M, int N, int K, int sm_count) {
  const bool pair = gemm_uses_pairs(M, N, K);
  const int tiles = cdiv(M, pair ? 256 : BM) * cdiv(N, BN);
  if (pair) sm_count /= 2;                     // work items are spread over CTA pairs
  const int kb = cdiv(K, BK);
  int max_s = kb / 8;
  if (max_s > 16) max_s = 16;
  if (max_s < 1) max_s = 1;
  double best = 0.0;
  for (int s = 1; s <= max_s; ++s) {
    const int items = tiles * s;
    const double eff = (double)items / ((double)cdiv(items, sm_count) * sm_count);
    if (eff > best) best = eff;
  }
  for (int s = 1; s <= max_s; ++s) {
    const int items = tiles * s;
    const double eff = (double)items / ((double)cdiv(items, sm_count) * sm_count);
    if (eff >= best - 0.03) return s;
  }
  return 1;
}

}  // namespace sm100

using namespace sm100;

bool sm100_gemm_supported(const blstm_desc& d) {
  if (d.flags & BLSTM_FLAG_FORCE_GENERIC) return false;
  if (d.dtype != BLSTM_F16 && d.dtype != BLSTM_BF16) return false;
  // 16-byte row pitches for TMA and 16-byte vector stores in the epilogues
  return d.input_size % 8 == 0 && d.hidden_size % 8 == 0;
}

static int wgrad_splits(const blstm_desc& d, int N) {
  return pick_splits(4 * d.hidden_size, N, d.seq_len * d.batch, plan_sm_count());
}

size_t sm100_bwd_gemm_workspace(const blstm_desc& d) {
  const size_t G = 4 * (size_t)d.hidden_size;
  const int sx = wgrad_splits(d, d.input_size), sh = wgrad_splits(d, d.hidden_size);
  size_t a = sx > 1 ? (size_t)sx * G * d.input_size * 4 : 0;
  size_t b = sh > 1 ? (size_t)sh * G * d.hidden_size * 4 : 0;
  return round_up(a > b ? a : b, 256);
}

int sm100_input_projection(const blstm_desc& d, const void* x, const void* Wx, const void* bx, const void* bh,
                           void* ifgo, cudaStream_t st) {
  const int M = d.seq_len * d.batch, N = 4 * d.hidden_size, K = d.input_size;
  return gemm(d.dtype, M, N, K, x, K, false, Wx, K, false, ifgo, N, false, bx, bh, 1, nullptr, nullptr, st);
}

int sm100_dgrad_input(const blstm_desc& d, const void* d_ifgo, const void* Wx, void* dx, void* ws, size_t ws_bytes,
                      cudaStream_t st) {
  (void)ws; (void)ws_bytes;
  const int M = d.seq_len * d.batch, N = d.input_size, K = 4 * d.hidden_size;
  return gemm(d.dtype, M, N, K, d_ifgo, K, false, Wx, N, true, dx, N, false, nullptr, nullptr, 1, nullptr, nullptr, st);
}

int sm100_wgrad(const blstm_desc& d, const void* d_ifgo, const void* x, const void* out, float* dWx, float* dWh,
                void* ws, size_t ws_bytes, cudaStream_t st) {
  const int TB = d.seq_len * d.batch, G = 4 * d.hidden_size, I = d.input_size, H = d.hidden_size;
  if (ws_bytes < sm100_bwd_gemm_workspace(d)) return BLSTM_E_WORKSPACE;
  int rc = gemm(d.dtype, G, I, TB, d_ifgo, G, true, x, I, true, dWx, I, true, nullptr, nullptr, wgrad_splits(d, I),
                (float*)ws, nullptr, st);
  if (rc) return rc;
  return gemm(d.dtype, G, H, TB, d_ifgo, G, true, out, H, true, dWh, H, true, nullptr, nullptr, wgrad_splits(d, H),
              (float*)ws, nullptr, st);
}

}  // namespace blstm
