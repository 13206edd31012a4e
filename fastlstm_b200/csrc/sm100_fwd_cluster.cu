// Persistent forward recurrence for small hidden sizes (H = 64, 128, 256; 16-bit), where a step is a
// pure latency chain: the H/16 CTAs that share a batch tile form ONE thread-block cluster and hand
// h[t+1] to each other through distributed shared memory instead of global memory.
// (Replaces persistent_fwd_kernel, fastlstm/kernels.py:414-663, and its global-atomic handshake,
// :546-548 and :659-661, for these shapes.)
//
// Per step the general kernel pays, one after the other, a release of the h stores at GPU scope, the
// trip of an arrival counter through L2 to the pollers, a proxy fence and a TMA load of h from L2 -
// more than half of the step.  Here every CTA keeps the whole h tile [128 rows x H] of the step in its
// own shared memory, as the MMA's A operand, in the un-swizzled K-major layout
//     [H/8 pieces of 8 units][128 rows][16 bytes]
// in which the 16 units a CTA produces are ONE contiguous 4 KB block (a batch of fewer than 128 rows
// keeps only its own rows per piece - what crosses the cluster is what limits the step - and the
// MMA's rows past them read the next piece: garbage in accumulator rows nobody uses).  The epilogue writes that block
// into a staging buffer and one warp sends it to all CTAs of the cluster (itself included) with
// cp.async.bulk.shared::cluster; the copies signal the receivers' mbarriers (one per 64-unit K chunk),
// on which the MMA issuers wait.  No flag, no polling, no fence on the chain.  Two operand buffers
// (by step parity) and two staging buffers: a CTA can only be one step ahead of a peer, because it needs
// that peer's slice of every step.  Clusters are independent (one per batch tile), so the launch is a
// plain cluster launch; the shape is only taken when all tiles' clusters can be resident at once.
//
//   warp 0      set-up (Wh slice by TMA, h0 tile), then the sender
//   warps 1..4  tcgen05.mma issuers, one K chunk and one TMEM accumulator each
//   warps 5..8  epilogue: thread = batch row x 16 units x 4 gates, c carried in fp32 registers
#include <stdio.h>

#include "sm100.cuh"
#include "sm100_common.cuh"
#include "sm100_rec_util.cuh"

namespace blstm {
namespace sm100 {

constexpr int CL_ROWS = 128;               // batch rows per tile (MMA M)
constexpr int CL_UH = 16;                  // hidden units per CTA
constexpr int CL_N = 4 * CL_UH;            // gate rows per CTA (MMA N)
constexpr int CL_SLICE = CL_ROWS * CL_UH * 2;   // bytes of one CTA's h slice (two 8-unit pieces) at 128 rows
constexpr int CL_MAX_TILES = 7;            // clusters of 16 that a B200 keeps resident with this footprint

struct ClusterFwdParams {
  int T, B, H;
  int nh;                   // CTAs per cluster = H / 16
  int ra;                   // rows a piece holds: 128, or the batch rounded up to 8 when it is a single smaller tile
  int fmt;
  int no_arrive;
  int inference;
  unsigned long long limit_ns;
  Control* ctl;
  void* ifgo;               // [T,B,4H] in/out
  void* out;                // [T+1,B,H]
  void* cell;               // [T+1,B,H]
};

__host__ __device__ constexpr uint64_t smem_desc_noswizzle(uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16) | (uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32) |
         (uint64_t(1) << 46);
}

static size_t cluster_fwd_smem(int H) {
  return 1024 + (size_t)CL_N * H * 2 + 2 * (size_t)CL_ROWS * H * 2 + 2 * CL_SLICE + 512;
}

template <typename T16>
__global__ void __launch_bounds__(288, 1)
fwd_cluster_kernel(const __grid_constant__ CUtensorMap tmW, const ClusterFwdParams p) {
  constexpr int NACC = 4;
  constexpr int FIRST_EPI = 1 + NACC;
  constexpr int ACC_STRIDE = 256;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int H = p.H, T = p.T;
  const int KC = H / 64;                                       // K chunks = issuers in use
  const int RA = p.ra;                                         // rows per piece
  const int PIECE = RA * 16, SLICE = 2 * PIECE;                // bytes of an 8-unit piece / of a CTA's 16 units
  const int A_BYTES = (H / 8) * PIECE;
  uint8_t* w_s = smem;                                         // [KC][64 gate rows][128 B], 128-byte swizzle
  uint8_t* a_s = w_s + (size_t)CL_N * H * 2;                   // [2][H/8][RA rows][16 B]
  uint8_t* stg = a_s + 2 * (size_t)CL_ROWS * H * 2;            // [2][2][RA rows][16 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg + 2 * CL_SLICE);
  uint64_t* cfull = bars;                                      // [2][4] chunk of h[t] complete (4 slices)
  uint64_t* acc_full = bars + 8;                               // [2]
  uint64_t* acc_empty = acc_full + 2;                          // [2]
  uint64_t* staged = acc_empty + 2;                            // [2] epilogue wrote its slice
  uint64_t* w_full = staged + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_full + 1);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ht = (int)cluster_ctarank();                       // which 16 units
  const int bt = blockIdx.x / p.nh;                            // which batch tile
  const int row_base = bt * CL_ROWS;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(&cfull[i], 1);       // one arming arrival + transaction bytes
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], KC); mbar_init(&acc_empty[a], 4); mbar_init(&staged[a], 4); }
    mbar_init(w_full, 1);
    *dead = 0;
    fence_mbar_init();
    for (int i = 0; i < 8; ++i) mbar_expect_tx(&cfull[i], 4 * SLICE);      // armed for their first use
    tma_prefetch_desc(&tmW);
    mbar_expect_tx(w_full, (uint32_t)((size_t)CL_N * H * 2));
    for (int kc = 0; kc < KC; ++kc) tma_load_3d(w_s + (size_t)kc * CL_N * 128, &tmW, w_full, kc * 64, ht * CL_UH, 0);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  // h[0] of this tile into operand buffer 0: 16-byte pieces (row, 8 units) -> [piece][row][16 B]
  {
    const T16* h0 = reinterpret_cast<const T16*>(p.out);
    const int pieces = H / 8;
    for (int i = threadIdx.x; i < RA * pieces; i += blockDim.x) {
      const int row = i / pieces, kp = i % pieces;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row_base + row < p.B) v = ldg16(h0 + (size_t)(row_base + row) * H + 8 * kp);
      *reinterpret_cast<uint4*>(a_s + (size_t)kp * PIECE + row * 16) = v;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();                 // every peer's barriers exist before anything is sent to them
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{dead, p.ctl, p.limit_ns, -1, (int)blockIdx.x};

  if (warp == 0) {
    // ---------------------------------------------------------------- sender
    // After step t the epilogue's slice of h[t+1] sits in staging buffer (t+1)&1; lane d copies it into
    // CTA d's operand buffer (t+1)&1 and counts its bytes on that CTA's barrier of the chunk it belongs to.
    bool ok = true;
    for (int t = 0; t + 1 < T && ok; ++t) {
      const int par = (t + 1) & 1;
      wc.d0 = t; wc.d1 = bt;
      if (!mbar_wait(&staged[par], (uint32_t)(t >> 1) & 1u, wc)) { ok = false; break; }
      if (lane < p.nh && !p.no_arrive) {
        const uint32_t dst = mapa_shared(smem_u32(a_s) + par * A_BYTES + ht * SLICE, lane);
        const uint32_t bar = mapa_shared(smem_u32(&cfull[par * 4 + (ht >> 2)]), lane);
        dsmem_bulk_copy(dst, stg + par * CL_SLICE, SLICE, bar);
      }
      __syncwarp();
    }
  } else if (warp < 1 + NACC) {
    // ---------------------------------------------------------------- MMA issuers
    const int x = warp - 1;                 // K chunk and accumulator of this issuer
    if (lane == 0 && x < KC) {
      const uint64_t descA = smem_desc_noswizzle(PIECE, 128);      // K-major, pieces PIECE bytes apart, 8-row groups 128 B
      constexpr uint64_t descB = smem_desc_base(16, 1024);         // Wh slice, K-major, 128-byte swizzle
      const uint32_t idesc = instr_desc(p.fmt, 0, 0, CL_ROWS, CL_N);
      bool ok = mbar_wait(w_full, 0, wc);
      uint32_t acc_ph[2] = {0, 0};
      const uint32_t sb = smem_u32(w_s) + (uint32_t)x * CL_N * 128;
      for (int t = 0; t < T && ok; ++t) {
        const int a = t & 1, par = t & 1;
        wc.d0 = t; wc.d1 = bt;
        if (!mbar_wait(&acc_empty[a], acc_ph[a] ^ 1, wc)) { ok = false; break; }
        acc_ph[a] ^= 1;
        if (t > 0) {
          // the four slices of this chunk of h[t]: buffer `par` on its ((t-1)/2)-th... use
          const uint32_t ph = (uint32_t)((t - (par ? 1 : 2)) >> 1) & 1u;
          if (!mbar_wait_cluster(&cfull[par * 4 + x], ph, wc)) { ok = false; break; }
          mbar_expect_tx(&cfull[par * 4 + x], 4 * SLICE);        // arm the barrier's next use (step t+2)
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(a_s) + par * A_BYTES + (uint32_t)x * 8 * PIECE;
        const uint32_t d_tmem = tmem_base + a * ACC_STRIDE + x * CL_N;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(d_tmem, smem_desc(descA, sa + k * 2 * PIECE), smem_desc(descB, sb + k * 32), idesc, k > 0 ? 1u : 0u);
        umma_commit(&acc_full[a]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const int row = row_base + row_in_tile;
    const bool row_ok = row < p.B;
    const int unit0 = ht * CL_UH;
    const size_t H4 = 4 * (size_t)H;
    T16* ifgo = reinterpret_cast<T16*>(p.ifgo);
    T16* out = reinterpret_cast<T16*>(p.out);
    T16* cell = reinterpret_cast<T16*>(p.cell);
    float c[CL_UH];
#pragma unroll
    for (int u = 0; u < CL_UH; ++u) c[u] = 0.f;
    uint4 pre[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) pre[i] = make_uint4(0, 0, 0, 0);
    if (row_ok) {
      unpack8<T16>(ldg16(cell + (size_t)row * H + unit0), &c[0]);
      unpack8<T16>(ldg16(cell + (size_t)row * H + unit0 + 8), &c[8]);
    }
    auto load_pre = [&](int t) {
      if (t < T && row_ok) {
        const T16* src = ifgo + ((size_t)t * p.B + row) * H4 + unit0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          pre[2 * g] = ldg16(src + (size_t)g * H);
          pre[2 * g + 1] = ldg16(src + (size_t)g * H + 8);
        }
      }
    };
    load_pre(0);
    bool ok = true;
    for (int t = 0; t < T && ok; ++t) {
      const int a = t & 1;
      wc.d0 = t; wc.d1 = bt;
      if (!mbar_wait(&acc_full[a], (uint32_t)(t >> 1) & 1u, wc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + a * ACC_STRIDE + (uint32_t(q * 32) << 16);
      float pa[4][CL_UH];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t w8[8] = {pre[2 * g].x, pre[2 * g].y, pre[2 * g].z, pre[2 * g].w,
                                pre[2 * g + 1].x, pre[2 * g + 1].y, pre[2 * g + 1].z, pre[2 * g + 1].w};
#pragma unroll
        for (int u = 0; u < CL_UH; ++u) {
          const float2 f2 = cvt2<T16>(w8[u >> 1]);
          pa[g][u] = (u & 1) ? f2.y : f2.x;
        }
        // the issuers' partial sums, two accumulators per wait (32 values in flight)
#pragma unroll
        for (int x0 = 0; x0 < NACC; x0 += 2) {
          if (x0 < KC) {
            uint32_t v[2][CL_UH];
            tmem_ld_32x16(taddr + x0 * CL_N + g * CL_UH, v[0]);
            if (x0 + 1 < KC) tmem_ld_32x16(taddr + (x0 + 1) * CL_N + g * CL_UH, v[1]);
            tmem_ld_wait();
#pragma unroll
            for (int u = 0; u < CL_UH; ++u) {
              pa[g][u] += __uint_as_float(v[0][u]);
              if (x0 + 1 < KC) pa[g][u] += __uint_as_float(v[1][u]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
      float hv[CL_UH];
#pragma unroll
      for (int u = 0; u < CL_UH; ++u) {
        const float cn = sigmoid_fast(pa[1][u]) * c[u] + sigmoid_fast(pa[0][u]) * tanh_fast(pa[2][u]);
        c[u] = cn;
        hv[u] = sigmoid_fast(pa[3][u]) * tanh_fast(cn);
      }
      // h[t+1]: first into the staging buffer the sender ships from (rows past B as zeros), then to global
      const int par = (t + 1) & 1;
      uint4 h0v = make_uint4(0, 0, 0, 0), h1v = make_uint4(0, 0, 0, 0);
      if (row_ok) {
        h0v = make_uint4(pk2<T16>(hv[0], hv[1]), pk2<T16>(hv[2], hv[3]), pk2<T16>(hv[4], hv[5]), pk2<T16>(hv[6], hv[7]));
        h1v = make_uint4(pk2<T16>(hv[8], hv[9]), pk2<T16>(hv[10], hv[11]), pk2<T16>(hv[12], hv[13]), pk2<T16>(hv[14], hv[15]));
      }
      if (t + 1 < T) {
        if (row_in_tile < RA) {
          uint8_t* sp = stg + par * CL_SLICE + row_in_tile * 16;
          *reinterpret_cast<uint4*>(sp) = h0v;
          *reinterpret_cast<uint4*>(sp + PIECE) = h1v;
        }
        fence_proxy_async_smem();             // visible to the bulk-copy engine
        __syncwarp();
        if (lane == 0) mbar_arrive(&staged[par]);
      }
      const size_t o1 = ((size_t)(t + 1) * p.B + row) * H + unit0;
      if (row_ok) {
        stg16(out + o1, h0v);
        stg16(out + o1 + 8, h1v);
      }
      // off the chain: next step's projected pre-activations, then what backward needs
      T16* gdst = ifgo + ((size_t)t * p.B + row) * H4 + unit0;
      load_pre(t + 1);
      if (row_ok && (!p.inference || t == T - 1)) {
        store8<T16>(cell + o1, &c[0]);
        store8<T16>(cell + o1 + 8, &c[8]);
      }
      if (row_ok && !p.inference) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          store8<T16>(gdst + (size_t)g * H, &pa[g][0]);
          store8<T16>(gdst + (size_t)g * H + 8, &pa[g][8]);
        }
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  cluster_sync_all();   // no CTA leaves while a peer may still write into its shared memory
}

template <typename T16>
static int launch_cluster_fwd(const blstm_desc& d, const CUtensorMap& tw, const ClusterFwdParams& p, int nbt, cudaStream_t st,
                              bool* taken) {
  auto kern = fwd_cluster_kernel<T16>;
  const size_t smem = cluster_fwd_smem(d.hidden_size);
  BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (p.nh > 8) BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.nh * nbt);
  cfg.blockDim = dim3(288);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = p.nh;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  // all tiles' clusters at once, or the general kernel takes the problem
  int max_clusters = 0;
  BLSTM_CUDA_OK(cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg));
  if (max_clusters < nbt) { *taken = false; return BLSTM_OK; }
  BLSTM_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tw, p));
  count_launch();
  *taken = true;
  return BLSTM_OK;
}

}  // namespace sm100

using namespace sm100;

bool sm100_fwd_cluster_shape(const blstm_desc& d) {
  if (d.flags & (BLSTM_FLAG_FORCE_GENERIC | BLSTM_FLAG_NO_CLUSTER)) return false;
  if (d.dtype != BLSTM_F16 && d.dtype != BLSTM_BF16) return false;
  const int H = d.hidden_size;
  if (H != 64 && H != 128 && H != 256) return false;
  return cdiv(d.batch, CL_ROWS) <= CL_MAX_TILES;
}

int sm100_fwd_cluster(const blstm_desc& d, void* ifgo, const void* Wh, void* out, void* cell, void* ws,
                      cudaStream_t st, bool* taken) {
  *taken = false;
  if (!sm100_fwd_cluster_shape(d)) return BLSTM_OK;
  const int H = d.hidden_size, B = d.batch, T = d.seq_len;
  CUtensorMap tw;
  {  // Wh [4H,H] as {k, unit row, gate}
    uint64_t dims[3] = {(uint64_t)H, (uint64_t)H, 4};
    uint64_t str[2] = {(uint64_t)H * 2, (uint64_t)H * H * 2};
    uint32_t box[3] = {64, (uint32_t)CL_UH, 4};
    int rc = encode_tensor_map(&tw, Wh, 3, dims, str, box);
    if (rc) return rc;
  }
  ClusterFwdParams p;
  p.T = T; p.B = B; p.H = H;
  p.nh = H / CL_UH;
  p.ra = B < CL_ROWS ? (int)round_up((size_t)B, 8) : CL_ROWS;
  p.fmt = d.dtype == BLSTM_BF16 ? 1 : 0;
  p.no_arrive = (d.flags & BLSTM_FLAG_TEST_NO_ARRIVE) ? 1 : 0;
  p.inference = (d.flags & BLSTM_FLAG_INFERENCE) ? 1 : 0;
  p.limit_ns = d.wait_limit_us > 0 ? (unsigned long long)d.wait_limit_us * 1000ull : kDefaultWaitNs;
  p.ctl = reinterpret_cast<Control*>(ws);
  p.ifgo = ifgo; p.out = out; p.cell = cell;
  const int nbt = cdiv(B, CL_ROWS);
  return d.dtype == BLSTM_BF16 ? launch_cluster_fwd<__nv_bfloat16>(d, tw, p, nbt, st, taken)
                               : launch_cluster_fwd<__half>(d, tw, p, nbt, st, taken);
}

}  // namespace blstm
