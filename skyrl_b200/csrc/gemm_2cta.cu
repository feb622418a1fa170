// bf16 GEMM on pairs of SMs: two CTAs of a cluster share one 256 x BN output tile (tcgen05 cta_group::2).
// Each CTA stages its own 128 rows of A and only *half* of the B tile (BN/2 rows) in shared memory; the leader CTA's
// single MMA thread issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and accumulates into both
// CTAs' tensor memory (rows 0-127 in the leader, 128-255 in its partner).  Per output element the operand traffic
// into an SM drops from (128 + BN) to (128 + BN/2) rows per k-block, which is what bounds the one-CTA kernel on
// shapes whose operands stream from L2/HBM (weight-heavy and square problems alike).
//
// Synchronisation (all waits bounded, error code in the status word):
//   full[s]   leader only   <- TMA bytes of both CTAs (partner's copies signal the leader's barrier)
//   empty[s]  both CTAs     <- tcgen05.commit with a cluster mask from the leader's MMA thread
//   tfull[a]  both CTAs     <- same commit form, after the last k-block of a tile
//   tempty[a] leader only   <- the four epilogue warps of both CTAs (remote arrive from the partner)
// No load in this file uses a cluster-broadcast form: every TMA copy has exactly one destination CTA.
#include <cuda_runtime.h>

#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int k2BM = 256;   // rows per CTA pair
constexpr int k2HalfM = 128;
constexpr int k2BK = 64;
constexpr int k2Threads = 192;
constexpr int k2GroupM = 4;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;  // clears the CTA-pair bit of a shared::cluster address -> leader CTA

template <int BN>
struct Gemm2Cfg {
  static constexpr int kStages = (BN == 256) ? 6 : 8;
  static constexpr int kABytes = k2HalfM * k2BK * 2;       // this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * k2BK * 2;      // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;                 // two accumulator buffers
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint64_t* leader_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(leader_bar) & kPeerMask), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerMask) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives (once all earlier MMAs of this thread retired) on the barrier at the same offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

// Fused SwiGLU epilogues of the MLP GEMMs (BN = 256 only).
//  mode 1 (gate/up projection, NT): B is the stacked [2F, K] weight; the leader CTA loads 128 gate rows, its partner
//    the matching 128 up rows, so accumulator columns 0-127 / 128-255 hold gate / up of the same F-columns.  The
//    epilogue stores both to C ([M, 2F], kept for the backward pass) and silu(gate) * up to c2 ([M, F], row stride ld2).
//  mode 2 (input gradient of the down projection, NN): the accumulator is d(act); the epilogue reads gate / up from
//    aux ([M, 2F]) and stores d(gate) | d(up) to C ([M, 2F]) -- d(act) never reaches memory.
struct EpiArgs {
  int mode;
  int F;
  void* c2;
  const void* aux;
  long long ld2;
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TileMap2 {
  int m_blocks, n_blocks;
  __device__ __forceinline__ void get(int tile, int& pm, int& pn) const {
    const int per_group = k2GroupM * n_blocks;
    const int group = tile / per_group;
    const int first_m = group * k2GroupM;
    const int gsize = min(m_blocks - first_m, k2GroupM);
    const int r = tile - group * per_group;
    pm = first_m + (r % gsize);
    pn = r / gsize;
  }
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(k2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ C,
                  const __nv_bfloat16* __restrict__ bias, int M, int N, int K, long long ldc, int out_mode, int* status,
                  const EpiArgs epi) {
  using Cfg = Gemm2Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* tfull = bars + 2 * Cfg::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  TileMap2 tm{(M + k2BM - 1) / k2BM, (N + BN - 1) / BN};
  const int tiles = tm.m_blocks * tm.n_blocks;
  const int k_blocks = (K + k2BK - 1) / k2BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);   // used in the leader only
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);  // used in the leader only: 4 epilogue warps x 2 CTAs
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrive / copy completion
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  // barriers and tensor memory are private to the pair: with a programmatic dependent launch they are set up while
  // the previous kernel drains; operands and outputs may belong to that kernel, so every role waits for it here
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += n_pairs) {
        int pm, pn;
        tm.get(tile, pm, pn);
        const int row0 = pm * k2BM + static_cast<int>(rank) * k2HalfM;     // this CTA's rows of A
        // this CTA's half of the B tile (fused gate/up projection: gate rows for the leader, up rows for the partner)
        const int col0 = (!B_MN && epi.mode == 1) ? pn * (BN / 2) + static_cast<int>(rank) * epi.F
                                                  : pn * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, status, 0x401)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * Cfg::kStageBytes;
          uint8_t* sB = sA + Cfg::kABytes;
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * Cfg::kStageBytes);  // bytes of both CTAs
          if (!A_MN) {
            tma_load_2d_pair(sA, &tmA, &full[s], kb * k2BK, row0);
          } else {
#pragma unroll
            for (int j = 0; j < k2HalfM / 64; ++j) tma_load_2d_pair(sA + j * 8192, &tmA, &full[s], row0 + j * 64, kb * k2BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, &full[s], kb * k2BK, col0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 2 / 64; ++j) tma_load_2d_pair(sB + j * 8192, &tmB, &full[s], col0 + j * 64, kb * k2BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(k2BM, BN, A_MN, B_MN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += n_pairs, ++tcount) {
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1, status, 0x402)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&full[s], ph, status, 0x403)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < k2BK / 16; ++k) {
            const uint64_t adesc =
                A_MN ? make_smem_desc(a_base + k * 2048, 8192, 1024) : make_smem_desc(a_base + k * 32, 0, 1024);
            const uint64_t bdesc =
                B_MN ? make_smem_desc(b_base + k * 2048, 8192, 1024) : make_smem_desc(b_base + k * 32, 0, 1024);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[s]);  // frees stage s in both CTAs once these MMAs retire
        }
        if (ok) umma_commit_pair(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
    const int q = warp & 3;
    int tcount = 0;
    for (int tile = pair; tile < tiles; tile += n_pairs, ++tcount) {
      int pm, pn;
      tm.get(tile, pm, pn);
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aph, status, 0x404)) break;
      tc_fence_after();
      const int row = pm * k2BM + static_cast<int>(rank) * k2HalfM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (BN == 256 && epi.mode == 1) {
        // gate | up of the same 128 F-columns: store both, and silu(gate) * up computed from the rounded values.
        // One epilogue warp per scheduler has nothing to hide latency with, so the arithmetic is kept short:
        // bf16 pairs are packed once (the packed words are what gets stored) and unpacked by shifts, and
        // sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5 costs a single special-function instruction.
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32b_x32(t_row + c * 32, rg);
          tmem_ld_32x32b_x32(t_row + 128 + c * 32, ru);
          tmem_ld_wait();
          const int col = pn * 128 + c * 32;
          if (row < M && col < epi.F) {
            uint32_t pg[16], pu[16], pa[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              pg[j] = pack_bf16x2(__uint_as_float(rg[2 * j]), __uint_as_float(rg[2 * j + 1]));
              pu[j] = pack_bf16x2(__uint_as_float(ru[2 * j]), __uint_as_float(ru[2 * j + 1]));
              const float g0 = __uint_as_float(pg[j] << 16), g1 = __uint_as_float(pg[j] & 0xFFFF0000u);
              const float u0 = __uint_as_float(pu[j] << 16), u1 = __uint_as_float(pu[j] & 0xFFFF0000u);
              pa[j] = pack_bf16x2(g0 * fmaf(0.5f, tanh_approx(0.5f * g0), 0.5f) * u0,
                                  g1 * fmaf(0.5f, tanh_approx(0.5f * g1), 0.5f) * u1);
            }
            if (C != nullptr) {  // forward-only callers do not keep gate / up
              uint4* crow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + static_cast<long long>(row) * ldc + col);
              uint4* urow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + static_cast<long long>(row) * ldc + col + epi.F);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                crow[v] = make_uint4(pg[4 * v], pg[4 * v + 1], pg[4 * v + 2], pg[4 * v + 3]);
                urow[v] = make_uint4(pu[4 * v], pu[4 * v + 1], pu[4 * v + 2], pu[4 * v + 3]);
              }
            }
            uint4* arow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(epi.c2) + static_cast<long long>(row) * epi.ld2 + col);
#pragma unroll
            for (int v = 0; v < 4; ++v) arow[v] = make_uint4(pa[4 * v], pa[4 * v + 1], pa[4 * v + 2], pa[4 * v + 3]);
          }
        }
      } else if (BN == 256 && epi.mode == 2) {
        // d(act) -> d(gate) | d(up); the gate / up values of the next chunk are requested before this chunk's arithmetic
        const bool live = row < M;
        const uint4* gsrc = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(epi.aux) +
                                                           static_cast<long long>(live ? row : 0) * epi.ld2 + pn * BN);
        const int f_vec = epi.F >> 3;  // uint4 between the gate and the up value of a column
        uint4 ng[4], nu[4];
        auto fetch = [&](int c) {
          if (live && pn * BN + c * 32 < epi.F) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              ng[v] = __ldg(gsrc + c * 4 + v);
              nu[v] = __ldg(gsrc + f_vec + c * 4 + v);
            }
          }
        };
        fetch(0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          uint4 cg[4], cu[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            cg[v] = ng[v];
            cu[v] = nu[v];
          }
          if (c + 1 < BN / 32) fetch(c + 1);
          tmem_ld_wait();
          const int col = pn * BN + c * 32;
          if (live && col < epi.F) {
            const uint32_t* wg = reinterpret_cast<const uint32_t*>(cg);
            const uint32_t* wu = reinterpret_cast<const uint32_t*>(cu);
            uint32_t pg[16], pu[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float dg2[2], du2[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float g = __uint_as_float(e ? (wg[j] & 0xFFFF0000u) : (wg[j] << 16));
                const float u = __uint_as_float(e ? (wu[j] & 0xFFFF0000u) : (wu[j] << 16));
                const float d = __uint_as_float(r[2 * j + e]);
                const float sig = fmaf(0.5f, tanh_approx(0.5f * g), 0.5f);
                const float silu = g * sig;
                du2[e] = d * silu;
                dg2[e] = d * u * fmaf(silu, 1.f - sig, sig);
              }
              pg[j] = pack_bf16x2(dg2[0], dg2[1]);
              pu[j] = pack_bf16x2(du2[0], du2[1]);
            }
            uint4* crow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + static_cast<long long>(row) * ldc + col);
            uint4* urow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + static_cast<long long>(row) * ldc + col + epi.F);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              crow[v] = make_uint4(pg[4 * v], pg[4 * v + 1], pg[4 * v + 2], pg[4 * v + 3]);
              urow[v] = make_uint4(pu[4 * v], pu[4 * v + 1], pu[4 * v + 2], pu[4 * v + 3]);
            }
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = pn * BN + c * 32;
        if (row < M && col0 < N) {
          const bool full_chunk = (col0 + 32 <= N);
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              const float b = (col < N) ? __bfloat162float(__ldg(bias + col)) : 0.f;
              r[j] = __float_as_uint(__uint_as_float(r[j]) + b);
            }
          }
          if (out_mode == 0) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(C) + static_cast<long long>(row) * ldc + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                reinterpret_cast<uint4*>(crow)[v] = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          } else {
            float* crow = reinterpret_cast<float*>(C) + static_cast<long long>(row) * ldc + col0;
            const bool vec = full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if (out_mode == 2) {
                  const float4 p = reinterpret_cast<float4*>(crow)[v];
                  o.x += p.x;
                  o.y += p.y;
                  o.z += p.z;
                  o.w += p.w;
                }
                reinterpret_cast<float4*>(crow)[v] = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) {
                  float o = __uint_as_float(r[j]);
                  if (out_mode == 2) o += crow[j];
                  crow[j] = o;
                }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[acc]);  // this accumulator buffer may be overwritten
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner may still be reading this CTA's shared / tensor memory until here
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm2(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                        long long ldb, long long ldc, int out_mode, cudaStream_t stream, EpiArgs epi = EpiArgs{}) {
  using Cfg = Gemm2Cfg<BN>;
  const CUtensorMap* ta = A_MN ? get_tmap_bf16_2d(A, K, M, lda, 64) : get_tmap_bf16_2d(A, M, K, lda, k2HalfM);
  const CUtensorMap* tb = B_MN ? get_tmap_bf16_2d(B, K, N, ldb, 64) : get_tmap_bf16_2d(B, N, K, ldb, BN / 2);
  if (!ta || !tb) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  auto kfn = gemm2_bf16_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  const int tiles = ((M + k2BM - 1) / k2BM) * ((N + BN - 1) / BN);
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  const cudaError_t e = launch_pdl(kfn, dim3(2 * pairs), dim3(k2Threads), Cfg::kSmemBytes, stream, *ta, *tb, C,
                                   reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, out_mode, device_status_ptr(),
                                   epi);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // namespace sb

extern "C" {

// Same contract as sb_gemm_bf16 (C = op(A) op(B) + bias; a_mn / b_mn operand layouts; out_mode 0 bf16, 1 fp32,
// 2 fp32 accumulate) on CTA pairs; bn in {128, 256}.
int sb_gemm_bf16_2cta(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                      long long ldb, long long ldc, int a_mn, int b_mn, int out_mode, int bn, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7)) return SB_ERR_ARG;
  if (out_mode < 0 || out_mode > 2) return SB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn != 128) bn = 256;
#define SB_G2(BNV, AM, BM_)                                                                                           \
  if (bn == BNV && (a_mn != 0) == AM && (b_mn != 0) == BM_)                                                           \
    return sb::launch_gemm2<BNV, AM, BM_>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, st);
  SB_G2(256, false, false) SB_G2(256, false, true) SB_G2(256, true, true) SB_G2(256, true, false)
  SB_G2(128, false, false) SB_G2(128, false, true) SB_G2(128, true, true) SB_G2(128, true, false)
#undef SB_G2
  return SB_ERR_ARG;
}

// Fused MLP products on CTA pairs (see EpiArgs).  F must be a multiple of 128, every pointer 16-byte aligned and
// every row stride a multiple of 8 elements.
//   sb_mlp_gate_up_swiglu: gu[M, 2F] = x[M, K] * W[2F, K]^T and act[M, F] = silu(gu[:, :F]) * gu[:, F:]
//                          (gu may be null: only act is stored)
//   sb_mlp_down_dgrad:     dgu[M, 2F] = d swiglu(gu) applied to (dy[M, H] * Wd[H, F]) without storing the product
int sb_mlp_gate_up_swiglu(const void* x, const void* w, void* gu, void* act, int M, int F, int K, long long ldx,
                          long long ldw, void* stream) {
  if (M <= 0 || F <= 0 || K <= 0 || (F % 128) != 0 || (ldx & 7) || (ldw & 7)) return SB_ERR_ARG;
  sb::EpiArgs epi{1, F, act, nullptr, F};
  return sb::launch_gemm2<256, false, false>(x, w, gu, nullptr, M, 2 * F, K, ldx, ldw, 2LL * F, 0,
                                             reinterpret_cast<cudaStream_t>(stream), epi);
}

int sb_mlp_down_dgrad(const void* dy, const void* wd, const void* gu, void* dgu, int M, int F, int H, long long lddy,
                      long long ldwd, void* stream) {
  if (M <= 0 || F <= 0 || H <= 0 || (F % 32) != 0 || (lddy & 7) || (ldwd & 7)) return SB_ERR_ARG;
  sb::EpiArgs epi{2, F, nullptr, gu, 2LL * F};
  return sb::launch_gemm2<256, false, true>(dy, wd, dgu, nullptr, M, F, H, lddy, ldwd, 2LL * F, 0,
                                            reinterpret_cast<cudaStream_t>(stream), epi);
}

}  // extern "C"
