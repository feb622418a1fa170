// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A * B (+bias) with
//   * operands staged in shared memory by TMA (128-byte swizzle), a multi-stage
//     mbarrier ring between one producer thread and one MMA-issuing thread,
//   * tcgen05.mma (cta_group::1, 128 x BN x 16) accumulating in TMEM, two
//     accumulator buffers so that the epilogue of tile i overlaps the main loop
//     of tile i+1,
//   * a persistent grid (one CTA per SM) walking tiles in an L2-friendly order.
//
// Operand layouts ("major" = which logical dimension is contiguous in memory):
//   A K-major : A stored [M, K] (row stride lda)      -> y = x W^T, dx = dy W
//   A MN-major: A stored [K, M]                        -> dW = dy^T x
//   B K-major : B stored [N, K] (nn.Linear weight)     -> y = x W^T
//   B MN-major: B stored [K, N]                        -> dx = dy W, dW = dy^T x
// so all three GEMMs of a linear layer's forward/backward run without an
// explicit transpose.
#include <cstdlib>

#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;  // warp0: TMA, warp1: MMA + TMEM alloc, warps 2-5: epilogue
constexpr int kGroupM = 8;

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

enum OutMode { kOutBf16 = 0, kOutF32 = 1, kOutF32Accum = 2 };

// Tensor-parallel extensions of the kernel (both optional, selected by template flags):
//  GATHER  - the A operand is sequence-sharded over n_ranks GPUs.  Four extra warps copy the remote shards into
//            this GPU's full-size A buffer piece by piece (plain peer loads over NVLink, each byte crosses once)
//            and publish a per-m-block counter; the TMA producer waits for an m-block's counter before loading
//            it, and tiles are walked starting with the local shard so the copies hide behind the math.
//  SCATTER - the epilogue stores each output tile straight into peer memory: to the rank that owns those rows
//            (reduce-scatter layout, slot = this rank) or to every rank (all-reduce layout); the consumer kernel
//            on the owning GPU adds the n_ranks slots.
constexpr int kTpMaxRanks = 8;
constexpr int kGatherWarps = 4;
constexpr int kPiecesPerBlock = 8;  // an m-block (128 rows) is copied as 8 pieces of 16 rows

struct TpArgs {
  const void* src[kTpMaxRanks];  // GATHER: rank r's own shard (rows [r*rows_per_rank, ...) of the full matrix)
  void* a_full;                  // GATHER: this GPU's full A buffer (the tensor map covers it)
  unsigned int* flags;           // GATHER: [m_blocks] piece counters followed by one work ticket
  void* dst[kTpMaxRanks];        // SCATTER: rank d's partial-sum buffer
  long long lda;                 // GATHER: row stride of A in elements
  long long slot_stride;         // SCATTER: elements between two source ranks' slots in a destination buffer
  int n_ranks, my_rank;
  int rows_per_rank;             // rows of the full matrix owned by each rank (A rows for GATHER, C rows for SCATTER)
  int scatter_all;               // SCATTER: 0 = rows go to their owner only, 1 = every rank receives every row
  // Sequence-parallel attention (all-to-all fused into the projections around it):
  //  scatter_cols: the output columns are up to three segments (q | k | v heads), each split evenly over the
  //    ranks; a column chunk goes to the rank that owns its heads, at row my_rank * rows_per_rank + row of that
  //    rank's [n_ranks * rows_per_rank, local width] buffer (sequence-sharded -> head-sharded).
  //  gather_cols: the A operand's rows are local, its columns are blocks of cols_per_rank owned by the ranks
  //    (head-sharded -> sequence-sharded): rank r's block comes from src[r] rows [my_rank * M, ...).
  int scatter_cols, gather_cols;
  int seg_start[3], seg_w[3];    // scatter_cols: first column and per-rank width of each segment (0 width = unused)
  int cols_per_rank;             // gather_cols
  long long src_ld;              // gather_cols / gather_idx: row stride of the source buffers
  // Expert-parallel MoE (token dispatch / combine fused into the expert GEMMs):
  //  gather_idx:  A row r is row idx_row[r] of rank idx_rank[r]'s token buffer src[rank] (dispatch).
  //  scatter_idx: C row r is stored to row idx_row[r] of rank idx_rank[r]'s buffer dst[rank] (combine).
  int gather_idx, scatter_idx;
  const int* idx_rank;
  const int* idx_row;
  // Grouped (per-expert) products; the tables live on the device, so no expert count ever visits the host.
  //  group_mode 1: the rows of A / C are grouped in blocks of 128: m-block pm belongs to expert tile_expert[pm]
  //    (< 0: unused block, skipped) and multiplies that expert's B matrix, which starts group_b_rows * expert rows
  //    further down the B tensor map.
  //  group_mode 2 (weight gradients): work item = (expert, output tile); the contraction runs over the row range
  //    [k_off[e], k_off[e + 1]) of both operands (multiples of 64; an empty range skips the item) and the result
  //    goes to C + e * split_stride.
  int group_mode;
  int group_b_rows;
  const int* tile_expert;
  const int* k_off;
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

struct TileMap {
  int m_blocks, n_blocks;
  __device__ __forceinline__ void get(int tile, int& pm, int& pn) const {
    const int per_group = kGroupM * n_blocks;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int gsize = min(m_blocks - first_m, kGroupM);
    const int r = tile - group * per_group;
    pm = first_m + (r % gsize);
    pn = r / gsize;
  }
};

template <int BN, bool A_MN, bool B_MN, bool GATHER = false, bool SCATTER = false>
__global__ void __launch_bounds__(kGemmThreads + (GATHER ? kGatherWarps * 32 : 0), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ C,
                 const __nv_bfloat16* __restrict__ bias, int M, int N, int K, long long ldc, int out_mode, int splits,
                 long long split_stride, int* status, const __grid_constant__ TpArgs tp, int prefetch_b) {
  // prefetch_b: the B operand is constant data (weights) that no kernel earlier in the stream writes, so its first
  // tiles may be requested before waiting for the predecessor grid (programmatic dependent launch).
  // splits > 1: split-K. Work item = (output tile, k slice); slice ks writes its fp32 partial sum to
  // C + ks * split_stride (the consumer kernel adds the partials), bias is applied by slice 0 only.
  using Cfg = GemmCfg<BN>;
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
  TileMap tm{(M + kBM - 1) / kBM, (N + BN - 1) / BN};
  const int tiles_mn = tm.m_blocks * tm.n_blocks;
  const int tiles = tiles_mn * splits;
  const int k_blocks = (K + kBK - 1) / kBK;
  const int kpb = (k_blocks + splits - 1) / splits;  // k blocks per slice (host guarantees no empty slice)
  auto krange = [&](int ks, int& kb0, int& kb1) {
    if (tp.group_mode == 2) {
      kb0 = __ldg(tp.k_off + ks) / kBK;
      kb1 = __ldg(tp.k_off + ks + 1) / kBK;
    } else {
      kb0 = ks * kpb;
      kb1 = min(k_blocks, kb0 + kpb);
    }
  };
  // GATHER: logical m-block 0 is the first block of the local shard, then the next rank's, and so on
  const int m_rot = (GATHER && !tp.gather_cols && !tp.gather_idx) ? tp.my_rank * (tp.rows_per_rank / kBM) : 0;
  auto rot = [&](int pm) { return GATHER ? (pm + m_rot) % tm.m_blocks : pm; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  // everything above (barriers, tensor memory) is private to this CTA and may overlap the previous kernel's tail;
  // operands and outputs may belong to that kernel, so all roles wait for it here
  pdl_launch_dependents();
  int b_ahead = 0;  // stages of the first tile whose B half is already in flight (producer thread only)
  if (prefetch_b && !GATHER && threadIdx.x == 0 && blockIdx.x < tiles) {
    int pm, pn;
    const int ks = blockIdx.x / tiles_mn;
    tm.get(blockIdx.x - ks * tiles_mn, pm, pn);
    const int kb0 = ks * kpb, kb1 = min(k_blocks, kb0 + kpb);
    b_ahead = min(Cfg::kStages, kb1 - kb0);
    for (int j = 0; j < b_ahead; ++j) {
      uint8_t* sB = smem + j * Cfg::kStageBytes + Cfg::kABytes;
      mbar_arrive_expect_tx(&full[j], Cfg::kStageBytes);
      if (!B_MN) {
        tma_load_2d(sB, &tmB, &full[j], (kb0 + j) * kBK, pn * BN);
      } else {
#pragma unroll
        for (int q2 = 0; q2 < BN / 64; ++q2) tma_load_2d(sB + q2 * 8192, &tmB, &full[j], pn * BN + q2 * 64, (kb0 + j) * kBK);
      }
    }
  }
  pdl_wait();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int it = 0;
      bool ok = true;
      unsigned long long ready_mask = 0;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int pm, pn;
        const int ks = tile / tiles_mn;
        tm.get(tile - ks * tiles_mn, pm, pn);
        pm = rot(pm);
        if (GATHER) {
          // rows of another rank: wait until the copy warps have landed every piece of this m-block
          const int owner = (tp.gather_cols || tp.gather_idx) ? -1 : (pm * kBM) / tp.rows_per_rank;
          const unsigned int need = tp.gather_cols ? kPiecesPerBlock * tp.n_ranks : kPiecesPerBlock;
          if (owner != tp.my_rank && !((ready_mask >> (pm & 63)) & 1ull)) {
            const unsigned long long t0 = globaltimer_ns();
            while (ld_acquire_gpu(tp.flags + pm) < need) {
              if (*reinterpret_cast<volatile int*>(status) != 0 || globaltimer_ns() - t0 > kWaitTimeoutNs) {
                atomicCAS(status, 0, 0x104);
                ok = false;
                break;
              }
            }
            if (!ok) break;
            fence_proxy_async_global();  // generic-proxy stores of the copy warps -> async-proxy (TMA) reads
            if (tm.m_blocks <= 64) ready_mask |= 1ull << pm;
          }
        }
        int kb0, kb1, b_off = 0;
        krange(ks, kb0, kb1);
        if (tp.group_mode == 1) {
          const int e = __ldg(tp.tile_expert + pm);
          if (e < 0) continue;
          b_off = e * tp.group_b_rows;
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, status, 0x101)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * Cfg::kStageBytes;
          uint8_t* sB = sA + Cfg::kABytes;
          const bool b_done = it < b_ahead;  // this stage's B half was requested before the dependency wait
          if (!b_done) mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, &full[s], kb * kBK, pm * kBM);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j) tma_load_2d(sA + j * 8192, &tmA, &full[s], pm * kBM + j * 64, kb * kBK);
          }
          if (b_done) continue;
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full[s], kb * kBK, pn * BN + b_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * 8192, &tmB, &full[s], pn * BN + j * 64, kb * kBK + b_off);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, A_MN, B_MN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int ks = tile / tiles_mn;
        int kb0, kb1;
        krange(ks, kb0, kb1);
        if (tp.group_mode == 1) {
          int pm, pn;
          tm.get(tile - ks * tiles_mn, pm, pn);
          if (__ldg(tp.tile_expert + pm) < 0) continue;
        }
        if (tp.group_mode && kb1 <= kb0) continue;
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        ++tcount;
        if (!mbar_wait(&tempty[acc], aph ^ 1, status, 0x201)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&full[s], ph, status, 0x202)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc =
                A_MN ? make_smem_desc(a_base + k * 2048, 8192, 1024) : make_smem_desc(a_base + k * 32, 0, 1024);
            const uint64_t bdesc =
                B_MN ? make_smem_desc(b_base + k * 2048, 8192, 1024) : make_smem_desc(b_base + k * 32, 0, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the smem stage once these MMAs retire
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue -----------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    int tcount = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      int pm, pn;
      const int ks = tile / tiles_mn;
      tm.get(tile - ks * tiles_mn, pm, pn);
      pm = rot(pm);
      if (tp.group_mode) {
        int kb0, kb1;
        krange(ks, kb0, kb1);
        if (kb1 <= kb0 || (tp.group_mode == 1 && __ldg(tp.tile_expert + pm) < 0)) continue;
      }
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      ++tcount;
      if (!mbar_wait(&tfull[acc], aph, status, 0x301)) break;
      tc_fence_after();
      const int row = pm * kBM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = pn * BN + c * 32;
        if (row < M && col0 < N) {
          const bool full_chunk = (col0 + 32 <= N);
          if (bias != nullptr && ks == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              const float b = (col < N) ? __bfloat162float(__ldg(bias + col)) : 0.f;
              r[j] = __float_as_uint(__uint_as_float(r[j]) + b);
            }
          }
          auto store_chunk = [&](void* cbase, long long elem_off) {
            if (out_mode == kOutBf16) {
              __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(cbase) + elem_off;
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
              float* crow = reinterpret_cast<float*>(cbase) + elem_off;
              const bool vec = full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
              if (vec) {
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                         __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                  if (out_mode == kOutF32Accum) {
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
                    if (out_mode == kOutF32Accum) o += crow[j];
                    crow[j] = o;
                  }
              }
            }
          };
          if (!SCATTER) {
            store_chunk(C, ks * split_stride + static_cast<long long>(row) * ldc + col0);
          } else if (tp.scatter_idx) {
            const int dest = __ldg(tp.idx_rank + row);
            if (dest >= 0) store_chunk(tp.dst[dest], static_cast<long long>(__ldg(tp.idx_row + row)) * ldc + col0);
          } else if (tp.scatter_cols) {
            int sg = 0, base = 0;
            if (tp.seg_w[1] > 0 && col0 >= tp.seg_start[1]) { sg = 1; base = tp.seg_w[0]; }
            if (tp.seg_w[2] > 0 && col0 >= tp.seg_start[2]) { sg = 2; base = tp.seg_w[0] + tp.seg_w[1]; }
            const int rel = col0 - tp.seg_start[sg];
            const int dest = rel / tp.seg_w[sg];
            store_chunk(tp.dst[dest], static_cast<long long>(tp.my_rank * tp.rows_per_rank + row) * ldc + base +
                                          (rel - dest * tp.seg_w[sg]));
          } else if (tp.scatter_all) {
            // all-reduce layout: every rank receives this rank's partial rows in slot my_rank
            // (with split-K, k slice ks of rank r fills slot r * splits + ks: the consumer adds n_ranks * splits slots)
            const long long off = (static_cast<long long>(tp.my_rank) * splits + ks) * tp.slot_stride +
                                  static_cast<long long>(row) * ldc + col0;
#pragma unroll 1
            for (int d = 0; d < tp.n_ranks; ++d) store_chunk(tp.dst[(tp.my_rank + d) % tp.n_ranks], off);
          } else {
            // reduce-scatter layout: the rows' owner receives them, at its local row index, in slot my_rank
            const int dest = row / tp.rows_per_rank;
            store_chunk(tp.dst[dest], tp.my_rank * tp.slot_stride +
                                          static_cast<long long>(row - dest * tp.rows_per_rank) * ldc + col0);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  } else if (GATHER) {
    // ------------------------------ copy warps (remote A shards -> local full buffer) ---------------
    // Work is handed out by a ticket counter so that whichever CTAs are resident finish every piece.
    const int bpr = (tp.gather_cols || tp.gather_idx) ? tm.m_blocks : tp.rows_per_rank / kBM;  // m-blocks per source rank
    const int total = (tp.gather_idx ? 1 : (tp.gather_cols ? tp.n_ranks : tp.n_ranks - 1)) * bpr * kPiecesPerBlock;
    const int vec_per_row = (tp.gather_cols ? tp.cols_per_rank : K) >> 3;   // 16-byte vectors per copied row
    constexpr int kRowsPerPiece = kBM / kPiecesPerBlock;
    unsigned int* ticket = tp.flags + tm.m_blocks;
    while (true) {
      int piece = 0;
      if (lane == 0) piece = static_cast<int>(atomicAdd(ticket, 1u));
      piece = __shfl_sync(0xffffffffu, piece, 0);
      if (piece >= total) break;
      const int bi = piece / kPiecesPerBlock, sub = piece - bi * kPiecesPerBlock;
      int src_rank, mb, row0, rows_here = kRowsPerPiece;
      const uint4* sp;
      uint4* dp;
      int ld_vec = static_cast<int>(tp.lda >> 3), sld_vec = ld_vec;
      if (tp.gather_idx) {
        // one table lookup per row: (rank, row) of the token routed to this expert slot
        mb = bi;
        row0 = mb * kBM + sub * kRowsPerPiece;
        rows_here = max(0, min(kRowsPerPiece, M - row0));
        sld_vec = static_cast<int>(tp.src_ld >> 3);
        for (int rr = 0; rr < rows_here; ++rr) {
          const int r = row0 + rr;
          const int sr = __ldg(tp.idx_rank + r);
          uint4* drow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(tp.a_full) + static_cast<long long>(r) * tp.lda);
          if (sr < 0) {  // padding row of an expert's last tile
            for (int c = lane; c < vec_per_row; c += 32) drow[c] = make_uint4(0, 0, 0, 0);
            continue;
          }
          const uint4* srow = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(tp.src[sr]) +
                                                             static_cast<long long>(__ldg(tp.idx_row + r)) * tp.src_ld);
          for (int base = 0; base < vec_per_row; base += 32 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = base + u * 32 + lane;
              if (c < vec_per_row) v[u] = srow[c];
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int c = base + u * 32 + lane;
              if (c < vec_per_row) drow[c] = v[u];
            }
          }
        }
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          atomicAdd(tp.flags + mb, 1u);
        }
        continue;
      }
      if (!tp.gather_cols) {
        src_rank = (tp.my_rank + 1 + bi / bpr) % tp.n_ranks;
        mb = src_rank * bpr + bi % bpr;
        row0 = mb * kBM + sub * kRowsPerPiece;  // row in the full matrix
        sp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(tp.src[src_rank]) +
                                            static_cast<long long>(row0 - src_rank * tp.rows_per_rank) * tp.lda);
        dp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(tp.a_full) + static_cast<long long>(row0) * tp.lda);
      } else {
        // m-blocks outermost so that the first blocks complete first; within a block, one source rank after another
        mb = bi / tp.n_ranks;
        src_rank = (tp.my_rank + bi % tp.n_ranks) % tp.n_ranks;  // the local block is copied the same way
        row0 = mb * kBM + sub * kRowsPerPiece;  // local row
        rows_here = max(0, min(kRowsPerPiece, M - row0));
        sld_vec = static_cast<int>(tp.src_ld >> 3);
        sp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(tp.src[src_rank]) +
                                            static_cast<long long>(tp.my_rank * tp.rows_per_rank + row0) * tp.src_ld);
        dp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(tp.a_full) + static_cast<long long>(row0) * tp.lda +
                                      static_cast<long long>(src_rank) * tp.cols_per_rank);
      }
      const int n_vec = rows_here * vec_per_row;
      for (int base = 0; base < n_vec; base += 32 * 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int idx = base + u * 32 + lane;
          if (idx < n_vec) {
            const int rr = idx / vec_per_row, cc = idx - rr * vec_per_row;
            v[u] = sp[static_cast<long long>(rr) * sld_vec + cc];
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int idx = base + u * 32 + lane;
          if (idx < n_vec) {
            const int rr = idx / vec_per_row, cc = idx - rr * vec_per_row;
            dp[static_cast<long long>(rr) * ld_vec + cc] = v[u];
          }
        }
      }
      fence_proxy_async_global();
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        atomicAdd(tp.flags + mb, 1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                       long long ldb, long long ldc, int out_mode, cudaStream_t stream, int splits = 1,
                       long long split_stride = 0, int prefetch_b = 0) {
  using Cfg = GemmCfg<BN>;
  const CUtensorMap* ta = A_MN ? get_tmap_bf16_2d(A, K, M, lda, 64) : get_tmap_bf16_2d(A, M, K, lda, kBM);
  const CUtensorMap* tb = B_MN ? get_tmap_bf16_2d(B, K, N, ldb, 64) : get_tmap_bf16_2d(B, N, K, ldb, BN);
  if (!ta || !tb) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  auto kfn = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN) * splits;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  const cudaError_t e = launch_pdl(kfn, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, *ta, *tb, C,
                                   reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, out_mode, splits, split_stride,
                                   device_status_ptr(), TpArgs{}, prefetch_b);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// Tensor-parallel launch: x @ W^T (B_MN = false) or dy @ W (B_MN = true) with the A operand gathered from peers
// and / or the output scattered to peers (see TpArgs).
template <int BN, bool B_MN, bool GATHER, bool SCATTER>
static int launch_gemm_tp(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int out_mode, const TpArgs& tp, cudaStream_t stream,
                          int b_groups = 1, int splits = 1) {
  using Cfg = GemmCfg<BN>;
  const CUtensorMap* ta = get_tmap_bf16_2d(A, M, K, lda, kBM);
  const CUtensorMap* tb = B_MN ? get_tmap_bf16_2d(B, static_cast<long long>(K) * b_groups, N, ldb, 64)
                               : get_tmap_bf16_2d(B, static_cast<long long>(N) * b_groups, K, ldb, BN);
  if (!ta || !tb) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  auto kfn = gemm_bf16_kernel<BN, false, B_MN, GATHER, SCATTER>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  const int m_blocks = (M + kBM - 1) / kBM;
  const int tiles = m_blocks * ((N + BN - 1) / BN) * splits;
  if (GATHER) {
    // piece counters and the ticket start at zero for every launch
    if (cudaMemsetAsync(tp.flags, 0, sizeof(unsigned int) * (m_blocks + 1), stream) != cudaSuccess) return SB_ERR_CUDA;
  }
  // with GATHER every CTA also carries copy warps, so launch the full machine even for few tiles
  const int grid = GATHER ? sm_count() : (tiles < sm_count() ? tiles : sm_count());
  const int threads = kGemmThreads + (GATHER ? kGatherWarps * 32 : 0);
  if (!GATHER) {
    // scatter modes sit in the decode chain of tensor-parallel engines: let the prologue (barrier set-up, tensor
    // memory allocation) overlap the tail of the preceding kernel; every operand access comes after pdl_wait()
    const cudaError_t e = launch_pdl(kfn, dim3(grid), dim3(threads), Cfg::kSmemBytes, stream, *ta, *tb, C,
                                     reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, out_mode, splits, 0LL,
                                     device_status_ptr(), tp, 0);
    return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
  }
  kfn<<<grid, threads, Cfg::kSmemBytes, stream>>>(*ta, *tb, C, reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc,
                                                  out_mode, 1, 0, device_status_ptr(), tp, 0);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// Grouped launch (see TpArgs::group_mode).  mode 1: A [M, K] with row blocks owned by experts, B = n_groups stacked
// matrices ([N, K] each when !B_MN, [K, N] each when B_MN).  mode 2: A [rows, M] and B [rows, N], both MN-major,
// C = n_groups stacked [M, N] results.
template <int BN, bool A_MN, bool B_MN>
static int launch_gemm_grouped(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                               long long ldc, int out_mode, int mode, int n_groups, const int* tile_expert,
                               const int* k_off, long long group_c_stride, int rows_total, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  const CUtensorMap* ta;
  const CUtensorMap* tb;
  TpArgs tp{};
  tp.group_mode = mode;
  tp.tile_expert = tile_expert;
  tp.k_off = k_off;
  int splits = 1;
  if (mode == 1) {
    ta = get_tmap_bf16_2d(A, M, K, lda, kBM);
    tb = B_MN ? get_tmap_bf16_2d(B, static_cast<long long>(n_groups) * K, N, ldb, 64)
              : get_tmap_bf16_2d(B, static_cast<long long>(n_groups) * N, K, ldb, BN);
    tp.group_b_rows = B_MN ? K : N;
  } else {
    ta = get_tmap_bf16_2d(A, rows_total, M, lda, 64);
    tb = get_tmap_bf16_2d(B, rows_total, N, ldb, 64);
    splits = n_groups;
  }
  if (!ta || !tb) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  auto kfn = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  const long long tiles = static_cast<long long>((M + kBM - 1) / kBM) * ((N + BN - 1) / BN) * splits;
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  const cudaError_t e = launch_pdl(kfn, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, *ta, *tb, C,
                                   static_cast<const __nv_bfloat16*>(nullptr), M, N, K, ldc, out_mode, splits,
                                   group_c_stride, device_status_ptr(), tp, 0);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

template <bool A_MN, bool B_MN>
static int dispatch_bn(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                       long long ldb, long long ldc, int out_mode, int bn_hint, cudaStream_t stream, int prefetch_b = 0) {
  int bn = bn_hint;
  if (bn != 64 && bn != 128 && bn != 256) {
    const long long mb = (M + kBM - 1) / kBM;
    const int sms = sm_count();
    if (mb * ((N + 255) / 256) >= sms || N >= 4096)
      bn = 256;
    else if (mb * ((N + 127) / 128) >= sms / 2)
      bn = 128;
    else
      bn = 64;
  }
  if (bn == 256) return launch_gemm<256, A_MN, B_MN>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, stream, 1, 0, prefetch_b);
  if (bn == 128) return launch_gemm<128, A_MN, B_MN>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, stream, 1, 0, prefetch_b);
  return launch_gemm<64, A_MN, B_MN>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, stream, 1, 0, prefetch_b);
}

}  // namespace sb

extern "C" int sb_gemm_bf16_2cta(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, int a_mn, int b_mn, int out_mode, int bn, void* stream);

namespace sb {
// Large problems run on CTA pairs (256 x 256 tiles, half of the B tile per SM): measured 7-22% faster than the
// one-CTA kernel on training shapes.  Small / skinny problems keep the one-CTA kernel (finer tiles, split-K).
// SB_GEMM_PAIR=0 in the environment disables the pair kernel (A/B comparisons).
static bool pair_kernel_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB_GEMM_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
static bool use_pair_kernel(int M, int N, int K, int bn_hint) {
  if (!pair_kernel_enabled() || bn_hint != 0) return false;
  if (M < 512 || N < 256 || K < 256) return false;
  const long long tiles = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256);
  return tiles >= 56;  // at least ~3/4 of the 74 SM pairs busy in the first wave
}
}  // namespace sb

extern "C" {

// C[M,N] = op(A) * op(B) (+ bias[N]).  a_mn / b_mn select the operand layouts described at the
// top of this file; out_mode: 0 = bf16 store, 1 = fp32 store, 2 = fp32 accumulate into C.
// lda/ldb/ldc are row strides in elements of the stored matrices. bn_hint 0 = automatic tile width.
int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int a_mn, int b_mn, int out_mode, int bn_hint, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return SB_ERR_ARG;
  if ((lda & 7) || (ldb & 7)) return SB_ERR_ARG;
  if (out_mode < 0 || out_mode > 2) return SB_ERR_ARG;
  // bit 12 of bn_hint: the B operand is constant data (weights), its first tiles may be fetched ahead of the
  // dependency wait of a programmatic dependent launch
  const int prefetch_b = (bn_hint >> 12) & 1;
  bn_hint &= 0xFFF;
  if (sb::use_pair_kernel(M, N, K, bn_hint))
    return sb_gemm_bf16_2cta(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, 256, stream);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return sb::dispatch_bn<false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, bn_hint, st, prefetch_b);
  if (!a_mn && b_mn) return sb::dispatch_bn<false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, bn_hint, st);
  if (a_mn && b_mn) return sb::dispatch_bn<true, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, bn_hint, st);
  return sb::dispatch_bn<true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, bn_hint, st);
}


// Grouped products for mixture-of-experts layers; every table is device memory.
//   mode 1, b_mn = 0: C[r, :] = A[r, :] * B[e(r)]^T   A [M, K], B [n_groups, N, K], C [M, N]; tile_expert[M / 128]
//   mode 1, b_mn = 1: C[r, :] = A[r, :] * B[e(r)]     A [M, K], B [n_groups, K, N], C [M, N]
//   mode 2:           C[e] (+)= A[rows_e, :]^T * B[rows_e, :]   A [rows, M], B [rows, N], C [n_groups, M, N];
//                     rows_e = [k_off[e], k_off[e + 1]), multiples of 64; experts without rows leave C[e] untouched.
// M of mode 1 must be a multiple of 128 (whole row blocks).
int sb_gemm_grouped(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                    int b_mn, int out_mode, int mode, int n_groups, const int* tile_expert, const int* k_off,
                    long long group_c_stride, int rows_total, void* stream) {
  if (M <= 0 || N <= 0 || n_groups <= 0 || (lda & 7) || (ldb & 7) || out_mode < 0 || out_mode > 2) return SB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mode == 1) {
    if (K <= 0 || (M % sb::kBM) != 0 || !tile_expert) return SB_ERR_ARG;
    const bool wide = N >= 256;
    if (!b_mn) {
      return wide ? sb::launch_gemm_grouped<256, false, false>(A, B, C, M, N, K, lda, ldb, ldc, out_mode, 1, n_groups,
                                                               tile_expert, nullptr, 0, 0, st)
                  : sb::launch_gemm_grouped<128, false, false>(A, B, C, M, N, K, lda, ldb, ldc, out_mode, 1, n_groups,
                                                               tile_expert, nullptr, 0, 0, st);
    }
    return wide ? sb::launch_gemm_grouped<256, false, true>(A, B, C, M, N, K, lda, ldb, ldc, out_mode, 1, n_groups,
                                                            tile_expert, nullptr, 0, 0, st)
                : sb::launch_gemm_grouped<128, false, true>(A, B, C, M, N, K, lda, ldb, ldc, out_mode, 1, n_groups,
                                                            tile_expert, nullptr, 0, 0, st);
  }
  if (mode == 2) {
    if (!k_off || rows_total <= 0 || (rows_total % sb::kBK) != 0) return SB_ERR_ARG;
    return N >= 256 ? sb::launch_gemm_grouped<256, true, true>(A, B, C, M, N, rows_total, lda, ldb, ldc, out_mode, 2,
                                                               n_groups, nullptr, k_off, group_c_stride, rows_total, st)
                    : sb::launch_gemm_grouped<128, true, true>(A, B, C, M, N, rows_total, lda, ldb, ldc, out_mode, 2,
                                                               n_groups, nullptr, k_off, group_c_stride, rows_total, st);
  }
  return SB_ERR_ARG;
}

// Split-K product for skinny problems (decode: M <= a few hundred rows): x[M,K] * W[N,K]^T as `splits` fp32
// partial sums, partial s at C + s * split_stride (row stride ldc).  `splits` is clamped so that no slice is
// empty; the value used is returned through splits_used.  bias (optional) is added into partial 0.
int sb_gemm_bf16_splitk(const void* A, const void* B, float* C, const void* bias, int M, int N, int K, long long lda,
                        long long ldb, long long ldc, long long split_stride, int splits, int bn, int* splits_used,
                        void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || splits < 1) return SB_ERR_ARG;
  const int k_blocks = (K + sb::kBK - 1) / sb::kBK;
  if (splits > k_blocks) splits = k_blocks;
  int kpb = (k_blocks + splits - 1) / splits;
  splits = (k_blocks + kpb - 1) / kpb;
  if (splits_used) *splits_used = splits;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // B is a weight matrix here by contract (decode projections): its first tiles are prefetched ahead of the wait
  if (bn == 256) return sb::launch_gemm<256, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, 1, st, splits, split_stride, 1);
  if (bn == 128) return sb::launch_gemm<128, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, 1, st, splits, split_stride, 1);
  return sb::launch_gemm<64, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, 1, st, splits, split_stride, 1);
}


// Tensor-parallel GEMM with the collective inside the kernel.
//   gather != 0 : A is the full [M, K] buffer on this GPU whose rows [r*rows_per_rank, (r+1)*rows_per_rank) belong to
//                 rank r; peers[r] points at rank r's own shard (in rank r's memory).  The kernel copies the remote
//                 shards in while it computes (all-gather fused into the GEMM).  flags: (M/128 + 1) uint32 of scratch.
//                 M must equal n_ranks * rows_per_rank and rows_per_rank must be a multiple of 128.
//   scatter = 1 : C rows are stored to their owner rank's buffer outs[row / rows_per_rank] at slot my_rank
//                 (reduce-scatter layout; the owner adds the n_ranks slots), scatter = 2: to every rank (all-reduce).
//   b_mn selects W stored [N, K] (0) or [K, N] (1).  out_mode 0 = bf16, 1 = fp32.
int sb_gemm_tp(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda, long long ldb,
               long long ldc, int b_mn, int out_mode, int gather, int scatter, const void* const* peers,
               void* const* outs, int n_ranks, int my_rank, int rows_per_rank, long long slot_stride,
               unsigned int* flags, int bn, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || (K & 7)) return SB_ERR_ARG;
  if (n_ranks < 1 || n_ranks > sb::kTpMaxRanks || my_rank < 0 || my_rank >= n_ranks || rows_per_rank <= 0) return SB_ERR_ARG;
  if (out_mode != 0 && out_mode != 1) return SB_ERR_ARG;
  if (!gather && !scatter) return SB_ERR_ARG;
  sb::TpArgs tp{};
  tp.n_ranks = n_ranks;
  tp.my_rank = my_rank;
  tp.rows_per_rank = rows_per_rank;
  tp.lda = lda;
  tp.slot_stride = slot_stride;
  tp.scatter_all = scatter == 2;
  if (gather) {
    if (!peers || !flags || rows_per_rank % sb::kBM != 0 || M != n_ranks * rows_per_rank) return SB_ERR_ARG;
    for (int r = 0; r < n_ranks; ++r) {
      if (!peers[r] || (reinterpret_cast<uintptr_t>(peers[r]) & 15)) return SB_ERR_ARG;
      tp.src[r] = peers[r];
    }
    tp.a_full = const_cast<void*>(A);
    tp.flags = flags;
  }
  if (scatter) {
    if (!outs) return SB_ERR_ARG;
    if (scatter == 1 && M > n_ranks * rows_per_rank) return SB_ERR_ARG;
    for (int r = 0; r < n_ranks; ++r) {
      if (!outs[r]) return SB_ERR_ARG;
      tp.dst[r] = outs[r];
    }
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn != 128 && bn != 256) bn = (static_cast<long long>((M + 127) / 128) * ((N + 255) / 256) >= sb::sm_count()) ? 256 : 128;
#define SB_TP_CASE(BNV, BMN, G, S)                                                                                   \
  if (bn == BNV && (b_mn != 0) == BMN && (gather != 0) == G && (scatter != 0) == S)                                  \
    return sb::launch_gemm_tp<BNV, BMN, G, S>(A, B, C, bias, M, N, K, lda, ldb, ldc, out_mode, tp, st);
  SB_TP_CASE(128, false, true, false)
  SB_TP_CASE(256, false, true, false)
  SB_TP_CASE(128, true, true, false)
  SB_TP_CASE(256, true, true, false)
  SB_TP_CASE(128, false, false, true)
  SB_TP_CASE(256, false, false, true)
  SB_TP_CASE(128, true, false, true)
  SB_TP_CASE(256, true, false, true)
#undef SB_TP_CASE
  return SB_ERR_ARG;
}

// Row-parallel projection of a tensor-parallel decode step: x[M, K_local] @ W[N, K_local]^T as fp32 split-K partial
// sums stored from the epilogue into EVERY rank's slot buffer (all-reduce layout).  Slot (my_rank * splits + ks) of
// each destination receives k slice ks; a consumer (fused residual + RMSNorm) adds the n_ranks * splits slots after a
// barrier.  Split-K is what lets a skinny projection (M <= 256 rows) stream its weights with all SMs.
int sb_gemm_tp_scatter_splitk(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                              void* const* outs, int n_ranks, int my_rank, long long slot_stride, int splits,
                              void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || (K & 7) || !outs) return SB_ERR_ARG;
  if (n_ranks < 1 || n_ranks > sb::kTpMaxRanks || my_rank < 0 || my_rank >= n_ranks) return SB_ERR_ARG;
  const int k_blocks = (K + sb::kBK - 1) / sb::kBK;
  if (splits < 1 || splits > k_blocks) return SB_ERR_ARG;
  const int kpb = (k_blocks + splits - 1) / splits;
  if ((k_blocks + kpb - 1) / kpb != splits) return SB_ERR_ARG;  // an empty slice would leave its slot unwritten
  sb::TpArgs tp{};
  tp.n_ranks = n_ranks;
  tp.my_rank = my_rank;
  tp.rows_per_rank = M;
  tp.lda = lda;
  tp.slot_stride = slot_stride;
  tp.scatter_all = 1;
  for (int r = 0; r < n_ranks; ++r) {
    if (!outs[r]) return SB_ERR_ARG;
    tp.dst[r] = outs[r];
  }
  return sb::launch_gemm_tp<128, false, false, true>(A, B, nullptr, nullptr, M, N, K, lda, ldb, N, 1, tp,
                                                     reinterpret_cast<cudaStream_t>(stream), 1, splits);
}


// Projections around sequence-parallel attention with the all-to-all inside the GEMM kernel (x @ W^T, W stored [N, K]).
//   mode 1 (scatter columns): x is this rank's [M = rows_per_rank, K] token shard; output column segments
//       (seg_start[i], seg_w[i] per rank, i < 3: q | k | v heads) are stored to the rank owning those heads, into its
//       [n_ranks * rows_per_rank, sum(seg_w)] buffer peers[dest] at rows my_rank * rows_per_rank + row.
//   mode 2 (gather columns): A is this rank's [M, K = n_ranks * cols_per_rank] buffer; column block r is copied from
//       peers[r] (rank r's [n_ranks * rows_per_rank, cols_per_rank] attention output, row stride src_ld), rows
//       my_rank * rows_per_rank + [0, M), while the GEMM runs; C is a plain local output.
int sb_gemm_sp(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda, long long ldb,
               long long ldc, int mode, void* const* peers, int n_ranks, int my_rank, int rows_per_rank,
               const int* seg_start, const int* seg_w, int cols_per_rank, long long src_ld, unsigned int* flags, int bn,
               void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || (K & 7) || !peers) return SB_ERR_ARG;
  if (n_ranks < 1 || n_ranks > sb::kTpMaxRanks || my_rank < 0 || my_rank >= n_ranks || M > rows_per_rank) return SB_ERR_ARG;
  sb::TpArgs tp{};
  tp.n_ranks = n_ranks;
  tp.my_rank = my_rank;
  tp.rows_per_rank = rows_per_rank;
  tp.lda = lda;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn != 128 && bn != 256) bn = 128;
  if (mode == 1) {
    if (!seg_start || !seg_w) return SB_ERR_ARG;
    int covered = 0;
    for (int i = 0; i < 3; ++i) {
      tp.seg_start[i] = seg_start[i];
      tp.seg_w[i] = seg_w[i];
      if (seg_w[i] < 0 || (seg_w[i] & 31) || (seg_start[i] & 31)) return SB_ERR_ARG;  // chunks of 32 columns stay whole
      covered += seg_w[i] * n_ranks;
    }
    if (covered != N || seg_w[0] == 0) return SB_ERR_ARG;
    tp.scatter_cols = 1;
    for (int r = 0; r < n_ranks; ++r) {
      if (!peers[r]) return SB_ERR_ARG;
      tp.dst[r] = peers[r];
    }
    if (bn == 256) return sb::launch_gemm_tp<256, false, false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, tp, st);
    return sb::launch_gemm_tp<128, false, false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, tp, st);
  }
  if (mode == 2) {
    if (!flags || cols_per_rank <= 0 || (cols_per_rank & 7) || K != n_ranks * cols_per_rank || (src_ld & 7)) return SB_ERR_ARG;
    tp.gather_cols = 1;
    tp.cols_per_rank = cols_per_rank;
    tp.src_ld = src_ld;
    tp.a_full = const_cast<void*>(A);
    tp.flags = flags;
    for (int r = 0; r < n_ranks; ++r) {
      if (!peers[r] || (reinterpret_cast<uintptr_t>(peers[r]) & 15)) return SB_ERR_ARG;
      tp.src[r] = peers[r];
    }
    if (bn == 256) return sb::launch_gemm_tp<256, false, true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, tp, st);
    return sb::launch_gemm_tp<128, false, true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, 0, tp, st);
  }
  return SB_ERR_ARG;
}


// Expert GEMM with the token exchange inside the kernel (x @ W^T with W [N, K], or x @ W with W [K, N] when b_mn).
//   mode 1 (dispatch): A row r is fetched from row idx_row[r] of peers[idx_rank[r]] (row stride src_ld) into the local
//       buffer A while the GEMM runs; C is a plain local output.  flags: (M/128 + 2) uint32 of scratch.
//   mode 2 (combine): A is local; C row r is stored to row idx_row[r] of peers[idx_rank[r]] (row stride ldc).
// n_groups > 0: the rows are grouped by expert in 128-row tiles (tile_expert[M / 128], -1 = unused tile), B holds
// n_groups stacked matrices and rows whose idx_rank is negative are padding (zero on dispatch, not stored on combine).
int sb_gemm_ep_grouped(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int b_mn, int mode, void* const* peers, int n_ranks, int my_rank,
                       const int* idx_rank, const int* idx_row, long long src_ld, unsigned int* flags, int bn,
                       int n_groups, const int* tile_expert, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || (K & 7) || !peers || !idx_rank || !idx_row) return SB_ERR_ARG;
  if (n_ranks < 1 || n_ranks > sb::kTpMaxRanks || my_rank < 0 || my_rank >= n_ranks) return SB_ERR_ARG;
  if (n_groups > 0 && (!tile_expert || (M % sb::kBM) != 0)) return SB_ERR_ARG;
  const int bg = n_groups > 0 ? n_groups : 1;
  sb::TpArgs tp{};
  if (n_groups > 0) {
    tp.group_mode = 1;
    tp.tile_expert = tile_expert;
    tp.group_b_rows = b_mn ? K : N;
  }
  tp.n_ranks = n_ranks;
  tp.my_rank = my_rank;
  tp.rows_per_rank = M;
  tp.lda = lda;
  tp.idx_rank = idx_rank;
  tp.idx_row = idx_row;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn != 128 && bn != 256) bn = 128;
  if (mode == 1) {
    if (!flags || (src_ld & 7)) return SB_ERR_ARG;
    tp.gather_idx = 1;
    tp.src_ld = src_ld;
    tp.a_full = const_cast<void*>(A);
    tp.flags = flags;
    for (int r = 0; r < n_ranks; ++r) {
      if (!peers[r] || (reinterpret_cast<uintptr_t>(peers[r]) & 15)) return SB_ERR_ARG;
      tp.src[r] = peers[r];
    }
    if (b_mn) {
      if (bn == 256) return sb::launch_gemm_tp<256, true, true, false>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
      return sb::launch_gemm_tp<128, true, true, false>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
    }
    if (bn == 256) return sb::launch_gemm_tp<256, false, true, false>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
    return sb::launch_gemm_tp<128, false, true, false>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
  }
  if (mode == 2) {
    tp.scatter_idx = 1;
    for (int r = 0; r < n_ranks; ++r) {
      if (!peers[r]) return SB_ERR_ARG;
      tp.dst[r] = peers[r];
    }
    if (b_mn) {
      if (bn == 256) return sb::launch_gemm_tp<256, true, false, true>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
      return sb::launch_gemm_tp<128, true, false, true>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
    }
    if (bn == 256) return sb::launch_gemm_tp<256, false, false, true>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
    return sb::launch_gemm_tp<128, false, false, true>(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, tp, st, bg);
  }
  return SB_ERR_ARG;
}

int sb_gemm_ep(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
               int b_mn, int mode, void* const* peers, int n_ranks, int my_rank, const int* idx_rank, const int* idx_row,
               long long src_ld, unsigned int* flags, int bn, void* stream) {
  return sb_gemm_ep_grouped(A, B, C, M, N, K, lda, ldb, ldc, b_mn, mode, peers, n_ranks, my_rank, idx_rank, idx_row, src_ld,
                            flags, bn, 0, nullptr, stream);
}

}  // extern "C"
