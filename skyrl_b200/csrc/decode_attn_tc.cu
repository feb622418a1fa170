// Paged-KV decode attention on TMA + tcgen05 (head dim 128, up to 16 query heads per KV head).
//
// Decode attention is a pure streaming problem: every K and V row of the context is read once.
// One CTA handles (sequence, KV head, context split).  A producer thread walks the block table and
// issues one TMA box per cache page, filling 128-token K and V tiles in a 3-stage shared-memory
// ring (192 KB in flight per SM).  The products are transposed so that the *token* axis is the
// tensor-core M dimension:
//     S^T[128 tok, 16 heads] = K_tile[128, 128] * Q^T        (K-major A, K-major B)
//     O^T[128 d,   16 heads] = V_tile^T[128 d, 128 tok] * P   (MN-major A straight from the row-major V tile)
// Softmax runs over TMEM lanes: each of the 128 softmax threads owns one token of the tile, the
// per-head maximum is a warp shuffle + one shared-memory exchange, exponent sums stay per-thread until
// the end.  O^T is folded into per-thread fp32 accumulators (thread = output dimension).
#include <cstdlib>

#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kDtThreads = 192;
constexpr int kDtThreadsPersist = 224;  // + one warp streaming the V tiles
constexpr int kDtStages = 3;
constexpr int kDtTile = 128 * 128 * 2;                 // one K or V tile: 32 KB (two 16 KB halves)
constexpr int kDtStageBytes = 2 * kDtTile;             // K + V
constexpr int kDtQBytes = 2 * 16 * 128;                // Q^T operand: two [16 x 128 B] halves
constexpr int kDtPBytes = 2 * 16 * 128;                // P operand:   two [16 x 128 B] halves
constexpr int kDtSmem = kDtStages * kDtStageBytes + kDtQBytes + kDtPBytes + 1024 + 512;
constexpr int kDtSmemPersist = kDtSmem + kDtPBytes;  // second P buffer

__device__ __forceinline__ float dt_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int G>
__global__ void __launch_bounds__(kDtThreads, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ block_tables,
                      const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ ws, int nq,
                      int nkv, int block_size, int max_blocks, int splits, long long q_stride, float scale_log2,
                      int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + kDtStages * kDtStageBytes;
  uint8_t* sP = sQ + kDtQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kDtPBytes);
  uint64_t* full = bars;               // [3]
  uint64_t* empty = bars + 3;          // [3]
  uint64_t* s_full = bars + 6;         // [2]
  uint64_t* p_ready = bars + 8;
  uint64_t* o_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  __shared__ float s_red[4][16];
  __shared__ float s_lsum[4][16];

  const int seq = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();  // q, the cache rows of this step and ctx_lens come from the preceding kernels
  const int ctx = ctx_lens[seq];
  const int per_split = (((ctx + splits - 1) / splits) + 127) & ~127;
  const int t0 = split * per_split;
  const int t1 = min(ctx, t0 + per_split);
  const int n_tiles = (t1 > t0) ? (t1 - t0 + 127) / 128 : 0;

  if (n_tiles == 0) {
    // nothing in this split (or an inactive slot): emit neutral results
    if (threadIdx.x < 128) {
      const int d = threadIdx.x;
      for (int h = 0; h < G; ++h) {
        const size_t head = static_cast<size_t>(seq) * nq + g * G + h;
        if (splits == 1) {
          out[head * 128 + d] = __float2bfloat16(0.f);
        } else {
          float* w = ws + (head * splits + split) * 130;
          w[d] = 0.f;
          if (d == 0) {
            w[128] = -INFINITY;
            w[129] = 0.f;
          }
        }
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDtStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_ready, 4);
    mbar_init(o_full, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  // Q^T operand and the zero rows of P: written once by the softmax warps (generic proxy)
  if (warp >= 2) {
    const int t = threadIdx.x - 64;  // 0..127
    // zero both small operand tiles (4 KB + 4 KB = 512 x 16 B)
    for (int i = t; i < (kDtQBytes + kDtPBytes) / 16; i += 128) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  if (warp >= 2) {
    const int t = threadIdx.x - 64;
    // G heads x 128 dims = G x 16 chunks of 8 bf16
    for (int i = t; i < G * 16; i += 128) {
      const int h = i >> 4, c = i & 15;  // c: 16-byte chunk along d (0..15)
      const uint4 v = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(seq) * q_stride + (g * G + h) * 128 + c * 8);
      const int half = c >> 3, cc = c & 7;
      *reinterpret_cast<uint4*>(sQ + half * 2048 + h * 128 + ((cc ^ (h & 7)) << 4)) = v;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const int* bt = block_tables + static_cast<size_t>(seq) * max_blocks;
  const int pages_per_tile = 128 / block_size;

  if (warp == 0) {
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kDtStages;
        if (!mbar_wait(&empty[s], ((j / kDtStages) & 1) ^ 1, status, 0x801)) break;
        uint8_t* sK = smem + s * kDtStageBytes;
        uint8_t* sV = sK + kDtTile;
        mbar_arrive_expect_tx(&full[s], kDtStageBytes);
        const int tok0 = t0 + j * 128;
        for (int p = 0; p < pages_per_tile; ++p) {
          int pi = (tok0 + p * block_size) / block_size;
          pi = pi < max_blocks ? pi : max_blocks - 1;
          const int slot0 = bt[pi] * block_size;
          const int off = p * block_size * 128;
          tma_load_3d(sK + off, &tm_k, &full[s], 0, g, slot0);
          tma_load_3d(sK + 16384 + off, &tm_k, &full[s], 64, g, slot0);
          tma_load_3d(sV + off, &tm_v, &full[s], 0, g, slot0);
          tma_load_3d(sV + 16384 + off, &tm_v, &full[s], 64, g, slot0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 16, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 16, true, false);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int s = j % kDtStages;
        if (!mbar_wait(&full[s], (j / kDtStages) & 1, status, 0x811)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(smem + s * kDtStageBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16(tmem_base + (j & 1) * 16, make_smem_desc(k_base + (k >> 2) * 16384 + (k & 3) * 32, 0, 1024),
                   make_smem_desc(q_base + (k >> 2) * 2048 + (k & 3) * 32, 0, 1024), idesc_s, k != 0);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      bool ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        if (!mbar_wait(p_ready, j & 1, status, 0x812)) break;
        tc_fence_after();
        const int s = j % kDtStages;
        const uint32_t v_base = smem_u32(smem + s * kDtStageBytes + kDtTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16(tmem_base + 32, make_smem_desc(v_base + k * 2048, 16384, 1024),
                   make_smem_desc(p_base + (k >> 2) * 2048 + (k & 3) * 32, 0, 1024), idesc_o, k != 0);
        umma_commit(o_full);
        umma_commit(&empty[s]);
      }
    }
  } else {
    const int q = warp & 3;
    const int sw = warp - 2;
    const int r = q * 32 + lane;  // token within the tile (S^T phase) and output dimension (O^T phase)
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float m[G], lsum[G], O[G], alpha_prev[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      m[h] = -INFINITY;
      lsum[h] = 0.f;
      O[h] = 0.f;
      alpha_prev[h] = 1.f;
    }
    bool ok = true;
    auto fold_o = [&](int j) -> bool {
      if (!mbar_wait(o_full, j & 1, status, 0x821)) return false;
      tc_fence_after();
      uint32_t v[16];
      tmem_ld_32x32b_x16(tmem_base + 32 + lane_off, v);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < G; ++h) O[h] = O[h] * alpha_prev[h] + __uint_as_float(v[h]);
      return true;
    };
    // Every thread executes the same number of named barriers whatever happens: after a failed wait the
    // remaining waits are skipped (ok == false) but the loop structure is kept, so nobody is left behind.
    for (int j = 0; j < n_tiles; ++j) {
      if (ok) ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, status, 0x820);
      tc_fence_after();
      uint32_t v[16];
      tmem_ld_32x32b_x16(tmem_base + (j & 1) * 16 + lane_off, v);
      tmem_ld_wait();
      const bool valid = (t0 + j * 128 + r) < t1;
      float s[G];
#pragma unroll
      for (int h = 0; h < G; ++h) {
        s[h] = valid ? __uint_as_float(v[h]) * scale_log2 : -INFINITY;
        float mx = warp_max(s[h]);
        if (lane == 0) s_red[sw][h] = mx;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float alpha[G];
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float tile_max = fmaxf(fmaxf(s_red[0][h], s_red[1][h]), fmaxf(s_red[2][h], s_red[3][h]));
        const float mn = fmaxf(m[h], tile_max);
        alpha[h] = dt_exp2(m[h] - mn);  // first tile: exp2(-inf) = 0
        s[h] = valid ? dt_exp2(s[h] - mn) : 0.f;
        lsum[h] = lsum[h] * alpha[h] + s[h];
        m[h] = mn;
      }
      if (j > 0 && ok) ok = fold_o(j - 1);
      // P as K-major B operand: row = head, column = token of the tile
      {
        const int half = r >> 6, col = r & 63;
        uint8_t* base = sP + half * 2048 + (col & 7) * 2;
        const int chunk = col >> 3;
#pragma unroll
        for (int h = 0; h < G; ++h)
          *reinterpret_cast<__nv_bfloat16*>(base + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16(s[h]);
      }
#pragma unroll
      for (int h = 0; h < G; ++h) alpha_prev[h] = alpha[h];
      fence_proxy_async_smem();
      tc_fence_before();
      // second barrier: s_red may be overwritten by the next tile only after everyone has read it
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok) ok = fold_o(n_tiles - 1);
    // total exponent sum per head over the 128 token owners
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float t = warp_sum(lsum[h]);
      if (lane == 0) s_lsum[sw][h] = t;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (ok) {
      const int d = r;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float l = s_lsum[0][h] + s_lsum[1][h] + s_lsum[2][h] + s_lsum[3][h];
        const size_t head = static_cast<size_t>(seq) * nq + g * G + h;
        if (splits == 1) {
          out[head * 128 + d] = __float2bfloat16(l > 0.f ? O[h] / l : 0.f);
        } else {
          float* w = ws + (head * splits + split) * 130;
          w[d] = O[h];
          if (d == 0) {
            w[128] = m[h];
            w[129] = l;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 64);
}

// Persistent variant: one CTA per SM walks a list of (sequence, KV head, context split) items.  The TMA producer and
// the MMA issuer run ahead across item boundaries (the K/V ring, the TMEM buffers and every barrier phase are indexed
// by a tile counter that keeps counting), so the next item's first tiles are in flight while the softmax warps finish
// the current one, and the per-CTA prologue (barrier init, TMEM allocation) is paid once per SM instead of once per
// item.  The query operand is handed over inside the last tile of an item: as soon as the softmax warps have seen the
// last S^T product of the item complete, no MMA reads sQ any more and they store the next item's query rows (already
// fetched into registers) before they continue with that tile.
template <int G>
__global__ void __launch_bounds__(kDtThreadsPersist, 1)
attn_decode_tc_persist_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                              const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ block_tables,
                              const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ ws,
                              int n_seqs, int nq, int nkv, int block_size, int max_blocks, int splits, long long q_stride,
                              float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + kDtStages * kDtStageBytes;
  uint8_t* sP = sQ + kDtQBytes;
  // P and the O^T accumulator are double-buffered: the softmax warps store P(j) without waiting for the product of
  // tile j-1, whose result they fold afterwards
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kDtPBytes);
  // K and V tiles travel through rings of their own: a K tile is free again as soon as its S^T product has completed,
  // a whole tile period before the V tile of the same step, so its refill starts that much earlier
  uint64_t* kfull = bars;              // [3]
  uint64_t* kempty = bars + 3;         // [3]
  uint64_t* vfull = bars + 6;          // [3]
  uint64_t* vempty = bars + 9;         // [3]
  uint64_t* s_full = bars + 12;        // [2]
  uint64_t* p_ready = bars + 14;       // [2] (two barriers: the softmax warps may be a whole tile ahead of the issuer)
  uint64_t* o_full = bars + 16;        // [2]
  uint64_t* q_ready = bars + 18;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  __shared__ float s_red[4][16];
  __shared__ float s_lsum[4][16];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = n_seqs * nkv * splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDtStages; ++i) {
      mbar_init(&kfull[i], 1);
      mbar_init(&kempty[i], 1);
      mbar_init(&vfull[i], 1);
      mbar_init(&vempty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_ready[0], 4);
    mbar_init(&p_ready[1], 4);
    mbar_init(&o_full[0], 1);
    mbar_init(&o_full[1], 1);
    mbar_init(q_ready, 4);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  if (warp >= 2 && warp < 6) {
    const int t = threadIdx.x - 64;  // rows of heads >= G stay zero for the whole kernel
    for (int i = t; i < (kDtQBytes + 2 * kDtPBytes) / 16; i += 128) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  pdl_launch_dependents();
  pdl_wait();  // q, the cache rows of this step and ctx_lens come from the preceding kernels

  // item -> (sequence, kv head, split) and its token range; identical arithmetic in every role
  auto item_range = [&](int item, int& seq, int& g, int& split, int& t0, int& t1) -> int {
    split = item % splits;
    const int sg = item / splits;
    g = sg % nkv;
    seq = sg / nkv;
    const int ctx = __ldg(ctx_lens + seq);
    const int per_split = (((ctx + splits - 1) / splits) + 127) & ~127;
    t0 = split * per_split;
    t1 = min(ctx, t0 + per_split);
    return (t1 > t0) ? (t1 - t0 + 127) / 128 : 0;
  };
  auto next_work = [&](int item) -> int {  // first item >= `item` of this CTA's list that has tiles (n_items: none)
    for (; item < n_items; item += gridDim.x) {
      int a, b, c, d, e;
      if (item_range(item, a, b, c, d, e) > 0) return item;
    }
    return n_items;
  };
  const int pages_per_tile = 128 / block_size;

  if (warp == 0 || warp == 6) {
    // Warp 0 streams the K tiles, warp 6 the V tiles.  Lane 0 waits for a free stage; the boxes of the tile (one per
    // cache page and head-dim half, 4 KB each with 32-token pages) are then issued by as many lanes in one warp
    // instruction: a single thread issuing 4 KB boxes one after the other sustains only about half of the HBM
    // bandwidth (benchmarks/bench_kernels.py --which membench).
    {
      const bool is_v = warp == 6;
      uint64_t* fullb = is_v ? vfull : kfull;
      uint64_t* emptyb = is_v ? vempty : kempty;
      const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
      const int n_boxes = pages_per_tile * 2;  // <= 32 (pages of at least 8 tokens)
      int jt = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        int seq, g, split, t0, t1;
        const int n_tiles = item_range(item, seq, g, split, t0, t1);
        const int* bt = block_tables + static_cast<size_t>(seq) * max_blocks;
        for (int j = 0; j < n_tiles; ++j, ++jt) {
          const int s = jt % kDtStages;
          int go = 1;
          if (lane == 0) {
            go = mbar_wait(&emptyb[s], ((jt / kDtStages) & 1) ^ 1, status, is_v ? 0x832 : 0x831) ? 1 : 0;
            if (go) mbar_arrive_expect_tx(&fullb[s], kDtTile);
          }
          go = __shfl_sync(0xffffffffu, go, 0);
          if (!go) {
            ok = false;
            break;
          }
          if (lane < n_boxes) {
            const int p = lane >> 1, half = lane & 1;
            int pi = (t0 + j * 128 + p * block_size) / block_size;
            pi = pi < max_blocks ? pi : max_blocks - 1;
            const int slot0 = __ldg(bt + pi) * block_size;
            uint8_t* dst = smem + s * kDtStageBytes + (is_v ? kDtTile : 0) + half * 16384 + p * block_size * 128;
            tma_load_3d(dst, tm, &fullb[s], half * 64, g, slot0);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 16, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 16, true, false);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
      auto issue_s = [&](int jt) -> bool {
        const int s = jt % kDtStages;
        if (!mbar_wait(&kfull[s], (jt / kDtStages) & 1, status, 0x841)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(smem + s * kDtStageBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16(tmem_base + (jt & 1) * 16, make_smem_desc(k_base + (k >> 2) * 16384 + (k & 3) * 32, 0, 1024),
                   make_smem_desc(q_base + (k >> 2) * 2048 + (k & 3) * 32, 0, 1024), idesc_s, k != 0);
        umma_commit(&s_full[jt & 1]);
        umma_commit(&kempty[s]);  // the K tile is free once these products retire
        return true;
      };
      int jt = 0, qi = 0;
      bool ok = true, pre_issued = false;
      int item = next_work(blockIdx.x);
      while (item < n_items && ok) {
        int seq, g, split, t0, t1;
        const int n_tiles = item_range(item, seq, g, split, t0, t1);
        const int nxt = next_work(item + gridDim.x);
        if (!pre_issued) {
          ok = mbar_wait(q_ready, qi & 1, status, 0x842);
          if (ok) {
            tc_fence_after();
            ok = issue_s(jt);
          }
        }
        pre_issued = false;
        for (int j = 0; j < n_tiles && ok; ++j, ++jt) {
          if (j + 1 < n_tiles) {
            ok = issue_s(jt + 1);
          } else if (nxt < n_items) {
            // the next item's query rows arrive while the softmax warps work on this (last) tile
            ok = mbar_wait(q_ready, (qi + 1) & 1, status, 0x843);
            if (ok) {
              tc_fence_after();
              ok = issue_s(jt + 1);
              pre_issued = true;
            }
          }
          if (!ok) break;
          if (!mbar_wait(&p_ready[jt & 1], (jt >> 1) & 1, status, 0x844)) {
            ok = false;
            break;
          }
          const int s = jt % kDtStages;
          if (!mbar_wait(&vfull[s], (jt / kDtStages) & 1, status, 0x845)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t v_base = smem_u32(smem + s * kDtStageBytes + kDtTile);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16(tmem_base + 32 + (jt & 1) * 16, make_smem_desc(v_base + k * 2048, 16384, 1024),
                     make_smem_desc(p_base + (jt & 1) * kDtPBytes + (k >> 2) * 2048 + (k & 3) * 32, 0, 1024), idesc_o,
                     k != 0);
          umma_commit(&o_full[jt & 1]);
          umma_commit(&vempty[s]);
        }
        ++qi;
        item = nxt;
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    const int sw = warp - 2;
    const int tid = threadIdx.x - 64;  // 0..127
    const int r = q * 32 + lane;       // token within the tile (S^T phase) and output dimension (O^T phase)
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    constexpr int kQChunks = (G * 16 + 127) / 128;  // 16-byte query chunks per thread
    bool ok = true;
    int jt = 0;
    auto load_q = [&](int item, uint4* regs) {
      int seq, g, split, t0, t1;
      item_range(item, seq, g, split, t0, t1);
#pragma unroll
      for (int u = 0; u < kQChunks; ++u) {
        const int i = tid + u * 128;
        if (i < G * 16) {
          const int h = i >> 4, c = i & 15;
          regs[u] = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(seq) * q_stride + (g * G + h) * 128 + c * 8);
        }
      }
    };
    auto store_q = [&](const uint4* regs) {
#pragma unroll
      for (int u = 0; u < kQChunks; ++u) {
        const int i = tid + u * 128;
        if (i < G * 16) {
          const int h = i >> 4, c = i & 15;
          const int half = c >> 3, cc = c & 7;
          *reinterpret_cast<uint4*>(sQ + half * 2048 + h * 128 + ((cc ^ (h & 7)) << 4)) = regs[u];
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    };
    auto fold_o = [&](int jtile, float* O, const float* alpha_prev) -> bool {
      if (!mbar_wait(&o_full[jtile & 1], (jtile >> 1) & 1, status, 0x851)) return false;
      tc_fence_after();
      uint32_t v[16];
      tmem_ld_32x32b_x16(tmem_base + 32 + (jtile & 1) * 16 + lane_off, v);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < G; ++h) O[h] = O[h] * alpha_prev[h] + __uint_as_float(v[h]);
      return true;
    };
    uint4 qregs[kQChunks];
    int item = blockIdx.x;
    // items without tiles (inactive slots, empty splits) only emit neutral results
    auto emit_neutral = [&](int it) {
      int seq, g, split, t0, t1;
      item_range(it, seq, g, split, t0, t1);
      const int d = tid;
      for (int h = 0; h < G; ++h) {
        const size_t head = static_cast<size_t>(seq) * nq + g * G + h;
        if (splits == 1) {
          out[head * 128 + d] = __float2bfloat16(0.f);
        } else {
          float* w = ws + (head * splits + split) * 130;
          w[d] = 0.f;
          if (d == 0) {
            w[128] = -INFINITY;
            w[129] = 0.f;
          }
        }
      }
    };
    auto skip_empty = [&](int it) -> int {
      for (; it < n_items; it += gridDim.x) {
        int a, b, c, d, e;
        if (item_range(it, a, b, c, d, e) > 0) break;
        emit_neutral(it);
      }
      return it < n_items ? it : n_items;
    };
    item = skip_empty(item);
    if (item < n_items) {
      load_q(item, qregs);
      store_q(qregs);
    }
    while (item < n_items) {
      int seq, g, split, t0, t1;
      const int n_tiles = item_range(item, seq, g, split, t0, t1);
      const int nxt = skip_empty(item + gridDim.x);
      if (nxt < n_items) load_q(nxt, qregs);
      float m[G], lsum[G], O[G], alpha_prev[G];
#pragma unroll
      for (int h = 0; h < G; ++h) {
        m[h] = -INFINITY;
        lsum[h] = 0.f;
        O[h] = 0.f;
        alpha_prev[h] = 1.f;
      }
      // Every thread executes the same number of named barriers whatever happens: after a failed wait the remaining
      // waits are skipped (ok == false) but the loop structure is kept, so nobody is left behind.
      for (int j = 0; j < n_tiles; ++j, ++jt) {
        if (ok) ok = mbar_wait(&s_full[jt & 1], (jt >> 1) & 1, status, 0x850);
        tc_fence_after();
        if (j == n_tiles - 1 && nxt < n_items) store_q(qregs);  // every S^T product of this item has completed
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem_base + (jt & 1) * 16 + lane_off, v);
        tmem_ld_wait();
        const bool valid = (t0 + j * 128 + r) < t1;
        float s[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
          s[h] = valid ? __uint_as_float(v[h]) * scale_log2 : -INFINITY;
          float mx = warp_max(s[h]);
          if (lane == 0) s_red[sw][h] = mx;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        float alpha[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float tile_max = fmaxf(fmaxf(s_red[0][h], s_red[1][h]), fmaxf(s_red[2][h], s_red[3][h]));
          const float mn = fmaxf(m[h], tile_max);
          alpha[h] = dt_exp2(m[h] - mn);  // first tile: exp2(-inf) = 0
          s[h] = valid ? dt_exp2(s[h] - mn) : 0.f;
          lsum[h] = lsum[h] * alpha[h] + s[h];
          m[h] = mn;
        }
        {
          const int half = r >> 6, col = r & 63;
          uint8_t* base = sP + (jt & 1) * kDtPBytes + half * 2048 + (col & 7) * 2;
          const int chunk = col >> 3;
#pragma unroll
          for (int h = 0; h < G; ++h)
            *reinterpret_cast<__nv_bfloat16*>(base + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16(s[h]);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (lane == 0) mbar_arrive(&p_ready[jt & 1]);
        // the previous tile's O^T (rescaled by that tile's alpha) is folded while the tensor core works on this one
        if (j > 0 && ok) ok = fold_o(jt - 1, O, alpha_prev);
#pragma unroll
        for (int h = 0; h < G; ++h) alpha_prev[h] = alpha[h];
      }
      if (ok) ok = fold_o(jt - 1, O, alpha_prev);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float t = warp_sum(lsum[h]);
        if (lane == 0) s_lsum[sw][h] = t;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok) {
        const int d = r;
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float l = s_lsum[0][h] + s_lsum[1][h] + s_lsum[2][h] + s_lsum[3][h];
          const size_t head = static_cast<size_t>(seq) * nq + g * G + h;
          if (splits == 1) {
            out[head * 128 + d] = __float2bfloat16(l > 0.f ? O[h] / l : 0.f);
          } else {
            float* w = ws + (head * splits + split) * 130;
            w[d] = O[h];
            if (d == 0) {
              w[128] = m[h];
              w[129] = l;
            }
          }
        }
      }
      // s_lsum is rewritten at the end of the next item, s_red in its first tile: both after further barriers
      asm volatile("bar.sync 1, 128;" ::: "memory");
      item = nxt;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 64);
}

__global__ void attn_decode_tc_combine_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int d = threadIdx.x;
  const float* base = ws + row * splits * 130;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[s * 130 + 128]);
  float ll = 0.f, oo = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = base[s * 130 + 128];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += base[s * 130 + 129] * w;
    oo += base[s * 130 + d] * w;
  }
  out[row * 128 + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
}

}  // namespace sb

extern "C" {

// Same contract as sb_attn_decode_paged (caches [num_blocks, block_size, nkv, 128] bf16; workspace of
// n * nq * splits * 130 floats when splits > 1).  block_size must divide 128 and be a multiple of 8.
int sb_attn_decode_paged_tc(const void* qkv, const void* k_cache, const void* v_cache, const int* block_tables,
                            const int* ctx_lens, void* out, float* workspace, int n, int nq, int nkv, int D,
                            int block_size, int num_blocks, int max_blocks, int splits, long long q_stride, float scale,
                            void* stream) {
  if (D != 128 || nq % nkv != 0 || n <= 0 || splits < 1) return SB_ERR_ARG;
  if (128 % block_size != 0 || block_size % 8 != 0) return SB_ERR_ARG;
  const int G = nq / nkv;
  if (G > 16) return SB_ERR_ARG;
  if (splits > 1 && !workspace) return SB_ERR_ARG;
  const uint64_t slots = static_cast<uint64_t>(num_blocks) * block_size;
  const CUtensorMap* tk = sb::get_tmap_bf16_3d(k_cache, 128, nkv, slots, 256, static_cast<uint64_t>(nkv) * 256, 64, 1,
                                               block_size);
  const CUtensorMap* tv = sb::get_tmap_bf16_3d(v_cache, 128, nkv, slots, 256, static_cast<uint64_t>(nkv) * 256, 64, 1,
                                               block_size);
  if (!tk || !tv) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(n, nkv, splits);
  const float sl2 = scale * 1.4426950408889634f;
  // persistent kernel (one CTA per SM walking the item list) unless SB_DECODE_ATTN_PERSIST=0
  static int persist = -1;
  if (persist < 0) {
    const char* e = getenv("SB_DECODE_ATTN_PERSIST");
    persist = (e && e[0] == '0') ? 0 : 1;
  }
  const int n_items = n * nkv * splits;
  const int pgrid = n_items < sb::sm_count() ? n_items : sb::sm_count();
#define SB_DT_CASE(GV)                                                                                              \
  case GV: {                                                                                                        \
    static bool attr_dev[64] = {};                                                                                  \
    bool& attr = attr_dev[sb::device_index()];                                                                      \
    if (!attr) {                                                                                                    \
      if (cudaFuncSetAttribute(sb::attn_decode_tc_kernel<GV>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                               sb::kDtSmem) != cudaSuccess)                                                         \
        return SB_ERR_CUDA;                                                                                         \
      attr = true;                                                                                                  \
    }                                                                                                               \
    static bool attr_p_dev[64] = {};                                                                                \
    bool& attr_p = attr_p_dev[sb::device_index()];                                                                  \
    if (!attr_p) {                                                                                                  \
      if (cudaFuncSetAttribute(sb::attn_decode_tc_persist_kernel<GV>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                               sb::kDtSmemPersist) != cudaSuccess)                                                      \
        return SB_ERR_CUDA;                                                                                         \
      attr_p = true;                                                                                                \
    }                                                                                                               \
    if (persist)                                                                                                    \
      sb::launch_pdl(sb::attn_decode_tc_persist_kernel<GV>, dim3(pgrid), dim3(sb::kDtThreadsPersist), sb::kDtSmemPersist,  \
                     st,                                                                                            \
                     *tk, *tv, reinterpret_cast<const __nv_bfloat16*>(qkv), block_tables, ctx_lens,                 \
                     reinterpret_cast<__nv_bfloat16*>(out), workspace, n, nq, nkv, block_size, max_blocks, splits,  \
                     q_stride, sl2, sb::device_status_ptr());                                                       \
    else                                                                                                            \
      sb::launch_pdl(sb::attn_decode_tc_kernel<GV>, grid, dim3(sb::kDtThreads), sb::kDtSmem, st, *tk, *tv,          \
                     reinterpret_cast<const __nv_bfloat16*>(qkv), block_tables, ctx_lens,                           \
                     reinterpret_cast<__nv_bfloat16*>(out), workspace, nq, nkv, block_size, max_blocks, splits,     \
                     q_stride, sl2, sb::device_status_ptr());                                                       \
  } break;
  switch (G) {
    SB_DT_CASE(1)
    SB_DT_CASE(2)
    SB_DT_CASE(3)
    SB_DT_CASE(4)
    SB_DT_CASE(5)
    SB_DT_CASE(6)
    SB_DT_CASE(7)
    SB_DT_CASE(8)
    SB_DT_CASE(12)
    SB_DT_CASE(16)
    default:
      return SB_ERR_ARG;
  }
#undef SB_DT_CASE
  if (splits > 1)
    sb::launch_pdl(sb::attn_decode_tc_combine_kernel, dim3(n * nq), dim3(128), 0, st, workspace,
                   reinterpret_cast<__nv_bfloat16*>(out), splits);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
