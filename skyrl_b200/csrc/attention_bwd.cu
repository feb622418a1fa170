// Causal variable-length attention backward (GQA, head dim 128) on tcgen05 tensor cores.
//
// Three kernels:
//   delta   : delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]
//   dK / dV : one CTA per (sequence, 64-row KV block, KV head); loops over the query heads of the
//             group and the 128-row query blocks that see the KV block.  Per step:
//               S = Q K^T, dP = dO V^T                 (tensor cores -> TMEM, double buffered)
//               P = exp2(S*c - lse), dS = P (dP - delta) * scale   (softmax warps, from TMEM)
//               dV^T += dO^T P,  dK^T += Q^T dS        (tensor cores, accumulators stay in TMEM)
//             The transposed accumulators ([d, kv]) keep M = 128 for every MMA; Q and dO tiles
//             are consumed K-major for the first two products and MN-major for the last two, so
//             each tile is loaded once.
//   dQ      : one CTA per (sequence, 128-row query block, query head); loops over KV blocks:
//               S, dP as above; dS -> shared memory; dQ += dS K   (accumulator in TMEM)
// No atomics: every output element is written by exactly one CTA, so results are deterministic.
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kBwdThreads = 320;  // warp0 TMA, warp1 MMA, warps 2..9 softmax
constexpr int kQTile = 128 * 128 * 2;  // 32 KB (two 16 KB halves)
constexpr int kKVTile = 64 * 128 * 2;  // 16 KB (two 8 KB halves)
constexpr int kPTile = 128 * 64 * 2;   // 16 KB
constexpr int kDkvSmem = 2 * kKVTile + 4 * kQTile + 2 * kPTile + 1024 + 256;
constexpr int kDqSmem = 2 * kQTile + 4 * kKVTile + kPTile + 1024 + 256;

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool find_block_sz(const int* __restrict__ cu, int B, int flat, int blk, int& seq,
                                              int& idx, int& nblk) {
  int acc = 0;
  for (int b = 0; b < B; ++b) {
    const int len = cu[b + 1] - cu[b];
    const int nb = (len + blk - 1) / blk;
    if (flat < acc + nb) {
      seq = b;
      idx = flat - acc;
      nblk = nb;
      return true;
    }
    acc += nb;
  }
  return false;
}

// ------------------------------------------------------------------ delta
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int T, int nq) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T * nq) return;
  const int t = warp / nq, h = warp - t * nq;
  const size_t off = (static_cast<size_t>(t) * nq + h) * 128 + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(out + off);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + off);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<size_t>(h) * T + t] = s;
}

// Issue S = Q K^T and dP = dO V^T (M = 128 q rows, N = 64 kv rows, K = 128) into TMEM.
__device__ __forceinline__ void issue_s_dp(uint32_t tmem_s, uint32_t tmem_dp, uint32_t q_base, uint32_t do_base,
                                           uint32_t k_base, uint32_t v_base) {
  constexpr uint32_t idesc = make_idesc_bf16(128, 64, false, false);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t a_off = (k >> 2) * 16384 + (k & 3) * 32;
    const uint32_t b_off = (k >> 2) * 8192 + (k & 3) * 32;
    umma_f16(tmem_s, make_smem_desc(q_base + a_off, 0, 1024), make_smem_desc(k_base + b_off, 0, 1024), idesc, k != 0);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t a_off = (k >> 2) * 16384 + (k & 3) * 32;
    const uint32_t b_off = (k >> 2) * 8192 + (k & 3) * 32;
    umma_f16(tmem_dp, make_smem_desc(do_base + a_off, 0, 1024), make_smem_desc(v_base + b_off, 0, 1024), idesc,
             k != 0);
  }
}

// Softmax-side math shared by both kernels: thread owns q row r and 32 kv columns [c0, c0+32).
// Writes bf16 P (optional) and dS rows into [128 x 64] swizzled tiles.
__device__ __forceinline__ void softmax_bwd_row(uint32_t t_s, uint32_t t_dp, int c0, int r, bool row_ok, int q_pos,
                                                int kv_pos0, int kv_valid, float lse2, float delta, float scale,
                                                float scale_log2, uint8_t* sP, uint8_t* sDS) {
  uint32_t sv[32], dv[32];
  tmem_ld_32x32b_x32(t_s + c0, sv);
  tmem_ld_32x32b_x32(t_dp + c0, dv);
  tmem_ld_wait();
  uint32_t pp[16], dd[16];
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float p[2], ds[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int c = c0 + i + e;
      const bool ok = row_ok && (c < kv_valid) && (kv_pos0 + c <= q_pos);
      const float pv = bwd_exp2(__uint_as_float(sv[i + e]) * scale_log2 - lse2);
      p[e] = ok ? pv : 0.f;
      ds[e] = ok ? pv * (__uint_as_float(dv[i + e]) - delta) * scale : 0.f;
    }
    pp[i >> 1] = pack_bf16x2(p[0], p[1]);
    dd[i >> 1] = pack_bf16x2(ds[0], ds[1]);
  }
  const int chunk0 = c0 >> 3;  // 16-byte chunk index of the first column
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int sw = ((chunk0 + c) ^ (r & 7)) << 4;
    if (sP) *reinterpret_cast<uint4*>(sP + r * 128 + sw) = make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
    *reinterpret_cast<uint4*>(sDS + r * 128 + sw) = make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
  }
}

// ------------------------------------------------------------------ dK / dV
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_qkv128, const __grid_constant__ CUtensorMap tm_qkv64,
                    const __grid_constant__ CUtensorMap tm_do, const float* __restrict__ lse,
                    const float* __restrict__ delta, __nv_bfloat16* __restrict__ dqkv, long long dqkv_stride,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ q_begin, int B, int T, int nq, int nkv,
                    float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kKVTile;
  uint8_t* sQ = smem + 2 * kKVTile;                // 2 stages of Q
  uint8_t* sDO = smem + 2 * kKVTile + 2 * kQTile;  // 2 stages of dO
  uint8_t* sP = smem + 2 * kKVTile + 4 * kQTile;
  uint8_t* sDS = sP + kPTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kPTile);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* sdp_full = bars + 5;   // [2]
  uint64_t* pds_ready = bars + 7;
  uint64_t* acc_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  __shared__ int s_seq, s_blk, s_nblk, s_found;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    int seq = 0, blk = 0, nblk = 0;
    s_found = find_block_sz(cu_seqlens, B, blockIdx.x, 64, seq, blk, nblk) ? 1 : 0;
    s_seq = seq;
    s_blk = blk;
    s_nblk = nblk;
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
    }
    mbar_init(pds_ready, 8);
    mbar_init(acc_done, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (!s_found) return;
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int seq = s_seq, jblk = s_blk;
  const int g = blockIdx.y;
  const int rep = nq / nkv;
  const int seq_start = cu_seqlens[seq];
  const int seq_len = cu_seqlens[seq + 1] - seq_start;
  const int kv_pos0 = jblk * 64;
  const int kv_valid = min(64, seq_len - kv_pos0);
  const int nqb = (seq_len + 127) / 128;
  // query blocks that see this key/value block: from its own block on, and not before the sequence's first query row
  const int i0 = max(kv_pos0 / 128, q_begin ? min(nqb, max(0, q_begin[seq]) / 128) : 0);
  const int per_head = nqb - i0;
  const int n_it = rep * per_head;
  const int col_k = (nq + g) * 128, col_v = (nq + nkv + g) * 128;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * kKVTile);
      tma_load_2d(sK, &tm_qkv64, kv_full, col_k, seq_start + kv_pos0);
      tma_load_2d(sK + 8192, &tm_qkv64, kv_full, col_k + 64, seq_start + kv_pos0);
      tma_load_2d(sV, &tm_qkv64, kv_full, col_v, seq_start + kv_pos0);
      tma_load_2d(sV + 8192, &tm_qkv64, kv_full, col_v + 64, seq_start + kv_pos0);
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        const int hh = it / per_head, i = i0 + (it - hh * per_head);
        const int h = g * rep + hh;
        const int row = seq_start + i * 128;
        if (!mbar_wait(&qdo_empty[s], ((it >> 1) & 1) ^ 1, status, 0x501)) break;
        mbar_arrive_expect_tx(&qdo_full[s], 2 * kQTile);
        tma_load_2d(sQ + s * kQTile, &tm_qkv128, &qdo_full[s], h * 128, row);
        tma_load_2d(sQ + s * kQTile + 16384, &tm_qkv128, &qdo_full[s], h * 128 + 64, row);
        tma_load_2d(sDO + s * kQTile, &tm_do, &qdo_full[s], h * 128, row);
        tma_load_2d(sDO + s * kQTile + 16384, &tm_do, &qdo_full[s], h * 128 + 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_t = make_idesc_bf16(128, 64, true, true);  // [d x kv] += X^T[d x q] * Y[q x kv]
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), p_base = smem_u32(sP), ds_base = smem_u32(sDS);
      auto issue = [&](int it) -> bool {
        const int s = it & 1;
        if (!mbar_wait(&qdo_full[s], (it >> 1) & 1, status, 0x511)) return false;
        tc_fence_after();
        issue_s_dp(tmem_base + s * 64, tmem_base + 128 + s * 64, smem_u32(sQ + s * kQTile),
                   smem_u32(sDO + s * kQTile), k_base, v_base);
        umma_commit(&sdp_full[s]);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, status, 0x510);
      if (ok) ok = issue(0);
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) {
          ok = issue(it + 1);
          if (!ok) break;
        }
        const int s = it & 1;
        if (!mbar_wait(pds_ready, it & 1, status, 0x512)) break;
        tc_fence_after();
        const uint32_t q_base = smem_u32(sQ + s * kQTile), do_base = smem_u32(sDO + s * kQTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dV^T += dO^T P
          umma_f16(tmem_base + 256, make_smem_desc(do_base + k * 2048, 16384, 1024),
                   make_smem_desc(p_base + k * 2048, 16384, 1024), idesc_t, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dK^T += Q^T dS
          umma_f16(tmem_base + 320, make_smem_desc(q_base + k * 2048, 16384, 1024),
                   make_smem_desc(ds_base + k * 2048, 16384, 1024), idesc_t, (it | k) != 0);
        umma_commit(&qdo_empty[s]);
        umma_commit(acc_done);
      }
    }
  } else {
    const int q = warp & 3, hf = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const int hh = it / per_head, i = i0 + (it - hh * per_head);
      const int h = g * rep + hh;
      const int q_pos = i * 128 + r;
      const bool row_ok = q_pos < seq_len;
      float lse2 = 0.f, dl = 0.f;
      if (row_ok) {
        lse2 = lse[static_cast<size_t>(h) * T + seq_start + q_pos] * 1.4426950408889634f;
        dl = delta[static_cast<size_t>(h) * T + seq_start + q_pos];
      }
      if (!mbar_wait(&sdp_full[s], (it >> 1) & 1, status, 0x520)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (it > 0 && !mbar_wait(acc_done, (it - 1) & 1, status, 0x521)) {
        ok = false;
        break;
      }
      softmax_bwd_row(tmem_base + s * 64 + lane_off, tmem_base + 128 + s * 64 + lane_off, hf * 32, r, row_ok, q_pos,
                      kv_pos0, kv_valid, lse2, dl, scale, scale_log2, sP, sDS);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
    }
    if (ok && n_it > 0) ok = mbar_wait(acc_done, (n_it - 1) & 1, status, 0x522);
    if (ok) {
      tc_fence_after();
      // accumulators are transposed: TMEM lane = d index, column = kv row
      const int d = r;
      uint32_t a[32], b[32];
      if (n_it > 0) {
        tmem_ld_32x32b_x32(tmem_base + 256 + hf * 32 + lane_off, a);
        tmem_ld_32x32b_x32(tmem_base + 320 + hf * 32 + lane_off, b);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) a[c] = b[c] = 0u;
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int kv = hf * 32 + c;
        if (kv < kv_valid) {
          __nv_bfloat16* row = dqkv + static_cast<size_t>(seq_start + kv_pos0 + kv) * dqkv_stride;
          row[col_v + d] = __float2bfloat16(__uint_as_float(a[c]));
          row[col_k + d] = __float2bfloat16(__uint_as_float(b[c]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------------ dQ
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qkv128, const __grid_constant__ CUtensorMap tm_qkv64,
                   const __grid_constant__ CUtensorMap tm_do, const float* __restrict__ lse,
                   const float* __restrict__ delta, __nv_bfloat16* __restrict__ dqkv, long long dqkv_stride,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ q_begin, int B, int T, int nq, int nkv,
                   float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + kQTile;
  uint8_t* sK = smem + 2 * kQTile;                // 2 stages
  uint8_t* sV = smem + 2 * kQTile + 2 * kKVTile;  // 2 stages
  uint8_t* sDS = smem + 2 * kQTile + 4 * kKVTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kPTile);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* sdp_full = bars + 5;  // [2]
  uint64_t* ds_ready = bars + 7;
  uint64_t* acc_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  __shared__ int s_seq, s_blk, s_nblk, s_found;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    int seq = 0, blk = 0, nblk = 0;
    s_found = find_block_sz(cu_seqlens, B, blockIdx.x, 128, seq, blk, nblk) ? 1 : 0;
    s_seq = seq;
    s_blk = s_found ? (nblk - 1 - blk) : 0;  // heavy blocks first
    s_nblk = nblk;
    // blocks before the sequence's first query row have no dQ to compute (the caller zero-fills dqkv)
    if (s_found && q_begin != nullptr && s_blk < min(nblk, max(0, q_begin[seq]) / 128)) s_found = 0;
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
    }
    mbar_init(ds_ready, 8);
    mbar_init(acc_done, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (!s_found) return;
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int seq = s_seq, iblk = s_blk;
  const int h = blockIdx.y;
  const int g = h / (nq / nkv);
  const int seq_start = cu_seqlens[seq];
  const int seq_len = cu_seqlens[seq + 1] - seq_start;
  const int q_pos0 = iblk * 128;
  const int q_end = min(seq_len, q_pos0 + 128);
  const int n_kv = (q_end + 63) / 64;
  const int col_k = (nq + g) * 128, col_v = (nq + nkv + g) * 128;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (warp == 0) {
    if (lane == 0) {
      const int row = seq_start + q_pos0;
      mbar_arrive_expect_tx(qdo_full, 2 * kQTile);
      tma_load_2d(sQ, &tm_qkv128, qdo_full, h * 128, row);
      tma_load_2d(sQ + 16384, &tm_qkv128, qdo_full, h * 128 + 64, row);
      tma_load_2d(sDO, &tm_do, qdo_full, h * 128, row);
      tma_load_2d(sDO + 16384, &tm_do, qdo_full, h * 128 + 64, row);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const int kvrow = seq_start + j * 64;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, status, 0x601)) break;
        mbar_arrive_expect_tx(&kv_full[s], 2 * kKVTile);
        tma_load_2d(sK + s * kKVTile, &tm_qkv64, &kv_full[s], col_k, kvrow);
        tma_load_2d(sK + s * kKVTile + 8192, &tm_qkv64, &kv_full[s], col_k + 64, kvrow);
        tma_load_2d(sV + s * kKVTile, &tm_qkv64, &kv_full[s], col_v, kvrow);
        tma_load_2d(sV + s * kKVTile + 8192, &tm_qkv64, &kv_full[s], col_v + 64, kvrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 128, false, true);  // dQ[q x d] += dS[q x kv] * K[kv x d]
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), ds_base = smem_u32(sDS);
      auto issue = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&kv_full[s], (j >> 1) & 1, status, 0x611)) return false;
        tc_fence_after();
        issue_s_dp(tmem_base + s * 64, tmem_base + 128 + s * 64, q_base, do_base, smem_u32(sK + s * kKVTile),
                   smem_u32(sV + s * kKVTile));
        umma_commit(&sdp_full[s]);
        return true;
      };
      bool ok = mbar_wait(qdo_full, 0, status, 0x610);
      if (ok) ok = issue(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          ok = issue(j + 1);
          if (!ok) break;
        }
        const int s = j & 1;
        if (!mbar_wait(ds_ready, j & 1, status, 0x612)) break;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + s * kKVTile);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_base + 256, make_smem_desc(ds_base + k * 32, 0, 1024),
                   make_smem_desc(k_base + k * 2048, 8192, 1024), idesc_dq, (j | k) != 0);
        umma_commit(&kv_empty[s]);
        umma_commit(acc_done);
      }
    }
  } else {
    const int q = warp & 3, hf = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int q_pos = q_pos0 + r;
    const bool row_ok = q_pos < seq_len;
    float lse2 = 0.f, dl = 0.f;
    if (row_ok) {
      lse2 = lse[static_cast<size_t>(h) * T + seq_start + q_pos] * 1.4426950408889634f;
      dl = delta[static_cast<size_t>(h) * T + seq_start + q_pos];
    }
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&sdp_full[s], (j >> 1) & 1, status, 0x620)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (j > 0 && !mbar_wait(acc_done, (j - 1) & 1, status, 0x621)) {
        ok = false;
        break;
      }
      const int kv_valid = min(64, seq_len - j * 64);
      softmax_bwd_row(tmem_base + s * 64 + lane_off, tmem_base + 128 + s * 64 + lane_off, hf * 32, r, row_ok, q_pos,
                      j * 64, kv_valid, lse2, dl, scale, scale_log2, nullptr, sDS);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    if (ok) ok = mbar_wait(acc_done, (n_kv - 1) & 1, status, 0x622);
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + 256 + hf * 64 + c * 32 + lane_off, v);
        tmem_ld_wait();
        if (row_ok) {
          __nv_bfloat16* row =
              dqkv + static_cast<size_t>(seq_start + q_pos) * dqkv_stride + h * 128 + hf * 64 + c * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
            reinterpret_cast<uint4*>(row)[i] = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace sb

extern "C" {

// dqkv (same layout and row stride as qkv) receives dQ | dK | dV.  `delta_ws` is an fp32 workspace of
// nq * T elements (null -> error; the caller owns all memory).  q_begin: null, or [B] int32 on device as in the
// forward pass; the dQ rows of the skipped query blocks are not written (pass a zero-filled dqkv).
int sb_attn_bwd_varlen(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                       const int* cu_seqlens, const int* q_begin, float* delta_ws, int B, int T, int nq, int nkv,
                       int head_dim, long long row_stride, float softmax_scale, void* stream) {
  if (head_dim != 128 || nq % nkv != 0 || T <= 0 || B <= 0 || !delta_ws) return SB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long W = static_cast<long long>(nq + 2 * nkv) * 128;
  const CUtensorMap* tq128 = sb::get_tmap_bf16_2d(qkv, T, W, row_stride, 128);
  const CUtensorMap* tq64 = sb::get_tmap_bf16_2d(qkv, T, W, row_stride, 64);
  const CUtensorMap* tdo = sb::get_tmap_bf16_2d(dout, T, static_cast<long long>(nq) * 128, static_cast<long long>(nq) * 128, 128);
  if (!tq128 || !tq64 || !tdo) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  if (!attr_set) {
    if (cudaFuncSetAttribute(sb::attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sb::kDkvSmem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(sb::attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sb::kDqSmem) !=
            cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  const long long warps = static_cast<long long>(T) * nq;
  sb::attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta_ws, T, nq);
  dim3 g_kv((T + 63) / 64 + B, nkv);
  sb::attn_bwd_dkv_kernel<<<g_kv, sb::kBwdThreads, sb::kDkvSmem, st>>>(
      *tq128, *tq64, *tdo, lse, delta_ws, reinterpret_cast<__nv_bfloat16*>(dqkv), row_stride, cu_seqlens, q_begin, B, T, nq,
      nkv, softmax_scale, sb::device_status_ptr());
  dim3 g_q((T + 127) / 128 + B, nq);
  sb::attn_bwd_dq_kernel<<<g_q, sb::kBwdThreads, sb::kDqSmem, st>>>(
      *tq128, *tq64, *tdo, lse, delta_ws, reinterpret_cast<__nv_bfloat16*>(dqkv), row_stride, cu_seqlens, q_begin, B, T, nq,
      nkv, softmax_scale, sb::device_status_ptr());
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
