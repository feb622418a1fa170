// Causal variable-length attention forward (GQA, head dim 128) for packed sequences.
//
// One CTA computes a 128-row query block of one (sequence, query head).  For each 128-row KV
// block:   S = Q K^T  (tcgen05.mma, accumulator in TMEM)  ->  softmax warps read S from TMEM,
// keep running max / sum, write P (bf16, 128-byte swizzled) to shared memory  ->  O_blk = P V
// (tcgen05.mma, V consumed MN-major straight from its row-major tile)  ->  softmax warps fold
// O_blk into fp32 register accumulators.  S is double-buffered in TMEM so that S_{j+1} is
// computed while the softmax of block j runs.  Q/K/V tiles are TMA loads from the packed
// [T, (nq + 2 nkv) * 128] QKV activation; nothing is unpadded or repacked on the host.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..9 = softmax
// (two threads per query row, each owning 64 of the 128 output columns).
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kAttnD = 128;
constexpr int kAttnBQ = 128;
constexpr int kAttnBKV = 128;
constexpr int kAttnThreads = 320;
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KB: one [128 x 128] bf16 tile = two 16 KB swizzled halves
constexpr int kAttnSmem = 6 * kTileBytes + 1024 + 256;  // Q, K x2, V x2, P

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Locate the (sequence, q-block) of a flat block index; heavy (late) blocks first.
__device__ __forceinline__ bool find_block(const int* __restrict__ cu, int B, int flat, int& seq, int& qblk) {
  int acc = 0;
  for (int b = 0; b < B; ++b) {
    const int len = cu[b + 1] - cu[b];
    const int nb = (len + kAttnBQ - 1) / kAttnBQ;
    if (flat < acc + nb) {
      seq = b;
      qblk = nb - 1 - (flat - acc);
      return true;
    }
    acc += nb;
  }
  return false;
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                const int* __restrict__ cu_seqlens, int B, int T, int nq, int nkv, float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;      // 2 stages
  uint8_t* sV = smem + 3 * kTileBytes;  // 2 stages
  uint8_t* sP = smem + 5 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* p_ready = bars + 11;
  uint64_t* o_full = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  __shared__ int s_seq, s_qblk, s_found;
  __shared__ float s_l[128];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    int seq = 0, qblk = 0;
    s_found = find_block(cu_seqlens, B, blockIdx.x, seq, qblk) ? 1 : 0;
    s_seq = seq;
    s_qblk = qblk;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_ready, 8);
    mbar_init(o_full, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (!s_found) return;  // uniform for the CTA; nothing allocated yet

  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int seq = s_seq, qblk = s_qblk;
  const int h = blockIdx.y;
  const int g = h / (nq / nkv);
  const int seq_start = cu_seqlens[seq];
  const int seq_len = cu_seqlens[seq + 1] - seq_start;
  const int q_row0 = seq_start + qblk * kAttnBQ;
  const int rows_valid = min(kAttnBQ, seq_len - qblk * kAttnBQ);
  const int n_kv = qblk + 1;
  const int col_q = h * kAttnD;
  const int col_k = (nq + g) * kAttnD;
  const int col_v = (nq + nkv + g) * kAttnD;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_qkv);
      mbar_arrive_expect_tx(q_full, kTileBytes);
      tma_load_2d(sQ, &tm_qkv, q_full, col_q, q_row0);
      tma_load_2d(sQ + 16384, &tm_qkv, q_full, col_q + 64, q_row0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kv_row = seq_start + j * kAttnBKV;
        if (!mbar_wait(&k_empty[s], ph ^ 1, status, 0x401)) break;
        mbar_arrive_expect_tx(&k_full[s], kTileBytes);
        tma_load_2d(sK + s * kTileBytes, &tm_qkv, &k_full[s], col_k, kv_row);
        tma_load_2d(sK + s * kTileBytes + 16384, &tm_qkv, &k_full[s], col_k + 64, kv_row);
        if (!mbar_wait(&v_empty[s], ph ^ 1, status, 0x402)) break;
        mbar_arrive_expect_tx(&v_full[s], kTileBytes);
        tma_load_2d(sV + s * kTileBytes, &tm_qkv, &v_full[s], col_v, kv_row);
        tma_load_2d(sV + s * kTileBytes + 16384, &tm_qkv, &v_full[s], col_v + 64, kv_row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t q_base = smem_u32(sQ);
      const uint32_t p_base = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1, status, 0x411)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + s * kTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16(tmem_base + s * 128, make_smem_desc(q_base + off, 0, 1024), make_smem_desc(k_base + off, 0, 1024),
                   idesc_s, k != 0);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, status, 0x410);
      if (ok) {
        tc_fence_after();
        ok = issue_s(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int s = j & 1;
        if (!mbar_wait(p_ready, j & 1, status, 0x412)) break;
        if (!mbar_wait(&v_full[s], (j >> 1) & 1, status, 0x413)) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sV + s * kTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t a_off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16(tmem_base + 256, make_smem_desc(p_base + a_off, 0, 1024),
                   make_smem_desc(v_base + k * 2048, 16384, 1024), idesc_o, k != 0);
        }
        umma_commit(o_full);
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------- softmax --------------------------------
    const int sw = warp - 2;   // 0..7
    const int q = warp & 3;    // TMEM lane quadrant
    const int hf = sw >> 2;    // which 64 columns this thread owns
    const int r = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float O[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) O[i] = 0.f;
    bool ok = true;

    auto accumulate_o = [&](int j, float alpha) -> bool {
      if (!mbar_wait(o_full, j & 1, status, 0x421)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + 256 + hf * 64 + c * 32 + lane_off, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) O[c * 32 + i] = O[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      return true;
    };

    for (int j = 0; j < n_kv; ++j) {
      const int sb_ = j & 1;
      if (!mbar_wait(&s_full[sb_], (j >> 1) & 1, status, 0x420)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool diag = (j == qblk);
      const uint32_t t_s = tmem_base + sb_ * 128 + lane_off;
      float mx = m;
      // the other half of the row only contributes to the max
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        const int cbase = (1 - hf) * 64 + c * 32;
        tmem_ld_32x32b_x32(t_s + cbase, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]) * scale_log2;
          if (diag && (cbase + i > r)) s = -INFINITY;
          mx = fmaxf(mx, s);
        }
      }
      float sv[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        const int cbase = hf * 64 + c * 32;
        tmem_ld_32x32b_x32(t_s + cbase, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]) * scale_log2;
          if (diag && (cbase + i > r)) s = -INFINITY;
          sv[c * 32 + i] = s;
          mx = fmaxf(mx, s);
        }
      }
      const float alpha = fast_exp2(m - mx);  // m = -inf on the first block -> 0
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        sv[i] = fast_exp2(sv[i] - mx);
        psum += sv[i];
      }
      l = l * alpha + psum;
      if (j > 0) {
        if (!accumulate_o(j - 1, alpha_prev)) {
          ok = false;
          break;
        }
      }
      // P (bf16) into the swizzled K-major tile: sub-tile hf, row r, eight 16-byte chunks
      uint8_t* prow = sP + hf * 16384 + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 o;
        o.x = pack_bf16x2(sv[8 * c + 0], sv[8 * c + 1]);
        o.y = pack_bf16x2(sv[8 * c + 2], sv[8 * c + 3]);
        o.z = pack_bf16x2(sv[8 * c + 4], sv[8 * c + 5]);
        o.w = pack_bf16x2(sv[8 * c + 6], sv[8 * c + 7]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = o;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      m = mx;
      alpha_prev = alpha;
    }
    if (ok) ok = accumulate_o(n_kv - 1, alpha_prev);
    // combine the two half-row sums
    if (hf == 1) s_l[r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (hf == 0) {
      const float other = s_l[r];
      s_l[r] = l + other;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_tot = s_l[r];
    if (ok && r < rows_valid) {
      const float inv = 1.f / l_tot;
      __nv_bfloat16* orow = out + static_cast<size_t>(q_row0 + r) * (nq * kAttnD) + h * kAttnD + hf * 64;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 o;
        o.x = pack_bf16x2(O[8 * c + 0] * inv, O[8 * c + 1] * inv);
        o.y = pack_bf16x2(O[8 * c + 2] * inv, O[8 * c + 3] * inv);
        o.z = pack_bf16x2(O[8 * c + 4] * inv, O[8 * c + 5] * inv);
        o.w = pack_bf16x2(O[8 * c + 6] * inv, O[8 * c + 7] * inv);
        reinterpret_cast<uint4*>(orow)[c] = o;
      }
      if (hf == 0 && lse) lse[static_cast<size_t>(h) * T + q_row0 + r] = (m + log2f(l_tot)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace sb

extern "C" {

// qkv: packed [T, (nq + 2 nkv) * 128] bf16 (RoPE already applied), row stride `row_stride` elements.
// out: [T, nq * 128] bf16; lse: [nq, T] fp32 (natural log) or null; cu_seqlens: [B + 1] int32 on device.
int sb_attn_fwd_varlen(const void* qkv, void* out, float* lse, const int* cu_seqlens, int B, int T, int nq, int nkv,
                       int head_dim, long long row_stride, float softmax_scale, void* stream) {
  if (head_dim != sb::kAttnD || nq % nkv != 0 || T <= 0 || B <= 0) return SB_ERR_ARG;
  const long long W = static_cast<long long>(nq + 2 * nkv) * sb::kAttnD;
  const CUtensorMap* tm = sb::get_tmap_bf16_2d(qkv, T, W, row_stride, 128);
  if (!tm) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  if (!attr_set) {
    if (cudaFuncSetAttribute(sb::attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sb::kAttnSmem) !=
        cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  dim3 grid((T + sb::kAttnBQ - 1) / sb::kAttnBQ + B, nq);
  sb::attn_fwd_kernel<<<grid, sb::kAttnThreads, sb::kAttnSmem, reinterpret_cast<cudaStream_t>(stream)>>>(
      *tm, reinterpret_cast<__nv_bfloat16*>(out), lse, cu_seqlens, B, T, nq, nkv,
      softmax_scale * 1.4426950408889634f, sb::device_status_ptr());
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
