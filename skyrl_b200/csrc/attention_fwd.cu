// Causal variable-length attention forward (GQA, head dim 128) for packed sequences.
//
// One CTA computes a 128-row query block of one (sequence, query head).  For each 128-row KV
// block:   S = Q K^T  (tcgen05.mma, accumulator in TMEM)  ->  softmax warps read S from TMEM,
// keep running max / sum, write P (bf16, 128-byte swizzled) to shared memory  ->  O_blk = P V
// (tcgen05.mma, V consumed MN-major straight from its row-major tile), accumulated in TMEM over
// all KV blocks; the softmax warps rescale that accumulator only when the reference maximum moves
// (lazily, see the softmax role).  S is double-buffered in TMEM so that S_{j+1} is computed while
// the softmax of block j runs.  Q/K/V tiles are TMA loads from the packed
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

// Locate the (sequence, q-block) of a flat block index; heavy (late) blocks first.  `q_begin` (optional): first row of
// each sequence that carries a query; the q-blocks before it are not computed (their rows are keys / values only: a
// cached prefix, or the part of a sequence another context-parallel rank owns).
__device__ __forceinline__ bool find_block(const int* __restrict__ cu, const int* __restrict__ q_begin, int B, int flat,
                                           int& seq, int& qblk) {
  int acc = 0;
  for (int b = 0; b < B; ++b) {
    const int len = cu[b + 1] - cu[b];
    const int nb = (len + kAttnBQ - 1) / kAttnBQ;
    const int first = q_begin ? min(nb, max(0, q_begin[b]) / kAttnBQ) : 0;
    const int live = nb - first;
    if (flat < acc + live) {
      seq = b;
      qblk = nb - 1 - (flat - acc);
      return true;
    }
    acc += live;
  }
  return false;
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                const int* __restrict__ cu_seqlens, const int* __restrict__ q_begin, int B, int T, int nq, int nkv,
                float scale_log2, int* status) {
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
  __shared__ float s_half[2][2][128];  // [block parity][column half][row]: half-row maxima exchanged by a row's two threads
  __shared__ int s_pub[2][128];        // [column half][row]: 1 + index of the last block whose half maximum is published

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 256) (&s_pub[0][0])[threadIdx.x] = 0;

  if (threadIdx.x == 0) {
    int seq = 0, qblk = 0;
    s_found = find_block(cu_seqlens, q_begin, B, blockIdx.x, seq, qblk) ? 1 : 0;
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
                   make_smem_desc(v_base + k * 2048, 16384, 1024), idesc_o, (k != 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------- softmax --------------------------------
    // Two threads per query row, each owning 64 of the 128 score columns of a block.  Per block a thread reads its
    // half of S once, the pair exchanges half-row maxima through shared memory (value + block counter, bounded wait),
    // and P = exp2(s * scale - m) goes to shared memory as bf16.  O accumulates in TMEM over all blocks
    // (the PV MMAs add into it); it is only touched here when the reference maximum m has to move: m follows the
    // running row maximum lazily, i.e. only when the maximum grew by more than kRescaleGap (in log2 units), so that
    // P stays below 2^kRescaleGap and the O / l rescale (a TMEM read-modify-write) is rare after the first blocks.
    const int sw = warp - 2;   // 0..7
    const int q = warp & 3;    // TMEM lane quadrant
    const int hf = sw >> 2;    // which 64 columns this thread owns
    const int r = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_o = tmem_base + 256 + hf * 64 + lane_off;
    constexpr float kRescaleGap = 8.f;
    float m = -INFINITY, l = 0.f;  // m: reference maximum in scaled (log2) units; l: this thread's half-row sum
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int sb_ = j & 1;
      {
        const bool have_s = mbar_wait(&s_full[sb_], (j >> 1) & 1, status, 0x420);
        if (!__all_sync(0xffffffffu, have_s)) {  // the whole warp stays or leaves: TMEM loads are warp-wide
          ok = false;
          break;
        }
      }
      tc_fence_after();
      const bool diag = (j == qblk);
      const uint32_t t_s = tmem_base + sb_ * 128 + hf * 64 + lane_off;
      uint32_t sv[64];
      tmem_ld_32x32b_x32(t_s, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
      tmem_ld_32x32b_x32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sv[32]));
      tmem_ld_wait();
      float mx = -INFINITY;
      if (diag) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          if (hf * 64 + i > r) sv[i] = 0xff800000u;  // -inf above the diagonal
          mx = fmaxf(mx, __uint_as_float(sv[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
      }
      // row maximum = max of the two halves.  The partner thread (other column half, same row) publishes its value
      // and then a block counter; the wait on that counter is bounded like every other wait of this kernel, so a
      // partner that gave up cannot strand this thread.
      {
        volatile float* vals = &s_half[sb_][0][0];
        volatile int* seqs = &s_pub[0][0];
        vals[hf * 128 + r] = mx;
        __threadfence_block();
        seqs[hf * 128 + r] = j + 1;
        int spins = 0;
        bool got = true;
        while (seqs[(1 - hf) * 128 + r] < j + 1) {
          if (++spins > (1 << 24)) {
            atomicCAS(status, 0, 0x423);
            got = false;
            break;
          }
        }
        // leave the loop as a whole warp: the TMEM loads below are warp-wide instructions
        if (!__all_sync(0xffffffffu, got)) {
          ok = false;
          break;
        }
        __threadfence_block();
        mx = fmaxf(mx, vals[(1 - hf) * 128 + r]) * scale_log2;
      }
      {
        // move the reference where the row maximum outgrew it: everything accumulated so far shrinks by alpha.  The
        // O rescale is a warp-wide TMEM read-modify-write, so the warp does it together whenever any of its rows
        // needs it; rows that keep their reference multiply by one.
        const bool grow = mx > m + kRescaleGap;
        const float alpha = grow ? fast_exp2(m - mx) : 1.f;  // m = -inf on the first block -> 0
        if (grow) m = mx;
        l *= alpha;
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          const bool landed = mbar_wait(o_full, (j - 1) & 1, status, 0x421);  // PV of block j-1 is in O
          if (!__all_sync(0xffffffffu, landed)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v[16];
            tmem_ld_32x32b_x16(t_o + c * 16, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32b_x16(t_o + c * 16, v);
          }
          tmem_st_wait();
        }
      }
      const float neg_m = -m;
      float psum = 0.f;
      // exponentials first (packed in place over the scores), the shared-memory stores after the wait below
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float e0 = fast_exp2(fmaf(__uint_as_float(sv[2 * i]), scale_log2, neg_m));
        const float e1 = fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), scale_log2, neg_m));
        psum += e0 + e1;
        sv[i] = pack_bf16x2(e0, e1);
      }
      // P is single-buffered: the PV MMA of block j-1 reads it until o_full(j-1) completes.  It was issued long before
      // this block's exponentials were done, so the wait is normally over already.
      if (j > 0) {
        const bool landed = mbar_wait(o_full, (j - 1) & 1, status, 0x424);
        if (!__all_sync(0xffffffffu, landed)) {
          ok = false;
          break;
        }
      }
      // P (bf16) into the swizzled K-major tile: sub-tile hf, row r, eight 16-byte chunks
      uint8_t* prow = sP + hf * 16384 + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(sv[4 * c], sv[4 * c + 1], sv[4 * c + 2], sv[4 * c + 3]);
      l += psum;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // final O: the last PV has to land first
    if (ok) ok = mbar_wait(o_full, (n_kv - 1) & 1, status, 0x422);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    // combine the two half-row sums
    if (hf == 1) s_l[r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (hf == 0) {
      const float other = s_l[r];
      s_l[r] = l + other;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_tot = s_l[r];
    const float inv = 1.f / l_tot;
    const bool store = ok && r < rows_valid;
    __nv_bfloat16* orow = out + static_cast<size_t>(q_row0 + r) * (nq * kAttnD) + h * kAttnD + hf * 64;
    if (ok) {  // warp-uniform: the TMEM loads are warp-wide, only the stores depend on the row
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_o + c * 32, v);
        tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * u + 0]) * inv, __uint_as_float(v[8 * u + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[8 * u + 2]) * inv, __uint_as_float(v[8 * u + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[8 * u + 4]) * inv, __uint_as_float(v[8 * u + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[8 * u + 6]) * inv, __uint_as_float(v[8 * u + 7]) * inv);
            reinterpret_cast<uint4*>(orow)[c * 4 + u] = o;
          }
        }
      }
    }
    if (store) {
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
// q_begin: null, or [B] int32 on device: rows of sequence b before q_begin[b] (rounded down to a 128-row block) carry
// no query; their rows of out / lse are left untouched.
int sb_attn_fwd_varlen(const void* qkv, void* out, float* lse, const int* cu_seqlens, const int* q_begin, int B, int T,
                       int nq, int nkv, int head_dim, long long row_stride, float softmax_scale, void* stream) {
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
      *tm, reinterpret_cast<__nv_bfloat16*>(out), lse, cu_seqlens, q_begin, B, T, nq, nkv,
      softmax_scale * 1.4426950408889634f, sb::device_status_ptr());
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
