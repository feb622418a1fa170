// Generation-engine kernels: KV-cache scatter, paged-KV decode attention (split-KV with a
// combine pass), Gumbel-max sampling with the chosen token's log-probability, and the
// token-embedding gather.
#include <curand_kernel.h>

#include <atomic>
#include <mutex>

#include "host_common.h"
#include "ptx.cuh"

namespace sb {

// ------------------------------------------------------------------ KV cache write
// qkv row t -> k_cache[slot[t]], v_cache[slot[t]]; caches are [num_slots, nkv, D] flattened.
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                                      __nv_bfloat16* __restrict__ vc, const int* __restrict__ slots, int T, int nq,
                                      int nkv, int D, long long row_stride) {
  const int vec_per_row = nkv * D / 8;
  const long long total = static_cast<long long>(T) * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec_per_row);
    const int v = static_cast<int>(idx - static_cast<long long>(t) * vec_per_row);
    const int slot = slots[t];
    if (slot < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(t) * row_stride + nq * D);
    reinterpret_cast<uint4*>(kc + static_cast<size_t>(slot) * nkv * D)[v] = src[v];
    reinterpret_cast<uint4*>(vc + static_cast<size_t>(slot) * nkv * D)[v] = src[vec_per_row + v];
  }
}

// ------------------------------------------------------------------ decode attention
// grid (n_seq, nkv, splits), 128 threads. 16 lanes cooperate on one token (8 dims each), so a warp
// covers 2 tokens per step and the CTA 8.  G = nq / nkv query heads share every K/V row read.
constexpr int kDecMaxG = 8;
constexpr int kDecThreads = 128;

template <int G>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_tables,
                   const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ ws, int nq,
                   int nkv, int block_size, int max_blocks, int splits, long long q_stride, float scale_log2) {
  constexpr int D = 128;
  const int seq = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int ctx = ctx_lens[seq];
  const int per_split = ((ctx + splits - 1) / splits + 7) & ~7;
  const int t0 = split * per_split;
  const int t1 = min(ctx, t0 + per_split);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 15, tok_in_warp = lane >> 4;

  float q[G][8], o[G][8], m[G], l[G];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(seq) * q_stride + (g * G + h) * D + sub * 8);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p[i]);
      q[h][2 * i] = f.x * scale_log2;
      q[h][2 * i + 1] = f.y * scale_log2;
    }
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[h][i] = 0.f;
  }

  const int* bt = block_tables + static_cast<size_t>(seq) * max_blocks;
  // the trip count is uniform per warp (full-mask shuffles below); the second token of the pair
  // may fall beyond the range and is then predicated off
  for (int tb = t0 + warp * 2; tb < t1; tb += 8) {
    const int t = tb + tok_in_warp;
    const bool valid = t < t1;
    uint4 kv4 = make_uint4(0u, 0u, 0u, 0u), vv4 = make_uint4(0u, 0u, 0u, 0u);
    if (valid) {
      const int blk = bt[t / block_size];
      const size_t slot = static_cast<size_t>(blk) * block_size + (t % block_size);
      const size_t off = (slot * nkv + g) * D + sub * 8;
      kv4 = *reinterpret_cast<const uint4*>(kc + off);
      vv4 = *reinterpret_cast<const uint4*>(vc + off);
    }
    float kf[8], vf[8];
    {
      const __nv_bfloat162* pk = reinterpret_cast<const __nv_bfloat162*>(&kv4);
      const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&vv4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(pk[i]);
        const float2 b = __bfloat1622float2(pv[i]);
        kf[2 * i] = a.x;
        kf[2 * i + 1] = a.y;
        vf[2 * i] = b.x;
        vf[2 * i + 1] = b.y;
      }
    }
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += q[h][i] * kf[i];
#pragma unroll
      for (int ofs = 8; ofs > 0; ofs >>= 1) s += __shfl_xor_sync(0xffffffffu, s, ofs);
      if (!valid) s = -INFINITY;
      const float mn = fmaxf(m[h], s);
      if (mn == -INFINITY) continue;
      const float alpha = exp2f(m[h] - mn);
      const float p = exp2f(s - mn);
      l[h] = l[h] * alpha + p;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[h][i] = o[h][i] * alpha + p * vf[i];
      m[h] = mn;
    }
  }
  // tokens beyond t1 simply did not iterate; lanes whose loop ended early hold (m=-inf, l=0)

  // merge the 8 token-groups of the CTA through shared memory
  __shared__ float s_m[8][G], s_l[8][G];
  __shared__ float s_o[8][G][D];
  const int grp = warp * 2 + tok_in_warp;
#pragma unroll
  for (int h = 0; h < G; ++h) {
    if (sub == 0) {
      s_m[grp][h] = m[h];
      s_l[grp][h] = l[h];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_o[grp][h][sub * 8 + i] = o[h][i];
  }
  __syncthreads();
  // thread d (0..127) merges column d for every head
  const int d = threadIdx.x;
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float mm = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; ++k) mm = fmaxf(mm, s_m[k][h]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float w = (s_m[k][h] == -INFINITY) ? 0.f : exp2f(s_m[k][h] - mm);
      ll += s_l[k][h] * w;
      oo += s_o[k][h][d] * w;
    }
    const int head = g * G + h;
    if (splits == 1) {
      out[(static_cast<size_t>(seq) * nq + head) * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
    } else {
      float* w = ws + ((static_cast<size_t>(seq) * nq + head) * splits + split) * (D + 2);
      w[d] = oo;
      if (d == 0) {
        w[D] = mm;
        w[D + 1] = ll;
      }
    }
  }
}

__global__ void attn_decode_combine_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int splits) {
  constexpr int D = 128;
  const size_t row = blockIdx.x;  // seq * nq + head
  const int d = threadIdx.x;
  const float* base = ws + row * splits * (D + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[s * (D + 2) + D]);
  float ll = 0.f, oo = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = base[s * (D + 2) + D];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += base[s * (D + 2) + D + 1] * w;
    oo += base[s * (D + 2) + d] * w;
  }
  out[row * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
}

// ------------------------------------------------------------------ sampling
// One CTA per row. token = argmax_i (z_i / T + Gumbel_i) is an exact sample of softmax(z / T);
// logprob = z_tok / T - logsumexp(z / T).  temperature <= 0 -> greedy.
constexpr int kSampThreads = 512;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One block per (row, vocabulary part).  Each part keeps the running maximum of logit + Gumbel noise (the sampled
// token) and an online log-sum-exp (for the token's log-probability); the part that finishes last for a row merges
// the parts (a per-row counter that it resets, so nothing has to be cleared between launches).
struct SamplePart {
  float best;
  int best_i;
  float m, s;
};

__device__ __forceinline__ void sample_merge(float& best, int& best_i, float& m, float& s, float ob, int oi, float om,
                                             float os) {
  if (ob > best || (ob == best && oi < best_i)) {
    best = ob;
    best_i = oi;
  }
  const float mn = fmaxf(m, om);
  s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (om == -INFINITY ? 0.f : os * __expf(om - mn));
  m = mn;
}

template <typename T>
__global__ void __launch_bounds__(kSampThreads)
sample_gumbel_kernel(const T* __restrict__ logits, long long row_stride, int V, const float* __restrict__ temperature,
                     unsigned long long seed, const long long* __restrict__ step_offsets, int* __restrict__ tokens,
                     float* __restrict__ logprobs, SamplePart* __restrict__ parts, unsigned int* __restrict__ counters) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int n_parts = gridDim.y, part = blockIdx.y;
  const T* z = logits + static_cast<size_t>(row) * row_stride;
  const float temp = temperature[row];
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  curandStatePhilox4_32_10_t rng;
  curand_init(seed, (static_cast<unsigned long long>(row) * n_parts + part) * kSampThreads + threadIdx.x,
              step_offsets ? static_cast<unsigned long long>(step_offsets[0]) * 1024ull : 0ull, &rng);
  // this part's range, in whole groups of 8 elements
  const int groups = (V + 7) / 8;
  const int g_per = (groups + n_parts - 1) / n_parts;
  const int g0 = part * g_per, g1 = min(groups, g0 + g_per);
  const bool vec_ok = (sizeof(T) == 2) && ((reinterpret_cast<uintptr_t>(z) & 15) == 0);
  float best = -INFINITY, m = -INFINITY, s = 0.f;
  int best_i = 0x7fffffff;
  for (int g = g0 + threadIdx.x; g < g1; g += kSampThreads) {
    const int i0 = g * 8;
    float x[8];
    if (vec_ok && i0 + 8 <= V) {
      const uint4 raw = *reinterpret_cast<const uint4*>(z + i0);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x[2 * e] = __uint_as_float(w[e] << 16) * inv_t;
        x[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u) * inv_t;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = (i0 + e < V) ? to_f<T>(z[i0 + e]) * inv_t : -INFINITY;
    }
    // log-sum-exp: one rescale per group instead of one per element
    float gm = x[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) gm = fmaxf(gm, x[e]);
    if (gm > -INFINITY) {
      const float mn = fmaxf(m, gm);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += __expf(x[e] - mn);
      s = s * __expf(m - mn) + acc;
      m = mn;
    }
    if (greedy) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (x[e] > best) {  // ascending index within a thread: ties keep the first
          best = x[e];
          best_i = i0 + e;
        }
    } else {
      const float4 ua = curand_uniform4(&rng), ub = curand_uniform4(&rng);
      const float u[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float y = x[e] - __logf(-__logf(u[e]));
        if (y > best) {
          best = y;
          best_i = i0 + e;
        }
      }
    }
  }
  __shared__ float sh_best[kSampThreads / 32], sh_m[kSampThreads / 32], sh_s[kSampThreads / 32];
  __shared__ int sh_i[kSampThreads / 32];
  __shared__ bool is_last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    sample_merge(best, best_i, m, s, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o),
                 __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sh_best[warp] = best;
    sh_i[warp] = best_i;
    sh_m[warp] = m;
    sh_s[warp] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kSampThreads / 32; ++w) sample_merge(best, best_i, m, s, sh_best[w], sh_i[w], sh_m[w], sh_s[w]);
    if (n_parts > 1) {
      parts[static_cast<size_t>(row) * n_parts + part] = SamplePart{best, best_i, m, s};
      __threadfence();
      is_last = atomicAdd(counters + row, 1u) == static_cast<unsigned int>(n_parts - 1);
      if (is_last) {
        __threadfence();
        best = -INFINITY;
        best_i = 0x7fffffff;
        m = -INFINITY;
        s = 0.f;
        for (int p = 0; p < n_parts; ++p) {
          const volatile SamplePart* sp = parts + static_cast<size_t>(row) * n_parts + p;
          sample_merge(best, best_i, m, s, sp->best, sp->best_i, sp->m, sp->s);
        }
        counters[row] = 0;
      }
    } else {
      is_last = true;
    }
    if (is_last) {
      best_i = best_i < V ? best_i : V - 1;
      tokens[row] = best_i;
      logprobs[row] = to_f<T>(z[best_i]) * inv_t - (m + __logf(s));
    }
  }
}

// ------------------------------------------------------------------ embedding gather
__global__ void embed_gather_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                    __nv_bfloat16* __restrict__ out, int T, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec = H / 8;
  const long long total = static_cast<long long>(T) * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec);
    const int v = static_cast<int>(idx - static_cast<long long>(t) * vec);
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[v] =
        reinterpret_cast<const uint4*>(table + static_cast<size_t>(ids[t]) * H)[v];
  }
}


// ------------------------------------------------------------------ decode state advance
// One thread per engine slot. Appends the sampled token / log-probability to the slot's output row,
// decides termination (EOS after min_new tokens, or max_new reached) and prepares the next step's
// input token, position, KV slot and context length, so that a decode step needs no host work.
struct DecodeState {
  int* cur_tokens;       // [S] input token of the next step
  int* positions;        // [S]
  int* slots;            // [S] KV slot of the next step's token (-1 = no write)
  int* ctx_lens;         // [S]
  const int* block_tables;  // [S, max_blocks]
  int* active;           // [S]
  int* finish_reason;    // [S] 0 = running, 1 = stop (EOS), 2 = length
  int* gen_count;        // [S]
  const int* max_new;    // [S]
  const int* min_new;    // [S]
  int* out_tokens;       // [S, out_stride]
  float* out_logprobs;   // [S, out_stride]
  const int* eos_ids;    // [n_eos]
  long long* step_counter;  // [1] incremented once per call (decorrelates the sampler across graph replays)
};

__global__ void decode_advance_kernel(DecodeState st, const int* __restrict__ sampled,
                                      const float* __restrict__ sampled_lp, int n, int max_blocks, int block_size,
                                      int out_stride, int n_eos) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0 && st.step_counter) *st.step_counter += 1;
  if (i >= n || !st.active[i]) return;
  const int tok = sampled[i];
  int gc = st.gen_count[i];
  if (gc < out_stride) {
    st.out_tokens[static_cast<size_t>(i) * out_stride + gc] = tok;
    st.out_logprobs[static_cast<size_t>(i) * out_stride + gc] = sampled_lp[i];
  }
  ++gc;
  st.gen_count[i] = gc;
  int reason = 0;
  if (gc >= st.min_new[i])
    for (int e = 0; e < n_eos; ++e)
      if (tok == st.eos_ids[e]) reason = 1;
  if (!reason && gc >= st.max_new[i]) reason = 2;
  if (reason) {
    st.active[i] = 0;
    st.finish_reason[i] = reason;
    st.slots[i] = -1;
    st.ctx_lens[i] = 0;
    return;
  }
  const int p = st.positions[i] + 1;
  st.positions[i] = p;
  st.cur_tokens[i] = tok;
  st.slots[i] = st.block_tables[static_cast<size_t>(i) * max_blocks + p / block_size] * block_size + p % block_size;
  st.ctx_lens[i] = p + 1;
}

static inline int grid_1d(long long items, int threads) {
  long long b = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace sb

extern "C" {

int sb_kv_cache_write(const void* qkv, void* k_cache, void* v_cache, const int* slots, int T, int nq, int nkv, int D,
                      long long row_stride, int reserved, void* stream) {
  (void)reserved;
  if (T <= 0) return SB_OK;
  if ((nkv * D) % 8 != 0) return SB_ERR_ARG;
  sb::kv_cache_write_kernel<<<sb::grid_1d(static_cast<long long>(T) * nkv * D / 8, 256), 256, 0,
                              reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), slots, T, nq, nkv, D, row_stride);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_attn_decode_paged(const void* qkv, const void* k_cache, const void* v_cache, const int* block_tables,
                         const int* ctx_lens, void* out, float* workspace, int n, int nq, int nkv, int D,
                         int block_size, int max_blocks, int splits, long long q_stride, float scale, void* stream) {
  if (D != 128 || nq % nkv != 0 || n <= 0 || splits < 1) return SB_ERR_ARG;
  const int G = nq / nkv;
  if (G > sb::kDecMaxG) return SB_ERR_ARG;
  if (splits > 1 && !workspace) return SB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(n, nkv, splits);
  const float sl2 = scale * 1.4426950408889634f;
#define SB_DEC_CASE(GV)                                                                                              \
  case GV:                                                                                                           \
    sb::attn_decode_kernel<GV><<<grid, sb::kDecThreads, 0, st>>>(                                                    \
        reinterpret_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const __nv_bfloat16*>(k_cache),                \
        reinterpret_cast<const __nv_bfloat16*>(v_cache), block_tables, ctx_lens, reinterpret_cast<__nv_bfloat16*>(out), \
        workspace, nq, nkv, block_size, max_blocks, splits, q_stride, sl2);                                          \
    break;
  switch (G) {
    SB_DEC_CASE(1)
    SB_DEC_CASE(2)
    SB_DEC_CASE(3)
    SB_DEC_CASE(4)
    SB_DEC_CASE(5)
    SB_DEC_CASE(6)
    SB_DEC_CASE(7)
    SB_DEC_CASE(8)
    default:
      return SB_ERR_ARG;
  }
#undef SB_DEC_CASE
  if (splits > 1)
    sb::attn_decode_combine_kernel<<<n * nq, 128, 0, st>>>(workspace, reinterpret_cast<__nv_bfloat16*>(out), splits);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// logits: [n, V] bf16 (is_bf16 = 1) or fp32; temperature: [n] fp32 on device; step_offsets: optional device
// int64 counter that decorrelates successive calls made from a replayed CUDA graph.
int sb_sample_gumbel(const void* logits, int is_bf16, long long row_stride, int n, int V, const float* temperature,
                     unsigned long long seed, const long long* step_offsets, int* tokens, float* logprobs,
                     void* stream) {
  if (n <= 0 || V <= 0) return SB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Rows are split into vocabulary parts until the grid has a few blocks per SM.  The partial records live in a
  // library-owned buffer of kSlots regions used round-robin, so that launches in flight on different streams (or
  // baked into different CUDA graphs) do not share a region.  The buffer is created by the first call (outside any
  // stream capture: engines run one eager step before they capture).
  constexpr int kSlots = 16, kMaxRows = 4096, kMaxParts = 8;
  static sb::SamplePart* part_buf = nullptr;
  static unsigned int* counter_buf = nullptr;
  static std::atomic<unsigned int> next_slot{0};
  static std::mutex alloc_mu;  // engines may be stepped from several host threads
  std::lock_guard<std::mutex> lock(alloc_mu);
  int n_parts = 1;
  if (n <= kMaxRows && V >= 32768) {
    const int want = (4 * sb::sm_count() + n - 1) / n;
    n_parts = want < 1 ? 1 : (want > kMaxParts ? kMaxParts : want);
  }
  if (n_parts > 1 && part_buf == nullptr) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cs);
    if (cs != cudaStreamCaptureStatusNone) {
      n_parts = 1;  // cannot allocate while capturing
    } else {
      if (cudaMalloc(&part_buf, sizeof(sb::SamplePart) * kSlots * kMaxRows * kMaxParts) != cudaSuccess ||
          cudaMalloc(&counter_buf, sizeof(unsigned int) * kSlots * kMaxRows) != cudaSuccess ||
          cudaMemset(counter_buf, 0, sizeof(unsigned int) * kSlots * kMaxRows) != cudaSuccess)
        return SB_ERR_CUDA;
    }
  }
  sb::SamplePart* parts = nullptr;
  unsigned int* counters = nullptr;
  if (n_parts > 1) {
    const unsigned int slot = next_slot.fetch_add(1) % kSlots;
    parts = part_buf + static_cast<size_t>(slot) * kMaxRows * kMaxParts;
    counters = counter_buf + static_cast<size_t>(slot) * kMaxRows;
  }
  const dim3 grid(n, n_parts);
  if (is_bf16)
    sb::launch_pdl(sb::sample_gumbel_kernel<__nv_bfloat16>, grid, dim3(sb::kSampThreads), 0, st,
                   reinterpret_cast<const __nv_bfloat16*>(logits), row_stride, V, temperature, seed, step_offsets, tokens,
                   logprobs, parts, counters);
  else
    sb::launch_pdl(sb::sample_gumbel_kernel<float>, grid, dim3(sb::kSampThreads), 0, st,
                   reinterpret_cast<const float*>(logits), row_stride, V, temperature, seed, step_offsets, tokens, logprobs,
                   parts, counters);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// ptrs: the 14 device pointers of DecodeState in declaration order.
int sb_decode_advance(void* const* ptrs, const int* sampled, const float* sampled_lp, int n, int max_blocks,
                      int block_size, int out_stride, int n_eos, void* stream) {
  if (n <= 0) return SB_OK;
  sb::DecodeState st;
  st.cur_tokens = static_cast<int*>(ptrs[0]);
  st.positions = static_cast<int*>(ptrs[1]);
  st.slots = static_cast<int*>(ptrs[2]);
  st.ctx_lens = static_cast<int*>(ptrs[3]);
  st.block_tables = static_cast<const int*>(ptrs[4]);
  st.active = static_cast<int*>(ptrs[5]);
  st.finish_reason = static_cast<int*>(ptrs[6]);
  st.gen_count = static_cast<int*>(ptrs[7]);
  st.max_new = static_cast<const int*>(ptrs[8]);
  st.min_new = static_cast<const int*>(ptrs[9]);
  st.out_tokens = static_cast<int*>(ptrs[10]);
  st.out_logprobs = static_cast<float*>(ptrs[11]);
  st.eos_ids = static_cast<const int*>(ptrs[12]);
  st.step_counter = static_cast<long long*>(ptrs[13]);
  const cudaError_t e = sb::launch_pdl(sb::decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0,
                                       reinterpret_cast<cudaStream_t>(stream), st, sampled, sampled_lp, n, max_blocks, block_size,
                                       out_stride, n_eos);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_embed_gather(const void* table, const int* ids, void* out, int T, int H, void* stream) {
  if (T <= 0) return SB_OK;
  if (H % 8 != 0) return SB_ERR_ARG;
  sb::launch_pdl(sb::embed_gather_kernel, dim3(sb::grid_1d(static_cast<long long>(T) * H / 8, 256)), dim3(256), 0,
                 reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(table), ids,
                 reinterpret_cast<__nv_bfloat16*>(out), T, H);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
