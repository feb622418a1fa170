// Token movement around the grouped expert GEMMs of a mixture-of-experts layer.
//
// The expert GEMMs work on a padded, expert-grouped row buffer [M_cap, H] (128-row tiles, one expert per tile).
//   moe_gather_rows : row r of the padded buffer = hidden row row_src[r] (zero when row_src[r] < 0, i.e. padding)
//   moe_combine     : out[t] = sum_s w[t, s] * y[slot_row[t, s]]   (w == nullptr: plain sum, the input gradient of
//                     the gather)
//   moe_combine_bwd : dy[slot_row[t, s]] = w[t, s] * dout[t];  dw[t, s] = <y[slot_row[t, s]], dout[t]>
// Every padded row is written by exactly one warp, so nothing needs atomics; the routing tables stay on the device.
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float* f) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// one warp per destination row; H % 8 == 0
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ row_src,
                                       __nv_bfloat16* __restrict__ dst, int rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vec = H >> 3;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_block) {
    const int s = __ldg(row_src + r);
    uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * H);
    if (s < 0) {
      for (int c = lane; c < vec; c += 32) d[c] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* p = reinterpret_cast<const uint4*>(src + static_cast<size_t>(s) * H);
      for (int c = lane; c < vec; c += 32) d[c] = __ldg(p + c);
    }
  }
}

// one warp per token; k <= 16
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_row,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T, int k, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vec = H >> 3;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    int rows[16];
    float ws[16];
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      if (s < k) {
        rows[s] = __ldg(slot_row + static_cast<size_t>(t) * k + s);
        ws[s] = w ? __ldg(w + static_cast<size_t>(t) * k + s) : 1.f;
      }
    }
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
    for (int c = lane; c < vec; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        if (s < k) {
          float f[8];
          bf16x8_to_float(__ldg(reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[s]) * H) + c), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += ws[s] * f[i];
        }
      }
      o[c] = float_to_bf16x8(acc);
    }
  }
}

// one warp per (token, slot)
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_row,
                                       const float* __restrict__ w, const __nv_bfloat16* __restrict__ dout,
                                       __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, long long n, int k, int H) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int vec = H >> 3;
  for (long long e = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); e < n;
       e += static_cast<long long>(gridDim.x) * warps_per_block) {
    const long long t = e / k;
    const int row = __ldg(slot_row + e);
    const float wt = w ? __ldg(w + e) : 1.f;
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(t) * H);
    const uint4* yr = reinterpret_cast<const uint4*>(y + static_cast<size_t>(row) * H);
    uint4* d = reinterpret_cast<uint4*>(dy + static_cast<size_t>(row) * H);
    float dot = 0.f;
    for (int c = lane; c < vec; c += 32) {
      float gf[8], yf[8], o[8];
      bf16x8_to_float(__ldg(g + c), gf);
      if (dw) {
        bf16x8_to_float(__ldg(yr + c), yf);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += gf[i] * yf[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = wt * gf[i];
      d[c] = float_to_bf16x8(o);
    }
    if (dw) {
      dot = warp_sum(dot);
      if (lane == 0) dw[e] = dot;
    }
  }
}


// Router: softmax over the experts, top-k, optional renormalisation of the k weights.  One warp per token; lane l
// holds experts l, l + 32, ...  (E <= 1024, k <= 16).  Ties go to the lower expert index.
constexpr int kRouteMaxPerLane = 32;

__global__ void moe_route_kernel(const float* __restrict__ logits, float* __restrict__ w, int* __restrict__ idx, int T, int E,
                                 int k, int norm) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) >> 5;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    const float* z = logits + static_cast<size_t>(t) * E;
    float p[kRouteMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      if (j < per) {
        const int e = j * 32 + lane;
        p[j] = e < E ? __ldg(z + e) : -INFINITY;
        mx = fmaxf(mx, p[j]);
      }
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      if (j < per) {
        p[j] = __expf(p[j] - mx);
        sum += p[j];
      }
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    float sel_sum = 0.f;
    float my_w = 0.f;  // lane s keeps the s-th selected weight
    int my_i = 0;
    for (int s = 0; s < k; ++s) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kRouteMaxPerLane; ++j) {
        if (j < per && p[j] > best) {  // ascending expert index within a lane: ties keep the lower one
          best = p[j];
          best_e = j * 32 + lane;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < kRouteMaxPerLane; ++j)
          if (j == (best_e >> 5)) p[j] = -1.f;  // taken
      }
      const float pv = best * inv;
      sel_sum += pv;
      if (lane == s) {
        my_w = pv;
        my_i = best_e;
      }
    }
    if (lane < k) {
      w[static_cast<size_t>(t) * k + lane] = norm ? my_w / sel_sum : my_w;
      idx[static_cast<size_t>(t) * k + lane] = my_i;
    }
  }
}

// d(logits) from d(w): w_j = p_j / S (S = sum of the selected p) when norm, else w_j = p_j, and p = softmax(logits).
__global__ void moe_route_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ w, const int* __restrict__ idx,
                                     const float* __restrict__ dw, float* __restrict__ dlogits, int T, int E, int k, int norm) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) >> 5;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block) {
    const float* z = logits + static_cast<size_t>(t) * E;
    float p[kRouteMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      if (j < per) {
        const int e = j * 32 + lane;
        p[j] = e < E ? __ldg(z + e) : -INFINITY;
        mx = fmaxf(mx, p[j]);
      }
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      if (j < per) {
        p[j] = __expf(p[j] - mx);
        sum += p[j];
      }
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    // lane s < k owns selected slot s
    const int my_e = lane < k ? __ldg(idx + static_cast<size_t>(t) * k + lane) : -1;
    const float my_dw = lane < k ? __ldg(dw + static_cast<size_t>(t) * k + lane) : 0.f;
    const float my_wt = lane < k ? __ldg(w + static_cast<size_t>(t) * k + lane) : 0.f;
    float dp_sel = my_dw;  // d/dp of the selected probability
    float p_sel = 0.f;
    if (norm) {
      const float dot = warp_sum(my_dw * my_wt);
      // S = p_j / w_j for any selected j with w_j > 0; recompute it from the probabilities instead
      float ps = 0.f;
      for (int s = 0; s < k; ++s) {
        const int e = __shfl_sync(0xffffffffu, my_e, s);
        float v = 0.f;
#pragma unroll
        for (int j = 0; j < kRouteMaxPerLane; ++j)
          if (j < per && j == (e >> 5) && (e & 31) == lane) v = p[j] * inv;
        v = warp_sum(v);
        ps += v;
        if (lane == s) p_sel = v;
      }
      dp_sel = (my_dw - dot) / ps;
    } else {
      for (int s = 0; s < k; ++s) {
        const int e = __shfl_sync(0xffffffffu, my_e, s);
        float v = 0.f;
#pragma unroll
        for (int j = 0; j < kRouteMaxPerLane; ++j)
          if (j < per && j == (e >> 5) && (e & 31) == lane) v = p[j] * inv;
        v = warp_sum(v);
        if (lane == s) p_sel = v;
      }
    }
    const float inner = warp_sum(lane < k ? p_sel * dp_sel : 0.f);  // sum_m p_m dp_m
    // dlogits_i = p_i * (dp_i - inner)
    float* out = dlogits + static_cast<size_t>(t) * E;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      if (j < per) {
        const int e = j * 32 + lane;
        if (e < E) out[e] = -p[j] * inv * inner;
      }
    }
    __syncwarp();
    if (lane < k) out[my_e] = p_sel * (dp_sel - inner);
  }
}


// Layout plan of a grouped expert launch, one CTA: histogram of the routed entries per expert, every expert's row
// range padded to whole 128-row tiles, and a *stable* placement of the entries (entry order is kept inside an expert,
// so the row order -- and with it the summation order of the weight gradients -- does not change from run to run).
// Each warp owns a contiguous segment of the entries: pass A counts its segment per expert, a scan over the warps
// turns the counts into per-warp cursors, pass B walks the segment again and places the entries.
//   k_off[E + 1]        first padded row of each expert
//   tile_expert[tiles]  owner of every 128-row tile, -1 = unused
//   row_src[m_cap]      token (entry / top_k) whose hidden row fills a padded row, -1 = padding
//   slot_row[n]         padded row of every entry
constexpr int kPlanThreads = 1024;
constexpr int kPlanWarps = kPlanThreads / 32;

template <typename IdT>
__global__ void __launch_bounds__(kPlanThreads, 1)
moe_plan_kernel(const IdT* __restrict__ ids, int n, int E, int top_k, int m_cap, int* __restrict__ k_off,
                int* __restrict__ tile_expert, int* __restrict__ row_src, int* __restrict__ slot_row) {
  extern __shared__ int plan_smem[];
  int* cnt = plan_smem;                 // [kPlanWarps][E] counts, then cursors
  int* off = plan_smem + kPlanWarps * E;  // [E + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kPlanWarps * E; i += kPlanThreads) cnt[i] = 0;
  for (int i = threadIdx.x; i < m_cap; i += kPlanThreads) row_src[i] = -1;
  for (int i = threadIdx.x; i < m_cap / 128; i += kPlanThreads) tile_expert[i] = -1;
  __syncthreads();
  const int seg = (n + kPlanWarps - 1) / kPlanWarps;
  const int lo = min(n, warp * seg), hi = min(n, lo + seg);
  for (int i = lo + lane; i < hi; i += 32) {
    const int e = static_cast<int>(ids[i]);
    if (e >= 0 && e < E) atomicAdd(&cnt[warp * E + e], 1);
  }
  __syncthreads();
  // per expert: total, padded total (thread e), then a serial scan over the experts by thread 0
  for (int e = threadIdx.x; e < E; e += kPlanThreads) {
    int tot = 0;
    for (int w = 0; w < kPlanWarps; ++w) {
      const int c = cnt[w * E + e];
      cnt[w * E + e] = tot;  // entries of this expert in earlier warps
      tot += c;
    }
    off[e + 1] = (tot + 127) & ~127;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    off[0] = 0;
    for (int e = 0; e < E; ++e) off[e + 1] += off[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += kPlanThreads) k_off[e] = off[e];
  for (int e = threadIdx.x; e < E; e += kPlanThreads)
    for (int t = off[e] / 128; t < off[e + 1] / 128; ++t) tile_expert[t] = e;
  // pass B: stable placement; only this warp touches its row of cursors
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const bool live = i < hi;
    const int e = live ? static_cast<int>(ids[i]) : -1;
    const bool ok = live && e >= 0 && e < E;
    const unsigned int peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int leader = __ffs(peers) - 1;
    int start = 0;
    if (ok && lane == leader) {
      start = cnt[warp * E + e];
      cnt[warp * E + e] = start + __popc(peers);
    }
    start = __shfl_sync(0xffffffffu, start, leader);
    if (ok) {
      const int row = off[e] + start + rank;
      slot_row[i] = row;
      row_src[row] = i / top_k;
    } else if (live) {
      slot_row[i] = 0;
    }
    __syncwarp();
  }
}

}  // namespace sb

extern "C" {

int sb_moe_gather_rows(const void* src, const int* row_src, void* dst, int rows, int H, void* stream) {
  if (rows <= 0 || H <= 0 || (H & 7)) return SB_ERR_ARG;
  const int blocks = (rows + 7) / 8;
  sb::launch_pdl(sb::moe_gather_rows_kernel, dim3(blocks < 148 * 16 ? blocks : 148 * 16), dim3(256), 0,
                 reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(src), row_src,
                 reinterpret_cast<__nv_bfloat16*>(dst), rows, H);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_moe_combine(const void* y, const int* slot_row, const float* w, void* out, int T, int k, int H, void* stream) {
  if (T <= 0 || k <= 0 || k > 16 || H <= 0 || (H & 7)) return SB_ERR_ARG;
  const int blocks = (T + 7) / 8;
  sb::launch_pdl(sb::moe_combine_kernel, dim3(blocks < 148 * 16 ? blocks : 148 * 16), dim3(256), 0,
                 reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(y), slot_row, w,
                 reinterpret_cast<__nv_bfloat16*>(out), T, k, H);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// dy must be zero-filled by the caller wherever no slot points (padding rows); dw may be null.
int sb_moe_combine_bwd(const void* y, const int* slot_row, const float* w, const void* dout, void* dy, float* dw, int T,
                       int k, int H, void* stream) {
  if (T <= 0 || k <= 0 || H <= 0 || (H & 7)) return SB_ERR_ARG;
  const long long n = static_cast<long long>(T) * k;
  const long long blocks = (n + 7) / 8;
  sb::moe_combine_bwd_kernel<<<static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0,
                               reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(y), slot_row, w, reinterpret_cast<const __nv_bfloat16*>(dout),
      reinterpret_cast<__nv_bfloat16*>(dy), dw, n, k, H);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_moe_route(const float* logits, float* w, int* idx, int T, int E, int k, int norm, void* stream) {
  if (T <= 0 || E <= 0 || E > 32 * sb::kRouteMaxPerLane || k <= 0 || k > 16 || k > E) return SB_ERR_ARG;
  const int blocks = (T + 7) / 8;
  sb::moe_route_kernel<<<blocks < 148 * 8 ? blocks : 148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, w, idx, T,
                                                                                                            E, k, norm);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_moe_route_bwd(const float* logits, const float* w, const int* idx, const float* dw, float* dlogits, int T, int E, int k,
                     int norm, void* stream) {
  if (T <= 0 || E <= 0 || E > 32 * sb::kRouteMaxPerLane || k <= 0 || k > 16 || k > E) return SB_ERR_ARG;
  const int blocks = (T + 7) / 8;
  sb::moe_route_bwd_kernel<<<blocks < 148 * 8 ? blocks : 148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, w, idx, dw, dlogits, T, E, k, norm);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// ids: [n] expert of every routed entry (int32 when ids_are_i64 == 0, else int64); E <= 1024; m_cap a multiple of 128
// and at least the padded row total.
int sb_moe_plan(const void* ids, int ids_are_i64, int n, int E, int top_k, int m_cap, int* k_off, int* tile_expert,
                int* row_src, int* slot_row, void* stream) {
  if (n < 0 || E <= 0 || E > 1024 || top_k <= 0 || m_cap <= 0 || (m_cap % 128) != 0) return SB_ERR_ARG;
  const size_t smem = sizeof(int) * (static_cast<size_t>(sb::kPlanWarps) * E + E + 1);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ids_are_i64) {
    static bool attr_dev[64] = {};
    bool& attr = attr_dev[sb::device_index()];
    if (!attr) {
      if (cudaFuncSetAttribute(sb::moe_plan_kernel<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, 140 * 1024) !=
          cudaSuccess)
        return SB_ERR_CUDA;
      attr = true;
    }
    sb::moe_plan_kernel<long long><<<1, sb::kPlanThreads, smem, st>>>(static_cast<const long long*>(ids), n, E, top_k, m_cap,
                                                                      k_off, tile_expert, row_src, slot_row);
  } else {
    static bool attr_dev[64] = {};
    bool& attr = attr_dev[sb::device_index()];
    if (!attr) {
      if (cudaFuncSetAttribute(sb::moe_plan_kernel<int>, cudaFuncAttributeMaxDynamicSharedMemorySize, 140 * 1024) != cudaSuccess)
        return SB_ERR_CUDA;
      attr = true;
    }
    sb::moe_plan_kernel<int><<<1, sb::kPlanThreads, smem, st>>>(static_cast<const int*>(ids), n, E, top_k, m_cap, k_off,
                                                                tile_expert, row_src, slot_row);
  }
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
