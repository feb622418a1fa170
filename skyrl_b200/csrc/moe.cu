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

}  // extern "C"
