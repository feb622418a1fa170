// Consumers of split-K GEMM partial sums on the decode path.  A skinny decode GEMM (a few hundred rows)
// only fills the machine when the K dimension is split across CTAs; instead of a separate reduction pass
// the fp32 partials are summed inside the kernel that needs the result next:
//   * add_rmsnorm_partials: residual += sum_p partial_p ; y = rmsnorm(residual) * w
//       (o-proj -> post-attention norm, down-proj -> next layer's input norm / final norm)
//   * qkv_finalize: qkv = sum_p partial_p (bias is already inside partial 0); rotary embedding on the
//       q and k heads; q (and k, v) stored as bf16; k and v also scattered into their paged-cache slot.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_common.h"

namespace sb {

constexpr int kFThreads = 256;
constexpr int kFMaxVec = 4;  // H <= 256 * 8 * 4

__device__ __forceinline__ float fused_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ void ld_bf16x8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

__global__ void __launch_bounds__(kFThreads)
add_rmsnorm_partials_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ part, int n_part,
                            long long part_stride, const __nv_bfloat16* __restrict__ w,
                            __nv_bfloat16* __restrict__ y, int T, int H, float eps) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  pdl_launch_dependents();
  pdl_wait();
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float vals[kFMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kFMaxVec; ++i) {
      const int v = threadIdx.x + i * kFThreads;
      if (v < nvec) {
        const size_t off = static_cast<size_t>(row) * H + v * 8;
        ld_bf16x8(x + off, vals[i]);
        for (int p = 0; p < n_part; ++p) {
          const float4* pp = reinterpret_cast<const float4*>(part + p * part_stride + off);
          const float4 a = pp[0], b = pp[1];
          vals[i][0] += a.x; vals[i][1] += a.y; vals[i][2] += a.z; vals[i][3] += a.w;
          vals[i][4] += b.x; vals[i][5] += b.y; vals[i][6] += b.z; vals[i][7] += b.w;
        }
        // the residual stream lives in bf16: round first so the statistics match the stored values
        const uint4 rounded = pack_bf16x8(vals[i]);
        *reinterpret_cast<uint4*>(x + off) = rounded;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rounded);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = __bfloat1622float2(h[j]);
          vals[i][2 * j] = t.x;
          vals[i][2 * j + 1] = t.y;
          ss += t.x * t.x + t.y * t.y;
        }
      }
    }
    const float tot = fused_block_sum(ss, red);
    const float rstd = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
    for (int i = 0; i < kFMaxVec; ++i) {
      const int v = threadIdx.x + i * kFThreads;
      if (v < nvec) {
        float wv[8], o[8];
        ld_bf16x8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * wv[j];
        *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H + v * 8) = pack_bf16x8(o);
      }
    }
  }
}

// One thread handles 4 adjacent dims i..i+3 of the low half and the matching 4 of the high half of one
// head (rotate-half pairing), or 8 contiguous dims of a v head.
__global__ void qkv_finalize_kernel(const float* __restrict__ part, int n_part, long long part_stride,
                                    const int* __restrict__ pos, const float* __restrict__ cos_sin,
                                    const int* __restrict__ slots, __nv_bfloat16* __restrict__ qkv,
                                    __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, int T, int nq,
                                    int nkv, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = D >> 1;
  const int units_per_head = D >> 3;  // 8 output elements per unit
  const int heads = nq + 2 * nkv;
  const int row_w = heads * D;
  const long long total = static_cast<long long>(T) * heads * units_per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / (heads * units_per_head));
    const int r = static_cast<int>(idx - static_cast<long long>(t) * heads * units_per_head);
    const int head = r / units_per_head;
    const int u = r - head * units_per_head;
    const size_t row_off = static_cast<size_t>(t) * row_w + head * D;
    const int slot = slots ? slots[t] : -1;
    if (head < nq + nkv) {
      const int i = u * 4;  // dims i..i+3 (low half) pair with half+i..half+i+3
      float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
      for (int p = 0; p < n_part; ++p) {
        const float* src = part + p * part_stride + row_off;
        const float4 a = *reinterpret_cast<const float4*>(src + i);
        const float4 b = *reinterpret_cast<const float4*>(src + half + i);
        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
        hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
      }
      // the unfused path rounds the projection to bf16 before rotating: keep that rounding point
      lo.x = __bfloat162float(__float2bfloat16(lo.x)); lo.y = __bfloat162float(__float2bfloat16(lo.y));
      lo.z = __bfloat162float(__float2bfloat16(lo.z)); lo.w = __bfloat162float(__float2bfloat16(lo.w));
      hi.x = __bfloat162float(__float2bfloat16(hi.x)); hi.y = __bfloat162float(__float2bfloat16(hi.y));
      hi.z = __bfloat162float(__float2bfloat16(hi.z)); hi.w = __bfloat162float(__float2bfloat16(hi.w));
      const int ps = pos[t];
      const float4 c = *reinterpret_cast<const float4*>(cos_sin + static_cast<size_t>(ps) * D + i);
      const float4 s = *reinterpret_cast<const float4*>(cos_sin + static_cast<size_t>(ps) * D + half + i);
      uint2 olo, ohi;
      __nv_bfloat162* pl = reinterpret_cast<__nv_bfloat162*>(&olo);
      __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&ohi);
      pl[0] = __floats2bfloat162_rn(lo.x * c.x - hi.x * s.x, lo.y * c.y - hi.y * s.y);
      pl[1] = __floats2bfloat162_rn(lo.z * c.z - hi.z * s.z, lo.w * c.w - hi.w * s.w);
      ph[0] = __floats2bfloat162_rn(hi.x * c.x + lo.x * s.x, hi.y * c.y + lo.y * s.y);
      ph[1] = __floats2bfloat162_rn(hi.z * c.z + lo.z * s.z, hi.w * c.w + lo.w * s.w);
      *reinterpret_cast<uint2*>(qkv + row_off + i) = olo;
      *reinterpret_cast<uint2*>(qkv + row_off + half + i) = ohi;
      if (head >= nq && slot >= 0) {
        __nv_bfloat16* dst = kc + static_cast<size_t>(slot) * nkv * D + (head - nq) * D;
        *reinterpret_cast<uint2*>(dst + i) = olo;
        *reinterpret_cast<uint2*>(dst + half + i) = ohi;
      }
    } else {
      const int i = u * 8;
      float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < n_part; ++p) {
        const float4* src = reinterpret_cast<const float4*>(part + p * part_stride + row_off + i);
        const float4 a = src[0], b = src[1];
        o[0] += a.x; o[1] += a.y; o[2] += a.z; o[3] += a.w;
        o[4] += b.x; o[5] += b.y; o[6] += b.z; o[7] += b.w;
      }
      const uint4 ov = pack_bf16x8(o);
      *reinterpret_cast<uint4*>(qkv + row_off + i) = ov;
      if (slot >= 0)
        *reinterpret_cast<uint4*>(vc + static_cast<size_t>(slot) * nkv * D + (head - nq - nkv) * D + i) = ov;
    }
  }
}

// out[i] = sum_s slots[s][i] (fp32 accumulation), 8 elements per thread.
template <typename T>
__global__ void reduce_slots_kernel(const T* __restrict__ slots, int n_slots, long long slot_stride,
                                    __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_slots; ++s) {
      if (sizeof(T) == 2) {
        float v[8];
        ld_bf16x8(reinterpret_cast<const __nv_bfloat16*>(slots) + s * slot_stride + i * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j];
      } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(slots) + s * slot_stride + i * 8);
        const float4 a = p[0], b = p[1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
    }
    *reinterpret_cast<uint4*>(out + i * 8) = pack_bf16x8(acc);
  }
}

}  // namespace sb

extern "C" {

// out (bf16, n elements) = sum over n_slots partial buffers (bf16 or fp32) spaced slot_stride elements apart.
int sb_reduce_slots(const void* slots, int n_slots, long long slot_stride, int slots_fp32, void* out, long long n,
                    void* stream) {
  if (n <= 0 || (n & 7) || (slot_stride & 7) || n_slots < 1) return SB_ERR_ARG;
  const long long n8 = n >> 3;
  long long blocks = (n8 + 255) / 256;
  const long long cap = static_cast<long long>(sb::sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (slots_fp32)
    sb::reduce_slots_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(
        reinterpret_cast<const float*>(slots), n_slots, slot_stride, reinterpret_cast<__nv_bfloat16*>(out), n8);
  else
    sb::reduce_slots_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(slots), n_slots, slot_stride, reinterpret_cast<__nv_bfloat16*>(out), n8);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}


// x[T,H] (bf16, in place) += sum of n_part fp32 partials [T,H]; y = rmsnorm(x) * w.
int sb_add_rmsnorm_partials(void* x, const float* part, int n_part, long long part_stride, const void* w, void* y,
                            int T, int H, float eps, void* stream) {
  if (H % 8 != 0 || H > sb::kFThreads * 8 * sb::kFMaxVec || T <= 0 || n_part < 0) return SB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(part) & 15) || (part_stride & 3)) return SB_ERR_ARG;
  const int cap = sb::sm_count() * 8;
  const int grid = T < cap ? T : cap;
  const cudaError_t e = sb::launch_pdl(sb::add_rmsnorm_partials_kernel, dim3(grid), dim3(sb::kFThreads), 0,
                                       reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<__nv_bfloat16*>(x), part, n_part,
                                       part_stride, reinterpret_cast<const __nv_bfloat16*>(w),
                                       reinterpret_cast<__nv_bfloat16*>(y), T, H, eps);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// partials [n_part][T, (nq+2nkv)*D] fp32 -> qkv bf16 [T, (nq+2nkv)*D] with rotary embedding on q,k;
// k,v rows additionally written to k_cache/v_cache[slot] (slot < 0 or slots == null: not cached).
int sb_qkv_finalize(const float* part, int n_part, long long part_stride, const int* pos, const float* cos_sin,
                    const int* slots, void* qkv, void* k_cache, void* v_cache, int T, int nq, int nkv, int D,
                    void* stream) {
  if (T <= 0 || D % 8 != 0 || n_part < 1) return SB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(part) & 15) || (part_stride & 3)) return SB_ERR_ARG;
  const long long total = static_cast<long long>(T) * (nq + 2 * nkv) * (D / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sb::sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  const cudaError_t e = sb::launch_pdl(sb::qkv_finalize_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0,
                                       reinterpret_cast<cudaStream_t>(stream), part, n_part, part_stride, pos, cos_sin, slots,
                                       reinterpret_cast<__nv_bfloat16*>(qkv), reinterpret_cast<__nv_bfloat16*>(k_cache),
                                       reinterpret_cast<__nv_bfloat16*>(v_cache), T, nq, nkv, D);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
