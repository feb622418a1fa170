// Bandwidth-bound transformer ops, one pass over HBM each:
//   * residual-add + RMSNorm forward (writes the new residual stream and the normed
//     activations together), RMSNorm backward fused with the residual gradient add
//   * rotary embedding applied in place on the packed QKV buffer (forward and inverse)
//   * SwiGLU forward / backward on the fused [gate | up] projection output
//   * flat fused AdamW on fp32 master shards writing bf16 parameters, with the
//     global-norm clip coefficient read from device memory
//   * squared-norm reduction of a flat fp32 buffer
// All kernels use 16-byte vector accesses and grid sizes that are multiples of the SM count.
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ---------------------------------------------------------------------------
// RMSNorm.  One CTA per row; H % 8 == 0, H <= 8 * 8 * blockDim.
// x_out = x (+ delta);  y = x_out * rstd * w
// ---------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // H <= 256 * 8 * 4 = 8192

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ x_out,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, int H, float eps) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + static_cast<size_t>(row) * H) : nullptr;
    float vals[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        bf16x8_to_float(xr[v], vals[i]);
        if (dr) {
          float d[8];
          bf16x8_to_float(dr[v], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += d[j];
          // the residual stream is kept in bf16: round before the statistics so that
          // forward and recomputation see identical values
          uint4 rounded = float_to_bf16x8(vals[i]);
          if (x_out) reinterpret_cast<uint4*>(x_out + static_cast<size_t>(row) * H)[v] = rounded;
          bf16x8_to_float(rounded, vals[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / static_cast<float>(H) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float wv[8], o[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(w)[v], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * wv[j];
        reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H)[v] = float_to_bf16x8(o);
      }
    }
  }
}

// dx = dres + rstd * (dy*w - xhat * mean(dy*w*xhat)),  dw[h] += sum_rows dy*xhat
// dw is accumulated with one atomicAdd per column per CTA into an fp32 buffer.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                   int T, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dw_acc[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  float wv[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) bf16x8_to_float(reinterpret_cast<const uint4*>(w)[v], wv[i]);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * H;
    const float rs = rstd[row];
    float g[kNormMaxVec][8], xh[kNormMaxVec][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float d[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(dy + off)[v], d);
        bf16x8_to_float(reinterpret_cast<const uint4*>(x + off)[v], xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rs;
          dw_acc[i][j] += d[j] * xh[i][j];
          g[i][j] = d[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    const float mean = block_sum(dot, red) / static_cast<float>(H);
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
        float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (dres) bf16x8_to_float(reinterpret_cast<const uint4*>(dres + off)[v], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r[j] + rs * (g[i][j] - xh[i][j] * mean);
        reinterpret_cast<uint4*>(dx + off)[v] = float_to_bf16x8(o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw + v * 8 + j, dw_acc[i][j]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Warp-per-row variants (H = NV * 256, NV <= 8): no block-level synchronisation in the row loop, eight rows in flight
// per CTA.  The row statistics are warp shuffles; the weight gradient is kept per lane and reduced once per CTA.
// ---------------------------------------------------------------------------
constexpr int kWarpNormThreads = 256;

template <int NV>
__global__ void __launch_bounds__(kWarpNormThreads)
rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ x_out,
                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, float eps) {
  constexpr int H = NV * 256;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  pdl_wait();
  uint4 wq[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) wq[i] = reinterpret_cast<const uint4*>(w)[i * 32 + lane];
  for (int row = blockIdx.x * 8 + warp; row < T; row += gridDim.x * 8) {
    const size_t off = static_cast<size_t>(row) * H;
    float vals[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = i * 32 + lane;
      bf16x8_to_float(reinterpret_cast<const uint4*>(x + off)[v], vals[i]);
      if (delta) {
        float d[8];
        bf16x8_to_float(reinterpret_cast<const uint4*>(delta + off)[v], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] += d[j];
        const uint4 rounded = float_to_bf16x8(vals[i]);  // the residual stream is stored in bf16: use those values
        if (x_out) reinterpret_cast<uint4*>(x_out + off)[v] = rounded;
        bf16x8_to_float(rounded, vals[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
    const float rs = rsqrtf(warp_sum(ss) / static_cast<float>(H) + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rs;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float wv[8], o[8];
      bf16x8_to_float(wq[i], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rs * wv[j];
      reinterpret_cast<uint4*>(y + off)[i * 32 + lane] = float_to_bf16x8(o);
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(kWarpNormThreads)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                        int T) {
  constexpr int H = NV * 256;
  extern __shared__ float sred[];  // [8 warps][H] for the final weight-gradient reduction
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4 wq[NV];
  float dw_acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    wq[i] = reinterpret_cast<const uint4*>(w)[i * 32 + lane];
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  }
  for (int row = blockIdx.x * 8 + warp; row < T; row += gridDim.x * 8) {
    const size_t off = static_cast<size_t>(row) * H;
    const float rs = rstd[row];
    uint4 dq[NV], xq[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      dq[i] = reinterpret_cast<const uint4*>(dy + off)[i * 32 + lane];
      xq[i] = reinterpret_cast<const uint4*>(x + off)[i * 32 + lane];
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float d[8], xh[8], wv[8];
      bf16x8_to_float(dq[i], d);
      bf16x8_to_float(xq[i], xh);
      bf16x8_to_float(wq[i], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[j] *= rs;
        dw_acc[i][j] += d[j] * xh[j];
        dot += d[j] * wv[j] * xh[j];
      }
    }
    const float mean = warp_sum(dot) / static_cast<float>(H);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float d[8], xh[8], wv[8], o[8];
      float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      bf16x8_to_float(dq[i], d);
      bf16x8_to_float(xq[i], xh);
      bf16x8_to_float(wq[i], wv);
      if (dres) bf16x8_to_float(reinterpret_cast<const uint4*>(dres + off)[i * 32 + lane], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = r[j] + rs * (d[j] * wv[j] - xh[j] * rs * mean);
      reinterpret_cast<uint4*>(dx + off)[i * 32 + lane] = float_to_bf16x8(o);
    }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) sred[warp * H + (i * 32 + lane) * 8 + j] = dw_acc[i][j];
    __syncthreads();
    for (int c = threadIdx.x; c < H; c += kWarpNormThreads) {
      float t = 0.f;
#pragma unroll
      for (int wq_ = 0; wq_ < 8; ++wq_) t += sred[wq_ * H + c];
      atomicAdd(dw + c, t);
    }
  }
}

// ---------------------------------------------------------------------------
// RoPE (rotate-half convention: pairs (i, i + D/2)) in place on the q and k heads
// of a packed [T, (nq + 2 nkv) * D] buffer. cos_sin is a [max_pos, D] fp32 table:
// cos in [:, :D/2], sin in [:, D/2:].  sign = +1 forward, -1 inverse (backward).
// ---------------------------------------------------------------------------
__global__ void rope_inplace_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                    const float* __restrict__ cos_sin, int T, int n_rot_heads, int row_stride, int D,
                                    float sign) {
  const int half = D >> 1;
  const int pairs_per_row = n_rot_heads * (half >> 1);  // each thread handles 2 adjacent pairs (bf16x2)
  const long long total = static_cast<long long>(T) * pairs_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / pairs_per_row);
    const int r = static_cast<int>(idx - static_cast<long long>(t) * pairs_per_row);
    const int head = r / (half >> 1);
    const int i = (r - head * (half >> 1)) * 2;
    const int p = pos[t];
    const float2 c = *reinterpret_cast<const float2*>(cos_sin + static_cast<size_t>(p) * D + i);
    float2 s = *reinterpret_cast<const float2*>(cos_sin + static_cast<size_t>(p) * D + half + i);
    s.x *= sign;
    s.y *= sign;
    __nv_bfloat16* base = qkv + static_cast<size_t>(t) * row_stride + head * D;
    __nv_bfloat162* lo = reinterpret_cast<__nv_bfloat162*>(base + i);
    __nv_bfloat162* hi = reinterpret_cast<__nv_bfloat162*>(base + half + i);
    const float2 a = __bfloat1622float2(*lo);
    const float2 b = __bfloat1622float2(*hi);
    *lo = __floats2bfloat162_rn(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
    *hi = __floats2bfloat162_rn(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
  }
}

// Same rotation, eight pairs per thread (16-byte accesses); needs D / 2 to be a multiple of 8 and 16-byte aligned rows.
__global__ void rope_inplace_vec8_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                         const float* __restrict__ cos_sin, int T, int n_rot_heads, int row_stride, int D,
                                         float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;
  const int vec_per_row = n_rot_heads * vec_per_head;
  const long long total = static_cast<long long>(T) * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / vec_per_row);
    const int r = static_cast<int>(idx - static_cast<long long>(t) * vec_per_row);
    const int head = r / vec_per_head;
    const int i = (r - head * vec_per_head) * 8;
    const float* cs = cos_sin + static_cast<size_t>(__ldg(pos + t)) * D;
    float c[8], sn[8], a[8], b[8], lo[8], hi[8];
    *reinterpret_cast<float4*>(c) = __ldg(reinterpret_cast<const float4*>(cs + i));
    *reinterpret_cast<float4*>(c + 4) = __ldg(reinterpret_cast<const float4*>(cs + i + 4));
    *reinterpret_cast<float4*>(sn) = __ldg(reinterpret_cast<const float4*>(cs + half + i));
    *reinterpret_cast<float4*>(sn + 4) = __ldg(reinterpret_cast<const float4*>(cs + half + i + 4));
    __nv_bfloat16* base = qkv + static_cast<size_t>(t) * row_stride + head * D;
    uint4* plo = reinterpret_cast<uint4*>(base + i);
    uint4* phi = reinterpret_cast<uint4*>(base + half + i);
    bf16x8_to_float(*plo, a);
    bf16x8_to_float(*phi, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sn[j] * sign;
      lo[j] = a[j] * c[j] - b[j] * s;
      hi[j] = b[j] * c[j] + a[j] * s;
    }
    *plo = float_to_bf16x8(lo);
    *phi = float_to_bf16x8(hi);
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on gu = [gate | up] of shape [T, 2F]
// ---------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                                  int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / fv;
    const int v = static_cast<int>(idx - t * fv);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    float g[8], u[8], o[8];
    bf16x8_to_float(row[v], g);
    bf16x8_to_float(row[fv + v], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<uint4*>(out + t * F)[v] = float_to_bf16x8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / fv;
    const int v = static_cast<int>(idx - t * fv);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    bf16x8_to_float(row[v], g);
    bf16x8_to_float(row[fv + v], u);
    bf16x8_to_float(reinterpret_cast<const uint4*>(dout + t * F)[v], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sig;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sig + silu * (1.f - sig));
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + t * 2 * F);
    orow[v] = float_to_bf16x8(dg);
    orow[fv + v] = float_to_bf16x8(du);
  }
}

// ---------------------------------------------------------------------------
// Flat fused AdamW (decoupled weight decay) over fp32 master / m / v shards.
// grad is fp32; grad_scale[0] (device) multiplies it (global-norm clip and loss
// scaling folded into one coefficient).  Writes the bf16 copy of the parameters.
// If skip_flag[0] != 0 (non-finite gradient norm) nothing is updated.
// ---------------------------------------------------------------------------
__global__ void adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                  const float* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n,
                                  float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                  const float* __restrict__ grad_scale, const int* __restrict__ skip_flag) {
  if (skip_flag && *skip_flag) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(master)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float* pp = reinterpret_cast<float*>(&p);
    float* pm = reinterpret_cast<float*>(&mm);
    float* pv = reinterpret_cast<float*>(&vv);
    const float* pg = reinterpret_cast<const float*>(&g4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g = pg[j] * gs;
      pm[j] = beta1 * pm[j] + (1.f - beta1) * g;
      pv[j] = beta2 * pv[j] + (1.f - beta2) * g * g;
      const float mhat = pm[j] / bc1;
      const float vhat = pv[j] / bc2;
      pp[j] = pp[j] * (1.f - lr * wd) - lr * mhat / (sqrtf(vhat) + eps);
    }
    reinterpret_cast<float4*>(master)[i] = p;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (param_bf16) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(param_bf16)[i] = o;
    }
  }
  // scalar tail
  const long long tail0 = nv << 2;
  for (long long i = tail0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = grad[i] * gs;
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float pnew = master[i] * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = pnew;
    if (param_bf16) param_bf16[i] = __float2bfloat16(pnew);
  }
}

// out[0] += sum(x^2)
__global__ void sqnorm_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  for (long long i = (nv << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    acc += x[i] * x[i];
  const float t = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, t);
}

// coef[0] = min(1, max_norm / (sqrt(sq[0]) + 1e-6)) * extra_scale ; skip[0] = !isfinite(norm); norm_out[0] = norm
__global__ void clip_coef_kernel(const float* __restrict__ sq, float max_norm, float extra_scale,
                                 float* __restrict__ coef, int* __restrict__ skip, float* __restrict__ norm_out) {
  const float norm = sqrtf(*sq) * fabsf(extra_scale);
  const bool finite = isfinite(norm);
  float c = extra_scale;
  if (max_norm > 0.f && finite) c *= fminf(1.f, max_norm / (norm + 1e-6f));
  *coef = c;
  *skip = finite ? 0 : 1;
  *norm_out = norm;
}

static inline int grid_for(long long work_items, int threads, int max_waves = 8) {
  const int sms = sm_count();
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sms) * max_waves;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace sb

extern "C" {

int sb_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* x_out, void* y, float* rstd, int T, int H,
                   float eps, void* stream) {
  if (H % 8 != 0 || H > sb::kNormThreads * 8 * sb::kNormMaxVec || T <= 0) return SB_ERR_ARG;
  if (H % 256 == 0 && H <= 2048) {
    const int blocks = (T + 7) / 8;
    const int wgrid = blocks < sb::sm_count() * 8 ? blocks : sb::sm_count() * 8;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define SB_NORM_FWD(NVV)                                                                                              \
  case NVV:                                                                                                           \
    sb::launch_pdl(sb::rmsnorm_fwd_warp_kernel<NVV>, dim3(wgrid), dim3(sb::kWarpNormThreads), 0, st,                  \
                   reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(delta),          \
                   reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(x_out),                \
                   reinterpret_cast<__nv_bfloat16*>(y), rstd, T, eps);                                                \
    return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
    switch (H / 256) {
      SB_NORM_FWD(1) SB_NORM_FWD(2) SB_NORM_FWD(3) SB_NORM_FWD(4) SB_NORM_FWD(5) SB_NORM_FWD(6) SB_NORM_FWD(7) SB_NORM_FWD(8)
    }
#undef SB_NORM_FWD
  }
  const int grid = T < sb::sm_count() * 8 ? T : sb::sm_count() * 8;
  sb::rmsnorm_fwd_kernel<<<grid, sb::kNormThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(delta),
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(x_out),
      reinterpret_cast<__nv_bfloat16*>(y), rstd, T, H, eps);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                   float* dw, int T, int H, void* stream) {
  if (H % 8 != 0 || H > sb::kNormThreads * 8 * sb::kNormMaxVec || T <= 0) return SB_ERR_ARG;
  if (H % 256 == 0 && H <= 2048) {
    const int blocks = (T + 7) / 8;
    const int wgrid = blocks < sb::sm_count() * 2 ? blocks : sb::sm_count() * 2;
    const int smem = 8 * H * static_cast<int>(sizeof(float));
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define SB_NORM_BWD(NVV)                                                                                              \
  case NVV: {                                                                                                         \
    static bool attr_dev[64] = {};                                                                                    \
    bool& attr = attr_dev[sb::device_index()];                                                                        \
    if (!attr) {                                                                                                      \
      cudaFuncSetAttribute(sb::rmsnorm_bwd_warp_kernel<NVV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2048 * 4); \
      attr = true;                                                                                                    \
    }                                                                                                                 \
    sb::rmsnorm_bwd_warp_kernel<NVV><<<wgrid, sb::kWarpNormThreads, smem, st>>>(                                      \
        reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),                        \
        reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<const __nv_bfloat16*>(dres),                \
        reinterpret_cast<__nv_bfloat16*>(dx), dw, T);                                                                 \
    return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;                                                   \
  }
    switch (H / 256) {
      SB_NORM_BWD(1) SB_NORM_BWD(2) SB_NORM_BWD(3) SB_NORM_BWD(4) SB_NORM_BWD(5) SB_NORM_BWD(6) SB_NORM_BWD(7) SB_NORM_BWD(8)
    }
#undef SB_NORM_BWD
  }
  const int grid = T < sb::sm_count() * 2 ? T : sb::sm_count() * 2;
  sb::rmsnorm_bwd_kernel<<<grid, sb::kNormThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<const __nv_bfloat16*>(dres),
      reinterpret_cast<__nv_bfloat16*>(dx), dw, T, H);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_rope_inplace(void* qkv, const int* pos, const float* cos_sin, int T, int n_rot_heads, int row_stride, int D,
                    float sign, void* stream) {
  if (D % 4 != 0 || T <= 0) return SB_ERR_ARG;
  if ((D % 16) == 0 && (row_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(cos_sin) & 15) == 0) {
    const long long total8 = static_cast<long long>(T) * n_rot_heads * (D / 16);
    sb::rope_inplace_vec8_kernel<<<sb::grid_for(total8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<__nv_bfloat16*>(qkv), pos, cos_sin, T, n_rot_heads, row_stride, D, sign);
    return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
  }
  const long long total = static_cast<long long>(T) * n_rot_heads * (D / 4);
  sb::rope_inplace_kernel<<<sb::grid_for(total, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(qkv), pos, cos_sin, T, n_rot_heads, row_stride, D, sign);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_swiglu_fwd(const void* gu, void* out, long long T, int F, void* stream) {
  if (F % 8 != 0 || T <= 0) return SB_ERR_ARG;
  sb::launch_pdl(sb::swiglu_fwd_kernel, dim3(sb::grid_for(T * (F / 8), 256)), dim3(256), 0,
                 reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(gu),
                 reinterpret_cast<__nv_bfloat16*>(out), T, F);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int F, void* stream) {
  if (F % 8 != 0 || T <= 0) return SB_ERR_ARG;
  sb::swiglu_bwd_kernel<<<sb::grid_for(T * (F / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<const __nv_bfloat16*>(dout),
      reinterpret_cast<__nv_bfloat16*>(dgu), T, F);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_adamw_flat(float* master, float* m, float* v, const float* grad, void* param_bf16, long long n, float lr,
                  float beta1, float beta2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
                  const int* skip_flag, void* stream) {
  if (n <= 0) return SB_OK;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(grad)) & 15)
    return SB_ERR_ARG;
  if (param_bf16 && (reinterpret_cast<uintptr_t>(param_bf16) & 7)) return SB_ERR_ARG;
  sb::adamw_flat_kernel<<<sb::grid_for(n / 4 + 1, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, reinterpret_cast<__nv_bfloat16*>(param_bf16), n, lr, beta1, beta2, eps, wd, bc1, bc2,
      grad_scale, skip_flag);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_sqnorm_accum(const float* x, long long n, float* out, void* stream) {
  if (n <= 0) return SB_OK;
  if (reinterpret_cast<uintptr_t>(x) & 15) return SB_ERR_ARG;
  sb::sqnorm_kernel<<<sb::grid_for(n / 4 + 1, 256, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, n, out);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_clip_coef(const float* sq, float max_norm, float extra_scale, float* coef, int* skip, float* norm_out,
                 void* stream) {
  sb::clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sq, max_norm, extra_scale, coef, skip,
                                                                           norm_out);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
