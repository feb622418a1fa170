// Peer-memory communication over NVLink / NVSwitch, issued from kernels (no NCCL on these paths).
//
//   * symmetric allocations: cudaMalloc + CUDA IPC handles, exchanged by the host bootstrap, so that every
//     rank holds a device pointer to every peer's buffer;
//   * peer_barrier: release/acquire flags at system scope with a bounded spin -- a rank that never shows up
//     makes the others record a status code and return instead of hanging;
//   * reduce-scatter of fp32 gradients by peer loads, fused with the squared-norm partial of the owned shard;
//   * AdamW on the owned shard fused with the bf16 parameter push to every peer's parameter buffer: the
//     all-gather of ZeRO and the trainer->rollout weight sync are the same stores;
//   * one-shot all-reduce (sum) of small bf16 activations for tensor-parallel decode.
// Loads from peers are plain ld.global through the mapped pointer; no bulk/tensor copy ever reads a peer.
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// pads.p[r] points at rank r's signal pad (int[kMaxPeers * channels]); slot [channel * kMaxPeers + src].
// Thread t signals peer t and waits for peer t's signal. wait_ns bounds the spin.
__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int world, int channel, int epoch,
                                    unsigned long long wait_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys(static_cast<int*>(pads.p[t]) + channel * kMaxPeers + rank, epoch);
  const int* mine = static_cast<const int*>(pads.p[rank]) + channel * kMaxPeers + t;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(mine) < epoch) {
    if (globaltimer_ns() - t0 > wait_ns) {
      atomicCAS(status, 0, 0x900 | t);
      return;
    }
    __nanosleep(64);
  }
}

// Same barrier for launch sequences that are replayed from a CUDA graph: the epoch cannot be a kernel argument there
// (it would be frozen at capture time), so it lives in device memory and every launch advances it by one.  All ranks
// run the same launch sequence, so their counters stay equal without any exchange.
__global__ void peer_barrier_counter_kernel(PeerPtrs pads, int rank, int world, int channel, int* epoch_counter,
                                            unsigned long long wait_ns, int* status) {
  __shared__ int epoch_s;
  pdl_launch_dependents();
  pdl_wait();  // the predecessor's stores (its peer stores included) are complete and visible before we signal
  if (threadIdx.x == 0) {
    epoch_s = *epoch_counter + 1;
    *epoch_counter = epoch_s;
  }
  __syncthreads();
  const int t = threadIdx.x;
  if (t >= world) return;
  const int epoch = epoch_s;
  __threadfence_system();
  st_release_sys(static_cast<int*>(pads.p[t]) + channel * kMaxPeers + rank, epoch);
  const int* mine = static_cast<const int*>(pads.p[rank]) + channel * kMaxPeers + t;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(mine) < epoch) {
    if (globaltimer_ns() - t0 > wait_ns) {
      atomicCAS(status, 0, 0x910 | t);
      return;
    }
    __nanosleep(32);
  }
}

// out[i] = sum_r grads[r][lo + i]; sq_partial += sum(out^2). All ranks' grads must be complete (barrier before).
__global__ void peer_reduce_scatter_kernel(PeerPtrs grads, int world, long long lo, long long n,
                                           float* __restrict__ out, float* __restrict__ sq_partial) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        const float4 v = reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + lo)[i];
        s.x += v.x;
        s.y += v.y;
        s.z += v.z;
        s.w += v.w;
      }
    }
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) atomicAdd(sq_partial, t);
  }
}

// Publishes this rank's squared-norm partial into slot [rank] of every peer's norm pad.
__global__ void peer_publish_scalar_kernel(PeerPtrs pads, int rank, int world, const float* __restrict__ value) {
  const int t = threadIdx.x;
  if (t < world) static_cast<float*>(pads.p[t])[rank] = *value;
}

// AdamW on the owned shard + bf16 push of the new parameters into every peer's parameter buffer.
// The clip coefficient is derived in-kernel from the world's squared-norm partials (norm_pad[0..world)).
__global__ void peer_adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                       const float* __restrict__ grad, PeerPtrs params, int world, long long lo,
                                       long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                       float bc2, const float* __restrict__ norm_pad, float max_norm, float grad_scale,
                                       float* __restrict__ norm_out, int* __restrict__ skipped,
                                       const int* __restrict__ status) {
  float sq = 0.f;
  for (int r = 0; r < world; ++r) sq += norm_pad[r];
  const float norm = sqrtf(sq) * fabsf(grad_scale);
  const bool finite = isfinite(norm);
  // a bounded wait that gave up earlier in this step (a peer never reached a barrier) means the reduced gradients
  // may be incomplete: publish nothing, the host reads the status word after the step and raises
  const bool broken = *reinterpret_cast<const volatile int*>(status) != 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *norm_out = norm;
    *skipped = broken ? 2 : (finite ? 0 : 1);
  }
  if (!finite || broken) return;  // leave parameters and moments untouched everywhere
  float gs = grad_scale;
  if (max_norm > 0.f) gs *= fminf(1.f, max_norm / (norm + 1e-6f));
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
      pp[j] = pp[j] * (1.f - lr * wd) - lr * (pm[j] / bc1) / (sqrtf(pv[j] / bc2) + eps);
    }
    reinterpret_cast<float4*>(master)[i] = p;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(params.p[r]) + lo)[i] = o;
  }
}

// Plain push: dst[r][dst_off + i] = src[i] (bf16) to `n_dst` destinations (weight sync into engine buffers).
__global__ void peer_push_bf16_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, int n_dst, long long dst_off,
                                      long long n) {
  const long long nv = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(src)[i];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_dst) reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(dst.p[r]) + dst_off)[i] = v;
  }
}

// fp32 master shard -> bf16 pushed to n_dst destinations (cast fused with the transfer).
__global__ void peer_push_cast_kernel(const float* __restrict__ src, PeerPtrs dst, int n_dst, long long dst_off,
                                      long long n) {
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < n_dst) reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(dst.p[r]) + dst_off)[i] = o;
  }
}

// One-shot all-reduce for small tensors: every rank reads all peers' buffers and sums (bf16 in, bf16 out).
// Inputs must be complete on every rank (barrier before) and must not be overwritten until all have read
// (barrier after, or double buffering by the caller).
__global__ void peer_allreduce_bf16_kernel(PeerPtrs bufs, int world, __nv_bfloat16* __restrict__ out, long long n) {
  const long long nv = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        const uint4 v = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(bufs.p[r]))[i];
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p2[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

static inline int comm_grid(long long items, int threads) {
  long long b = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

static inline PeerPtrs make_ptrs(void* const* ptrs, int n) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = i < n ? ptrs[i] : nullptr;
  return pp;
}

}  // namespace sb

extern "C" {

int sb_symm_alloc(unsigned long long bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return SB_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) return SB_ERR_CUDA;
  *out = p;
  return SB_OK;
}
int sb_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? SB_OK : SB_ERR_CUDA; }
int sb_ipc_get_handle(void* p, char* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return SB_ERR_CUDA;
  memcpy(out64, &h, sizeof(h));
  return SB_OK;
}
int sb_ipc_open_handle(const char* in64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return SB_ERR_CUDA;
  *out = p;
  return SB_OK;
}
int sb_ipc_close_handle(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? SB_OK : SB_ERR_CUDA; }

int sb_peer_barrier(void* const* pads, int rank, int world, int channel, int epoch, unsigned long long wait_ns,
                    void* stream) {
  if (world < 1 || world > sb::kMaxPeers || channel < 0 || channel >= 8) return SB_ERR_ARG;
  int* st = sb::device_status_ptr();
  if (st == nullptr) return SB_ERR_CUDA;
  sb::peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sb::make_ptrs(pads, world), rank, world, channel, epoch, wait_ns, st);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_barrier_counter(void* const* pads, int rank, int world, int channel, int* epoch_counter,
                            unsigned long long wait_ns, void* stream) {
  if (world < 1 || world > sb::kMaxPeers || channel < 0 || channel >= 8 || !epoch_counter) return SB_ERR_ARG;
  int* st = sb::device_status_ptr();
  if (st == nullptr) return SB_ERR_CUDA;
  const cudaError_t e = sb::launch_pdl(sb::peer_barrier_counter_kernel, dim3(1), dim3(32), 0,
                                       reinterpret_cast<cudaStream_t>(stream), sb::make_ptrs(pads, world), rank, world, channel,
                                       epoch_counter, wait_ns, st);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_reduce_scatter_f32(void* const* grads, int world, long long lo, long long n, float* out, float* sq_partial,
                               void* stream) {
  if (world < 1 || world > sb::kMaxPeers || (n & 3) || (lo & 3)) return SB_ERR_ARG;
  sb::peer_reduce_scatter_kernel<<<sb::comm_grid(n / 4, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sb::make_ptrs(grads, world), world, lo, n, out, sq_partial);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_publish_scalar(void* const* pads, int rank, int world, const float* value, void* stream) {
  if (world < 1 || world > sb::kMaxPeers) return SB_ERR_ARG;
  sb::peer_publish_scalar_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sb::make_ptrs(pads, world), rank,
                                                                                       world, value);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_adamw_push(float* master, float* m, float* v, const float* grad, void* const* params, int world,
                       long long lo, long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                       float bc2, const float* norm_pad, float max_norm, float grad_scale, float* norm_out, int* skipped,
                       void* stream) {
  if (world < 1 || world > sb::kMaxPeers || (n & 3) || (lo & 3)) return SB_ERR_ARG;
  const int* st = sb::device_status_ptr();
  if (st == nullptr) return SB_ERR_CUDA;
  sb::peer_adamw_push_kernel<<<sb::comm_grid(n / 4, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, m, v, grad, sb::make_ptrs(params, world), world, lo, n, lr, beta1, beta2, eps, wd, bc1, bc2, norm_pad,
      max_norm, grad_scale, norm_out, skipped, st);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_push_bf16(const void* src, void* const* dst, int n_dst, long long dst_off, long long n, void* stream) {
  if (n_dst < 1 || n_dst > sb::kMaxPeers || (n & 7) || (dst_off & 7)) return SB_ERR_ARG;
  sb::peer_push_bf16_kernel<<<sb::comm_grid(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), sb::make_ptrs(dst, n_dst), n_dst, dst_off, n);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_push_cast(const float* src, void* const* dst, int n_dst, long long dst_off, long long n, void* stream) {
  if (n_dst < 1 || n_dst > sb::kMaxPeers || (n & 3) || (dst_off & 3)) return SB_ERR_ARG;
  sb::peer_push_cast_kernel<<<sb::comm_grid(n / 4, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      src, sb::make_ptrs(dst, n_dst), n_dst, dst_off, n);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_peer_allreduce_bf16(void* const* bufs, int world, void* out, long long n, void* stream) {
  if (world < 1 || world > sb::kMaxPeers || (n & 7)) return SB_ERR_ARG;
  sb::peer_allreduce_bf16_kernel<<<sb::comm_grid(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sb::make_ptrs(bufs, world), world, reinterpret_cast<__nv_bfloat16*>(out), n);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
