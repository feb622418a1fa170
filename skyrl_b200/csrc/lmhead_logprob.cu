// Fused LM-head log-probability / entropy: logits = hidden @ W^T are produced tile by tile in TMEM
// and reduced on the fly, so the [T, V] logits matrix never exists in memory.
//
// forward:  per (128-token block, vocabulary split) a persistent CTA runs the tcgen05 GEMM main loop
//           over 256-wide vocabulary chunks; the epilogue warps fold each chunk into per-row online
//           statistics  (max, sum exp, sum exp*z, target logit)  and write one partial per split.
//           A combine kernel merges the splits (and, for vocabulary-parallel ranks, the partials
//           of peer GPUs read through their pointers) into logprob, entropy and logsumexp.
// backward: for a block of rows whose logits were recomputed by the plain GEMM, one elementwise
//           kernel turns logits into dlogits in place:
//             dz_j = inv_T * ( g_lp * (1[j = target] - p_j)  -  g_ent * p_j * (log p_j + H) )
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kLmBM = 128;
constexpr int kLmBN = 256;
constexpr int kLmBK = 64;
constexpr int kLmStages = 4;
constexpr int kLmABytes = kLmBM * kLmBK * 2;
constexpr int kLmBBytes = kLmBN * kLmBK * 2;
constexpr int kLmStageBytes = kLmABytes + kLmBBytes;
constexpr int kLmSmem = kLmStages * kLmStageBytes + 1024 + 256;
constexpr int kLmThreads = 192;

// partial record per (row, split): {max, sumexp, sum exp*z, target logit or -inf}
__global__ void __launch_bounds__(kLmThreads, 1)
lmhead_fwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const int* __restrict__ targets, float4* __restrict__ partials, int T, int V, int K, int splits,
                  int chunks_per_split, int vocab_offset, float inv_temp, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kLmStages * kLmStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kLmStages;
  uint64_t* tfull = bars + 2 * kLmStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (T + kLmBM - 1) / kLmBM;
  const int items = m_blocks * splits;
  const int k_blocks = (K + kLmBK - 1) / kLmBK;
  const int n_chunks_total = (V + kLmBN - 1) / kLmBN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kLmStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  // item -> (split, m block): consecutive CTAs share the same vocabulary split so that the weight
  // chunk streams through L2 once per wave
  auto item_coords = [&](int item, int& pm, int& split, int& c0, int& c1) {
    split = item / m_blocks;
    pm = item - split * m_blocks;
    c0 = split * chunks_per_split;
    c1 = min(n_chunks_total, c0 + chunks_per_split);
  };

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        int pm, split, c0, c1;
        item_coords(item, pm, split, c0, c1);
        for (int c = c0; c < c1 && ok; ++c) {
          for (int kb = 0; kb < k_blocks; ++kb, ++it) {
            const int s = it % kLmStages;
            if (!mbar_wait(&empty[s], ((it / kLmStages) & 1) ^ 1, status, 0x701)) {
              ok = false;
              break;
            }
            uint8_t* sA = smem + s * kLmStageBytes;
            mbar_arrive_expect_tx(&full[s], kLmStageBytes);
            tma_load_2d(sA, &tmA, &full[s], kb * kLmBK, pm * kLmBM);
            tma_load_2d(sA + kLmABytes, &tmB, &full[s], kb * kLmBK, c * kLmBN);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kLmBM, kLmBN, false, false);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        int pm, split, c0, c1;
        item_coords(item, pm, split, c0, c1);
        for (int c = c0; c < c1 && ok; ++c, ++tcount) {
          const int acc = tcount & 1;
          if (!mbar_wait(&tempty[acc], ((tcount >> 1) & 1) ^ 1, status, 0x711)) {
            ok = false;
            break;
          }
          tc_fence_after();
          for (int kb = 0; kb < k_blocks; ++kb, ++it) {
            const int s = it % kLmStages;
            if (!mbar_wait(&full[s], (it / kLmStages) & 1, status, 0x712)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_base = smem_u32(smem + s * kLmStageBytes);
            const uint32_t b_base = a_base + kLmABytes;
#pragma unroll
            for (int k = 0; k < kLmBK / 16; ++k)
              umma_f16(tmem_base + acc * kLmBN, make_smem_desc(a_base + k * 32, 0, 1024),
                       make_smem_desc(b_base + k * 32, 0, 1024), idesc, (kb | k) != 0);
            umma_commit(&empty[s]);
          }
          if (ok) umma_commit(&tfull[acc]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    int tcount = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      int pm, split, c0, c1;
      item_coords(item, pm, split, c0, c1);
      const int row = pm * kLmBM + q * 32 + lane;
      const int tgt = (row < T) ? targets[row] - vocab_offset : -1;
      float m = -INFINITY, s = 0.f, sz = 0.f, zt = -INFINITY;
      for (int c = c0; c < c1; ++c, ++tcount) {
        const int acc = tcount & 1;
        if (!mbar_wait(&tfull[acc], (tcount >> 1) & 1, status, 0x721)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int cc = 0; cc < kLmBN / 32; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + acc * kLmBN + cc * 32 + lane_off, r);
          tmem_ld_wait();
          const int col0 = c * kLmBN + cc * 32;
          if (col0 >= V) continue;
          float z[32];
          float cm = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            z[i] = (col0 + i < V) ? __uint_as_float(r[i]) * inv_temp : -INFINITY;
            cm = fmaxf(cm, z[i]);
          }
          if (tgt >= col0 && tgt < col0 + 32) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i == tgt) zt = z[i];
          }
          const float mn = fmaxf(m, cm);
          const float alpha = __expf(m - mn);
          float ps = 0.f, pz = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float e = __expf(z[i] - mn);
            ps += e;
            pz += (col0 + i < V) ? e * z[i] : 0.f;
          }
          s = s * alpha + ps;
          sz = sz * alpha + pz;
          m = mn;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
      }
      if (ok && row < T) partials[static_cast<size_t>(row) * splits + split] = make_float4(m, s, sz, zt);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Merge `n_src` partial arrays (this rank's and, for vocabulary parallelism, its peers') of `splits`
// records per row.  logprob = z_target - lse; entropy = lse - E_p[z].
struct PartialSources {
  const float4* ptr[8];
};

__global__ void lmhead_combine_kernel(PartialSources src, int n_src, int splits, int T, float* __restrict__ logprob,
                                      float* __restrict__ entropy, float* __restrict__ lse_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= T) return;
  float m = -INFINITY, s = 0.f, sz = 0.f, zt = -INFINITY;
  for (int k = 0; k < n_src; ++k) {
    const float4* p = src.ptr[k] + static_cast<size_t>(row) * splits;
    for (int i = 0; i < splits; ++i) {
      const float4 v = p[i];
      if (v.x == -INFINITY) continue;
      const float mn = fmaxf(m, v.x);
      const float a = __expf(m - mn), b = __expf(v.x - mn);
      s = s * a + v.y * b;
      sz = sz * a + v.z * b;
      m = mn;
      zt = fmaxf(zt, v.w);
    }
  }
  const float lse = m + __logf(s);
  if (logprob) logprob[row] = zt - lse;
  if (entropy) entropy[row] = lse - sz / s;
  if (lse_out) lse_out[row] = lse;
}

// In place: logits (bf16, [rows, V] with row stride ld, this rank's vocabulary slice) -> dlogits.
__global__ void lmhead_dlogits_kernel(__nv_bfloat16* __restrict__ logits, long long ld, int rows, int V,
                                      const int* __restrict__ targets, int vocab_offset, const float* __restrict__ lse,
                                      const float* __restrict__ entropy, const float* __restrict__ g_lp,
                                      const float* __restrict__ g_ent, float inv_temp) {
  const int row = blockIdx.y;
  if (row >= rows) return;
  const float l = lse[row];
  const float glp = g_lp ? g_lp[row] : 0.f;
  const float gen = g_ent ? g_ent[row] : 0.f;
  const float H = (g_ent && entropy) ? entropy[row] : 0.f;
  const int tgt = targets[row] - vocab_offset;
  __nv_bfloat16* zr = logits + static_cast<size_t>(row) * ld;
  const int nvec = V >> 3;
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += gridDim.x * blockDim.x) {
    uint4 raw = reinterpret_cast<uint4*>(zr)[v];
    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
    float o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p2[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float z = o[i] * inv_temp;
      const float logp = z - l;
      const float p = __expf(logp);
      const int col = v * 8 + i;
      o[i] = inv_temp * (glp * ((col == tgt ? 1.f : 0.f) - p) - gen * p * (logp + H));
    }
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]);
    w.y = pack_bf16x2(o[2], o[3]);
    w.z = pack_bf16x2(o[4], o[5]);
    w.w = pack_bf16x2(o[6], o[7]);
    reinterpret_cast<uint4*>(zr)[v] = w;
  }
  if (blockIdx.x == 0) {
    for (int col = (nvec << 3) + threadIdx.x; col < V; col += blockDim.x) {
      const float z = __bfloat162float(zr[col]) * inv_temp;
      const float logp = z - l;
      const float p = __expf(logp);
      zr[col] = __float2bfloat16(inv_temp * (glp * ((col == tgt ? 1.f : 0.f) - p) - gen * p * (logp + H)));
    }
  }
}

}  // namespace sb

extern "C" {

// Number of float4 partial records per row that sb_lmhead_partials writes for a vocabulary of V.
int sb_lmhead_num_splits(int T, int V) {
  const int m_blocks = (T + sb::kLmBM - 1) / sb::kLmBM;
  const int chunks = (V + sb::kLmBN - 1) / sb::kLmBN;
  const int sms = sb::sm_count();
  int splits = (2 * sms + m_blocks - 1) / m_blocks;  // aim for >= 2 waves of work items
  if (splits > chunks) splits = chunks;
  if (splits < 1) splits = 1;
  const int cps = (chunks + splits - 1) / splits;
  return (chunks + cps - 1) / cps;
}

// hidden [T, K] bf16 (row stride ldh), W [V, K] bf16 (row stride ldw), targets [T] int32 (global vocabulary
// ids; this rank owns [vocab_offset, vocab_offset + V)), partials: float4 [T, splits].
int sb_lmhead_partials(const void* hidden, const void* W, const int* targets, void* partials, int T, int V, int K,
                       long long ldh, long long ldw, int vocab_offset, float inv_temp, void* stream) {
  if (T <= 0 || V <= 0 || K <= 0 || (ldh & 7) || (ldw & 7)) return SB_ERR_ARG;
  const CUtensorMap* ta = sb::get_tmap_bf16_2d(hidden, T, K, ldh, sb::kLmBM);
  const CUtensorMap* tb = sb::get_tmap_bf16_2d(W, V, K, ldw, sb::kLmBN);
  if (!ta || !tb) return SB_ERR_TMAP;
  if (sb::device_status_ptr() == nullptr) return SB_ERR_CUDA;
  static bool attr_set_dev[64] = {};  // function attributes are per device
  bool& attr_set = attr_set_dev[sb::device_index()];
  if (!attr_set) {
    if (cudaFuncSetAttribute(sb::lmhead_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sb::kLmSmem) !=
        cudaSuccess)
      return SB_ERR_CUDA;
    attr_set = true;
  }
  const int splits = sb_lmhead_num_splits(T, V);
  const int chunks = (V + sb::kLmBN - 1) / sb::kLmBN;
  const int cps = (chunks + splits - 1) / splits;
  const int m_blocks = (T + sb::kLmBM - 1) / sb::kLmBM;
  const int items = m_blocks * splits;
  const int grid = items < sb::sm_count() ? items : sb::sm_count();
  sb::lmhead_fwd_kernel<<<grid, sb::kLmThreads, sb::kLmSmem, reinterpret_cast<cudaStream_t>(stream)>>>(
      *ta, *tb, targets, reinterpret_cast<float4*>(partials), T, V, K, splits, cps, vocab_offset, inv_temp,
      sb::device_status_ptr());
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

// Combine n_src (<= 8) partial arrays; any of logprob / entropy / lse may be null.
int sb_lmhead_combine(const void* const* partial_ptrs, int n_src, int splits, int T, float* logprob, float* entropy,
                      float* lse, void* stream) {
  if (n_src < 1 || n_src > 8 || T <= 0) return SB_ERR_ARG;
  sb::PartialSources src;
  for (int i = 0; i < 8; ++i) src.ptr[i] = i < n_src ? reinterpret_cast<const float4*>(partial_ptrs[i]) : nullptr;
  sb::lmhead_combine_kernel<<<(T + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(src, n_src, splits, T,
                                                                                               logprob, entropy, lse);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_lmhead_dlogits(void* logits, long long ld, int rows, int V, const int* targets, int vocab_offset,
                      const float* lse, const float* entropy, const float* g_lp, const float* g_ent, float inv_temp,
                      void* stream) {
  if (rows <= 0 || V <= 0 || (ld & 7)) return SB_ERR_ARG;
  int bx = (V / 8 + 255) / 256;
  if (bx > 64) bx = 64;
  if (bx < 1) bx = 1;
  dim3 grid(bx, rows);
  sb::lmhead_dlogits_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(logits), ld, rows, V, targets, vocab_offset, lse, entropy, g_lp, g_ent, inv_temp);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in lmhead_noalloc.h).
// ---------------------------------------------------------------------------------------------------------
#include "lmhead_noalloc.h"

#include <atomic>
#include <mutex>

namespace sb {

// Scratch for the per-(row, split) records of the no-alloc entry point: lives in the device image of
// every GPU that loads this library.  In host code this name is only a stand-in for the symbol; the
// device address is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) float4 g_lmhead_noalloc_scratch[SB_LMHEAD_NOALLOC_MAX_RECORDS];

typedef CUresult (*NoAllocEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct NoAllocDeviceState {
  float4* scratch = nullptr;
  int* status = nullptr;
  bool ready = false;
  std::mutex mu;  // serialises the one-time set-up of this device among host threads
};
static NoAllocDeviceState g_noalloc_state[64];
static std::atomic<NoAllocEncodeFn> g_noalloc_encode{nullptr};

// Once per device, with that device current: resolve the scratch address and configure the kernel.
// Safe to race from several host threads: the first one does the work under the device's mutex.
static int noalloc_setup(int dev) {
  NoAllocDeviceState& st = g_noalloc_state[dev];
  std::lock_guard<std::mutex> lock(st.mu);
  if (st.ready) return SB_OK;
  cudaFree(nullptr);  // bind the primary context to this thread (frees nothing, allocates nothing)
  float4* ptr = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_lmhead_noalloc_scratch) != cudaSuccess || ptr == nullptr)
    return SB_ERR_CUDA;
  if (cudaFuncSetAttribute(lmhead_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLmSmem) != cudaSuccess)
    return SB_ERR_CUDA;
  int* status = device_status_ptr();
  if (status == nullptr) return SB_ERR_CUDA;
  if (!g_noalloc_encode.load()) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !fn)
      return SB_ERR_TMAP;
    g_noalloc_encode.store(reinterpret_cast<NoAllocEncodeFn>(fn));
  }
  st.scratch = ptr;
  st.status = status;
  st.ready = true;
  return SB_OK;
}

// Tensor map built in caller-provided (stack) storage: no cache, no heap.
static int noalloc_encode_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                             uint32_t box_rows) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) return SB_ERR_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_noalloc_encode.load()(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SB_OK : SB_ERR_TMAP;
}

}  // namespace sb

extern "C" int sb_lmhead_logprob_noalloc(const void* hidden, const void* W, const int* targets, int T, int V, int K,
                                         long long ldh, long long ldw, float inv_temp, float* logprob, float* entropy,
                                         float* lse, void* stream) {
  if (T <= 0 || V <= 0 || K <= 0 || (ldh & 7) || (ldw & 7) || !hidden || !W || !targets) return SB_ERR_ARG;
  const int splits = sb_lmhead_num_splits(T, V);
  if (static_cast<long long>(T) * splits > SB_LMHEAD_NOALLOC_MAX_RECORDS) return SB_ERR_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SB_ERR_CUDA;
  int rc = sb::noalloc_setup(dev);
  if (rc != SB_OK) return rc;
  alignas(64) CUtensorMap ta, tb;
  rc = sb::noalloc_encode_2d(&ta, hidden, T, K, ldh, sb::kLmBM);
  if (rc != SB_OK) return rc;
  rc = sb::noalloc_encode_2d(&tb, W, V, K, ldw, sb::kLmBN);
  if (rc != SB_OK) return rc;
  float4* scratch = sb::g_noalloc_state[dev].scratch;  // device address, not the host-side symbol
  const int chunks = (V + sb::kLmBN - 1) / sb::kLmBN;
  const int cps = (chunks + splits - 1) / splits;
  const int m_blocks = (T + sb::kLmBM - 1) / sb::kLmBM;
  const int items = m_blocks * splits;
  const int grid = items < sb::sm_count() ? items : sb::sm_count();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  sb::lmhead_fwd_kernel<<<grid, sb::kLmThreads, sb::kLmSmem, st>>>(ta, tb, targets, scratch, T, V, K, splits, cps, 0,
                                                                  inv_temp, sb::g_noalloc_state[dev].status);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_CUDA;
  sb::PartialSources src;
  for (int i = 0; i < 8; ++i) src.ptr[i] = i == 0 ? scratch : nullptr;
  sb::lmhead_combine_kernel<<<(T + 255) / 256, 256, 0, st>>>(src, 1, splits, T, logprob, entropy, lse);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}
