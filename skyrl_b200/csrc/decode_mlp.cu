// Decode path: everything between the attention kernel of one layer and the QKV projection of the next as ONE
// persistent kernel.
//
//   phase 1  o-proj:      part[s] = att[:, k-slice s] @ Wo[:, k-slice s]^T           (tcgen05, split-K, fp32 partials)
//   phase 2  norm:        x += sum_s part[s] ; h_mid = rmsnorm(x) * ln_mid
//   phase 3  gate/up:     act = silu(h_mid @ Wg^T) * (h_mid @ Wu^T)                   (tcgen05, SwiGLU in the epilogue)
//   phase 4  down-proj:   part[s] = act[:, k-slice s] @ Wd[:, k-slice s]^T           (tcgen05, split-K, fp32 partials)
//   phase 5  norm:        x += sum_s part[s] ; h_out = rmsnorm(x) * ln_out           (input of the next layer / LM head)
//
// A decode step has a few hundred rows at most, so each of these five pieces is a kernel of a few microseconds whose
// cost is mostly its launch, its prologue (barrier set-up, tensor-memory allocation, first TMA round trip) and its
// drain.  Here the CTAs (one per SM) stay resident: barriers, tensor memory and the TMA/MMA pipeline are set up once
// and carried from phase to phase, and the phases are separated by a grid-wide barrier (an arrival counter in global
// memory) instead of a kernel boundary.
//
// Tiles: up to 256 rows are handled as two 128-row MMA blocks that share every weight tile, so each weight byte is
// read from HBM exactly once per step and is used by both row blocks while it sits in shared memory.  A stage of the
// ring holds A rows 0..127, A rows 128..255 and one 128-row weight tile (48 KB, four stages).  For gate/up the weight
// tile is 64 gate rows followed by the matching 64 up rows, so the SwiGLU of a column needs no second tile.
//
// All CTAs must be resident at the same time (they wait for each other); the launch is cooperative, so the driver
// either guarantees that or refuses the launch.  Every wait is bounded: a barrier that does not complete records a
// code in the status word and the kernel unwinds (tensor memory is released on every path).
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

constexpr int kDmThreads = 192;  // warp 0: TMA producer, warp 1: MMA issuer + TMEM owner, warps 2..5: epilogue
constexpr int kDmStages = 4;
constexpr int kDmTile = 128 * 64 * 2;        // one [128 x 64] bf16 tile, 128-byte swizzled
constexpr int kDmStageBytes = 3 * kDmTile;   // A rows 0..127 | A rows 128..255 | B
constexpr int kDmStageLd = 36;                // words per row of an epilogue staging tile (32 + 4: conflict-free 16-byte accesses)
constexpr int kDmStagingBytes = 4 * 32 * kDmStageLd * 4;  // one 32-row tile per epilogue warp
constexpr int kDmSmem = kDmStages * kDmStageBytes + 1024 /*align*/ + 256 /*barriers*/ + kDmStagingBytes;
constexpr int kDmTmemCols = 512;             // 2 accumulator buffers x 2 row blocks x 128 columns
constexpr int kDmMaxVec = 4;                 // hidden size <= 192 * 8 * 4
constexpr int kDmMaxRows = 256;

struct DmArgs {
  int n;                         // rows (sequences in the decode batch), 1..256
  int H, Q, F;                   // hidden size, attention output width, FFN width
  int splits_o, splits_d;        // k slices of the o-proj / down-proj
  float eps;
  __nv_bfloat16* x;              // residual stream [n, H], updated in place
  const __nv_bfloat16* ln_mid;   // post-attention norm weight [H]
  const __nv_bfloat16* ln_out;   // next layer's input norm (or the final norm) weight [H]
  __nv_bfloat16* h_mid;          // [n, H] workspace: input of gate/up
  __nv_bfloat16* act;            // [n, F] workspace: input of down-proj
  __nv_bfloat16* h_out;          // [n, H] result
  float* part;                   // [max(splits_o, splits_d), n, H] fp32 workspace
  unsigned long long* bar;       // grid barrier: one 64-bit arrival counter (zero before the first launch)
  unsigned long long* trace;     // optional [gridDim.x, 16] timestamps at the phase boundaries (profiling aid)
};

namespace {

__device__ __forceinline__ void dm_fence_proxy_async() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ float dm_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Grid-wide barrier on ONE monotonically increasing 64-bit arrival counter: barrier number k of this launch is passed
// when the counter reaches base + (k + 1) * gridDim.x.  A launch adds exactly kDmBarriers * gridDim.x, so `base` is
// the counter rounded down to a multiple of that, whenever it is read before the launch's last barrier completes.
// One release-add and an acquire poll per CTA: no reset, no second word.  `to_async`: the data written before the
// barrier is read by TMA after it, so the writers also order their stores against the async proxy.
// Returns false when the wait gave up (the counter is then inconsistent and must be zeroed by the host).
constexpr int kDmBarriers = 4;

__device__ __forceinline__ unsigned long long dm_ld_acquire64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool dm_grid_barrier(unsigned long long* counter, unsigned long long target, bool to_async,
                                                int* status, int code, int* s_ok, unsigned long long* tr = nullptr) {
  if (to_async) dm_fence_proxy_async();
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    if (tr) tr[0] = globaltimer_ns();
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(counter) : "memory");
    if (tr) tr[1] = globaltimer_ns();
    unsigned long long polls = 0;
    if (dm_ld_acquire64(counter) < target) {
      const unsigned long long t0 = globaltimer_ns();
      while (dm_ld_acquire64(counter) < target) {
        ++polls;
        if ((polls & 63) == 0 &&
            (*reinterpret_cast<volatile int*>(status) != 0 || globaltimer_ns() - t0 > kWaitTimeoutNs)) {
          atomicCAS(status, 0, code);
          ok = 0;
          break;
        }
      }
    }
    if (tr) {
      tr[2] = globaltimer_ns();
      tr[3] = polls;
    }
    *s_ok = ok;
  }
  __syncthreads();
  return *s_ok != 0;
}

struct DmPipe {
  uint8_t* smem;
  uint64_t *full, *empty, *tfull, *tempty;
  uint32_t* stage;  // epilogue staging tiles
  uint32_t tmem_base;
  int it;      // k-block counter (producer and MMA thread advance it identically)
  int tcount;  // accumulator-use counter (MMA thread and epilogue warps advance it identically)
};

// One GEMM phase over all work items (n-tile, k-slice) of this CTA.  SWIGLU = false: fp32 partial tiles to
// out_f32 + ks * n * N; SWIGLU = true: the tile is 64 gate + 64 up columns and silu(gate) * up goes to out_bf16.
template <bool SWIGLU>
__device__ __forceinline__ void dm_gemm_phase(DmPipe& p, const CUtensorMap* tmA, const CUtensorMap* tmB, int n, int n_tiles,
                                              int k_blocks, int splits, int up_row0, float* out_f32,
                                              __nv_bfloat16* out_bf16, int ld_out, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mb = n > 128 ? 2 : 1;
  const int items = n_tiles * splits;
  const int kpb = (k_blocks + splits - 1) / splits;
  if (warp == 0) {
    if (lane == 0) {
      dm_fence_proxy_async();  // A may have been written by other CTAs' generic stores in the previous phase
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int pn = item % n_tiles, ks = item / n_tiles;
        const int kb0 = ks * kpb, kb1 = min(k_blocks, kb0 + kpb);
        for (int kb = kb0; kb < kb1; ++kb, ++p.it) {
          const int s = p.it % kDmStages;
          const uint32_t ph = (p.it / kDmStages) & 1;
          if (!mbar_wait(&p.empty[s], ph ^ 1, status, 0x701)) {
            ok = false;
            break;
          }
          uint8_t* sA = p.smem + s * kDmStageBytes;
          uint8_t* sB = sA + 2 * kDmTile;
          mbar_arrive_expect_tx(&p.full[s], (mb + 1) * kDmTile);
          tma_load_2d(sA, tmA, &p.full[s], kb * 64, 0);
          if (mb == 2) tma_load_2d(sA + kDmTile, tmA, &p.full[s], kb * 64, 128);
          if (SWIGLU) {
            tma_load_2d(sB, tmB, &p.full[s], kb * 64, pn * 64);
            tma_load_2d(sB + kDmTile / 2, tmB, &p.full[s], kb * 64, up_row0 + pn * 64);
          } else {
            tma_load_2d(sB, tmB, &p.full[s], kb * 64, pn * 128);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, false);
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int ks = item / n_tiles;
        const int kb0 = ks * kpb, kb1 = min(k_blocks, kb0 + kpb);
        const int acc = p.tcount & 1;
        const uint32_t aph = (p.tcount >> 1) & 1;
        ++p.tcount;
        if (!mbar_wait(&p.tempty[acc], aph ^ 1, status, 0x702)) break;
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb, ++p.it) {
          const int s = p.it % kDmStages;
          const uint32_t ph = (p.it / kDmStages) & 1;
          if (!mbar_wait(&p.full[s], ph, status, 0x703)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(p.smem + s * kDmStageBytes);
          const uint32_t b_base = a_base + 2 * kDmTile;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t bdesc = make_smem_desc(b_base + k * 32, 0, 1024);
            const uint32_t accum = (kb > kb0 || k != 0) ? 1u : 0u;
            umma_f16(p.tmem_base + acc * 256, make_smem_desc(a_base + k * 32, 0, 1024), bdesc, idesc, accum);
            if (mb == 2)
              umma_f16(p.tmem_base + acc * 256 + 128, make_smem_desc(a_base + kDmTile + k * 32, 0, 1024), bdesc, idesc,
                       accum);
          }
          umma_commit(&p.empty[s]);
        }
        if (ok) umma_commit(&p.tfull[acc]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quadrant of this warp
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int pn = item % n_tiles, ks = item / n_tiles;
      const int acc = p.tcount & 1;
      const uint32_t aph = (p.tcount >> 1) & 1;
      ++p.tcount;
      if (!mbar_wait(&p.tfull[acc], aph, status, 0x704)) break;
      tc_fence_after();
      // Each thread owns one accumulator row (32 consecutive columns per TMEM load).  Storing that straight to global
      // memory makes every warp store touch 32 different lines; instead the 32 x 32 block goes through a padded
      // shared-memory tile and leaves as whole 128-byte lines (8 lanes per row, 4 rows per store instruction).
      uint32_t* stg = p.stage + (warp - 2) * (32 * kDmStageLd);
      const int srow = lane >> 3, schunk = lane & 7;  // read side: row within a group of 4, 16-byte chunk of the row
      for (int m = 0; m < mb; ++m) {
        const int row0 = m * 128 + q * 32;
        const uint32_t t_row = p.tmem_base + acc * 256 + m * 128 + (static_cast<uint32_t>(q * 32) << 16);
        if (SWIGLU) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32b_x32(t_row + c * 32, rg);
            tmem_ld_32x32b_x32(t_row + 64 + c * 32, ru);
            tmem_ld_wait();
            // the unfused path rounds gate and up to bf16 before the activation; do the same
            uint32_t pa[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t pg = pack_bf16x2(__uint_as_float(rg[2 * j]), __uint_as_float(rg[2 * j + 1]));
              const uint32_t pu = pack_bf16x2(__uint_as_float(ru[2 * j]), __uint_as_float(ru[2 * j + 1]));
              const float g0 = __uint_as_float(pg << 16), g1 = __uint_as_float(pg & 0xFFFF0000u);
              const float u0 = __uint_as_float(pu << 16), u1 = __uint_as_float(pu & 0xFFFF0000u);
              pa[j] = pack_bf16x2(g0 * fmaf(0.5f, dm_tanh(0.5f * g0), 0.5f) * u0,
                                  g1 * fmaf(0.5f, dm_tanh(0.5f * g1), 0.5f) * u1);
            }
            uint4* w = reinterpret_cast<uint4*>(stg + lane * kDmStageLd + c * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) w[v] = make_uint4(pa[4 * v], pa[4 * v + 1], pa[4 * v + 2], pa[4 * v + 3]);
          }
          __syncwarp();
          // 32 rows x 64 bf16 (128 bytes per row)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + srow;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + r * kDmStageLd + schunk * 4);
            if (row0 + r < n)
              *reinterpret_cast<uint4*>(out_bf16 + static_cast<size_t>(row0 + r) * ld_out + pn * 64 + schunk * 8) = v;
          }
          __syncwarp();
        } else {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + c * 32, r);
            tmem_ld_wait();
            uint4* w = reinterpret_cast<uint4*>(stg + lane * kDmStageLd);
#pragma unroll
            for (int v = 0; v < 8; ++v) w[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + srow;
              const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * kDmStageLd + schunk * 4);
              if (row0 + rr < n)
                *reinterpret_cast<uint4*>(out_f32 + (static_cast<size_t>(ks) * n + row0 + rr) * ld_out + pn * 128 + c * 32 +
                                          schunk * 4) = v;
            }
            __syncwarp();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p.tempty[acc]);
    }
  }
  // the single-lane roles above leave warps 0 and 1 diverged; block-wide barriers follow, which want whole warps
  __syncwarp();
}

__device__ __forceinline__ void dm_ld_bf16x8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 dm_pack_bf16x8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// x[row] += sum of the partial rows (added in slice order, rounded to bf16 and stored: the statistics are those of
// the stored values); y[row] = x[row] * rstd * w.  Whole CTA per row; rows are dealt round-robin to the CTAs.
__device__ __forceinline__ void dm_norm_phase(__nv_bfloat16* x, const float* part, int n_part, const __nv_bfloat16* w,
                                              __nv_bfloat16* y, int n, int H, float eps, float* red) {
  const int nvec = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t pstride = static_cast<size_t>(n) * H;
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    float vals[kDmMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kDmMaxVec; ++i) {
      const int v = threadIdx.x + i * kDmThreads;
      if (v < nvec) {
        const size_t off = static_cast<size_t>(row) * H + v * 8;
        dm_ld_bf16x8(x + off, vals[i]);
        for (int s = 0; s < n_part; ++s) {
          const float4* pp = reinterpret_cast<const float4*>(part + s * pstride + off);
          const float4 a = pp[0], b = pp[1];
          vals[i][0] += a.x; vals[i][1] += a.y; vals[i][2] += a.z; vals[i][3] += a.w;
          vals[i][4] += b.x; vals[i][5] += b.y; vals[i][6] += b.z; vals[i][7] += b.w;
        }
        const uint4 rounded = dm_pack_bf16x8(vals[i]);
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
    ss = warp_sum(ss);
    __syncthreads();
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kDmThreads / 32; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
    for (int i = 0; i < kDmMaxVec; ++i) {
      const int v = threadIdx.x + i * kDmThreads;
      if (v < nvec) {
        float wv[8], o[8];
        dm_ld_bf16x8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * wv[j];
        *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H + v * 8) = dm_pack_bf16x8(o);
      }
    }
  }
}

}  // namespace

__global__ void __launch_bounds__(kDmThreads, 1)
decode_mlp_block_kernel(const __grid_constant__ CUtensorMap tm_att, const __grid_constant__ CUtensorMap tm_wo,
                        const __grid_constant__ CUtensorMap tm_hmid, const __grid_constant__ CUtensorMap tm_wgu,
                        const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_wd,
                        const __grid_constant__ DmArgs a, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float red[8];
  __shared__ int s_ok;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDmStages * kDmStageBytes);
  DmPipe p;
  p.smem = smem;
  p.full = bars;
  p.empty = bars + kDmStages;
  p.tfull = bars + 2 * kDmStages;
  p.tempty = p.tfull + 2;
  p.it = 0;
  p.tcount = 0;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p.tempty + 2);
  p.stage = reinterpret_cast<uint32_t*>(smem + kDmStages * kDmStageBytes + 256);
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDmStages; ++s) {
      mbar_init(&p.full[s], 1);
      mbar_init(&p.empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p.tfull[i], 1);
      mbar_init(&p.tempty[i], 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tm_att);
    tma_prefetch_desc(&tm_wo);
    tma_prefetch_desc(&tm_hmid);
    tma_prefetch_desc(&tm_wgu);
    tma_prefetch_desc(&tm_act);
    tma_prefetch_desc(&tm_wd);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kDmTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  p.tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  auto stamp = [&](int k) {
    if (a.trace != nullptr && threadIdx.x == 0) a.trace[blockIdx.x * 16 + k] = globaltimer_ns();
  };
  const unsigned long long per_launch = static_cast<unsigned long long>(kDmBarriers) * gridDim.x;
  const unsigned long long bar_base = (dm_ld_acquire64(a.bar) / per_launch) * per_launch;
  bool ok = true;
  stamp(0);
  // phase 1: o-proj partials
  dm_gemm_phase<false>(p, &tm_att, &tm_wo, a.n, a.H / 128, a.Q / 64, a.splits_o, 0, a.part, nullptr, a.H, status);
  __syncthreads();
  stamp(1);
  ok = dm_grid_barrier(a.bar, bar_base + 1ull * gridDim.x, false, status, 0x711, &s_ok,
                       a.trace ? a.trace + blockIdx.x * 16 + 10 : nullptr);
  stamp(2);
  // phase 2: residual add + post-attention norm
  if (ok) {
    dm_norm_phase(a.x, a.part, a.splits_o, a.ln_mid, a.h_mid, a.n, a.H, a.eps, red);
    stamp(3);
    ok = dm_grid_barrier(a.bar, bar_base + 2ull * gridDim.x, true, status, 0x712, &s_ok);
    stamp(4);
  }
  // phase 3: gate/up with SwiGLU
  if (ok) {
    dm_gemm_phase<true>(p, &tm_hmid, &tm_wgu, a.n, a.F / 64, a.H / 64, 1, a.F, nullptr, a.act, a.F, status);
    __syncthreads();
    stamp(5);
    ok = dm_grid_barrier(a.bar, bar_base + 3ull * gridDim.x, true, status, 0x713, &s_ok);
    stamp(6);
  }
  // phase 4: down-proj partials
  if (ok) {
    dm_gemm_phase<false>(p, &tm_act, &tm_wd, a.n, a.H / 128, a.F / 64, a.splits_d, 0, a.part, nullptr, a.H, status);
    __syncthreads();
    stamp(7);
    ok = dm_grid_barrier(a.bar, bar_base + 4ull * gridDim.x, false, status, 0x714, &s_ok);
    stamp(8);
  }
  // phase 5: residual add + next norm
  if (ok) dm_norm_phase(a.x, a.part, a.splits_d, a.ln_out, a.h_out, a.n, a.H, a.eps, red);
  stamp(9);

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(p.tmem_base, kDmTmemCols);
}

static int dm_pick_splits(int grid, int tiles, int k_blocks, int min_kb) {
  int s = grid / tiles;
  if (s < 1) s = 1;
  const int cap = k_blocks / min_kb > 1 ? k_blocks / min_kb : 1;
  if (s > cap) s = cap;
  const int kpb = (k_blocks + s - 1) / s;
  return (k_blocks + kpb - 1) / kpb;  // no empty slice
}

}  // namespace sb

extern "C" {

// Number of fp32 elements the partial-sum workspace needs for a batch of n rows.
long long sb_decode_mlp_part_elems(int n, int H, int Q, int F) {
  const int grid = sb::sm_count();
  const int so = sb::dm_pick_splits(grid, H / 128, Q / 64, 4);
  const int sd = sb::dm_pick_splits(grid, H / 128, F / 64, 4);
  return static_cast<long long>(so > sd ? so : sd) * n * H;
}

// One launch = o-proj + residual/norm + gate/up/SwiGLU + down-proj + residual/norm (see the top of this file).
//   att [n, Q], x [n, H] (in place), wo [H, Q], wgu [2F, H] (gate rows then up rows), wd [H, F], ln_mid / ln_out [H],
//   h_mid [n, H], act [n, F], h_out [n, H] bf16; part: fp32 workspace of part_elems elements; bar: one zeroed 64-bit word;
//   trace: null, or [number of SMs, 16] words that receive each CTA's clock at the phase boundaries.
int sb_decode_mlp_block(const void* att, void* x, const void* wo, const void* ln_mid, const void* wgu, const void* wd,
                        const void* ln_out, void* h_mid, void* act, void* h_out, float* part, long long part_elems,
                        unsigned long long* bar, int n, int H, int Q, int F, float eps, cudaStream_t stream,
                        unsigned long long* trace) {
  using namespace sb;
  if (n < 1 || n > kDmMaxRows || H % 128 || Q % 64 || F % 64 || (H >> 3) > kDmThreads * kDmMaxVec) return SB_ERR_ARG;
  if (part == nullptr || bar == nullptr) return SB_ERR_ARG;
  int* status = device_status_ptr();
  if (status == nullptr) return SB_ERR_CUDA;
  static int grid_dev[64] = {};  // per device: 0 = not configured, < 0 = the kernel cannot be made resident
  int& grid = grid_dev[device_index()];
  if (grid == 0) {
    if (cudaFuncSetAttribute(decode_mlp_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDmSmem) != cudaSuccess)
      return SB_ERR_CUDA;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mlp_block_kernel, kDmThreads, kDmSmem) != cudaSuccess)
      return SB_ERR_CUDA;
    grid = per_sm >= 1 ? sm_count() : -1;
  }
  if (grid < 0) return SB_ERR_CUDA;
  DmArgs a;
  a.n = n;
  a.H = H;
  a.Q = Q;
  a.F = F;
  a.splits_o = dm_pick_splits(grid, H / 128, Q / 64, 4);
  a.splits_d = dm_pick_splits(grid, H / 128, F / 64, 4);
  a.eps = eps;
  a.x = reinterpret_cast<__nv_bfloat16*>(x);
  a.ln_mid = reinterpret_cast<const __nv_bfloat16*>(ln_mid);
  a.ln_out = reinterpret_cast<const __nv_bfloat16*>(ln_out);
  a.h_mid = reinterpret_cast<__nv_bfloat16*>(h_mid);
  a.act = reinterpret_cast<__nv_bfloat16*>(act);
  a.h_out = reinterpret_cast<__nv_bfloat16*>(h_out);
  a.part = part;
  a.bar = bar;
  a.trace = trace;
  const long long need = static_cast<long long>(a.splits_o > a.splits_d ? a.splits_o : a.splits_d) * n * H;
  if (part_elems < need) return SB_ERR_TOO_LARGE;
  const CUtensorMap* t_att = get_tmap_bf16_2d(att, n, Q, Q, 128);
  const CUtensorMap* t_wo = get_tmap_bf16_2d(wo, H, Q, Q, 128);
  const CUtensorMap* t_hm = get_tmap_bf16_2d(h_mid, n, H, H, 128);
  const CUtensorMap* t_wgu = get_tmap_bf16_2d(wgu, 2ll * F, H, H, 64);
  const CUtensorMap* t_act = get_tmap_bf16_2d(act, n, F, F, 128);
  const CUtensorMap* t_wd = get_tmap_bf16_2d(wd, H, F, F, 128);
  if (!t_att || !t_wo || !t_hm || !t_wgu || !t_act || !t_wd) return SB_ERR_TMAP;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kDmThreads);
  cfg.dynamicSmemBytes = kDmSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_mlp_block_kernel, *t_att, *t_wo, *t_hm, *t_wgu, *t_act, *t_wd, a, status);
  return e == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
