// RL objective kernels: one pass over the response tokens computes the clipped policy-gradient
// loss (PPO / dual-clip), the KL-to-reference penalty, their gradient with respect to the token
// log-probabilities and the reduction statistics; plus group-relative (GRPO / RLOO) advantage
// normalisation and the GAE reverse scan.
#include "host_common.h"
#include "ptx.cuh"

namespace sb {

enum { kLossRegular = 0, kLossDualClip = 1 };
enum { kKlK1 = 0, kKlAbs = 1, kKlK2 = 2, kKlK3 = 3 };

__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// stats: [0] sum policy loss, [1] sum clipped-token mask, [2] sum KL, [3] sum mask, [4] sum ratio*mask,
//        [5] sum dual-clip-active mask, [6] sum (logp - old)*mask (approx KL to old policy), [7] unused
// dlogp = w_pol * d(policy loss)/dlogp + w_kl * d(KL)/dlogp   (both already multiplied by the mask)
__global__ void policy_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_logp,
                                   const float* __restrict__ adv, const float* __restrict__ mask,
                                   const float* __restrict__ ref_logp, const float* __restrict__ tis,
                                   const float* __restrict__ klw, long long n,
                                   float eps_low, float eps_high, float clip_c, int loss_type, int kl_type, float w_pol,
                                   float w_kl, float* __restrict__ dlogp, float* __restrict__ stats) {
  __shared__ float red[32];
  float acc[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float mk = mask[i];
    const float lp = logp[i];
    const float A = adv[i];
    const float w = tis ? tis[i] : 1.f;
    const float d = fminf(fmaxf(lp - old_logp[i], -20.f), 20.f);
    const float r = __expf(d);
    const bool d_clamped = (lp - old_logp[i]) < -20.f || (lp - old_logp[i]) > 20.f;
    const float rc = fminf(fmaxf(r, 1.f - eps_low), 1.f + eps_high);
    const float l1 = -A * r, l2 = -A * rc;
    float loss = fmaxf(l1, l2);
    // gradient flows through the unclipped branch only
    float dr = (l1 >= l2) ? -A : 0.f;
    const bool clipped = l2 > l1;
    bool dual = false;
    if (loss_type == kLossDualClip && A < 0.f) {
      const float l3 = -A * clip_c;
      if (l3 < loss) {
        loss = l3;
        dr = 0.f;
        dual = true;
      }
    }
    float g = d_clamped ? 0.f : dr * r;  // d r / d logp = r
    float kl = 0.f, dkl = 0.f;
    if (ref_logp) {
      const float lr = lp - ref_logp[i];
      if (kl_type == kKlK1) {
        kl = lr;
        dkl = 1.f;
      } else if (kl_type == kKlAbs) {
        kl = fabsf(lr);
        dkl = lr > 0.f ? 1.f : (lr < 0.f ? -1.f : 0.f);
      } else if (kl_type == kKlK2) {
        kl = 0.5f * lr * lr;
        dkl = lr;
      } else {
        // k3 = exp(x) - x - 1 with x = clamp(ref - logp, -20, 20), result clamped to [-10, 10]
        const float xr = -lr;
        const float x = fminf(fmaxf(xr, -20.f), 20.f);
        const float e = __expf(x);
        kl = e - x - 1.f;
        dkl = (xr == x) ? (1.f - e) : 0.f;
        if (kl > 10.f || kl < -10.f) {
          kl = fminf(fmaxf(kl, -10.f), 10.f);
          dkl = 0.f;
        }
      }
    }
    const float kw = klw ? klw[i] : 1.f;  // per-token weight of the KL term (e.g. 1 / tokens-in-sequence)
    if (dlogp) dlogp[i] = mk * (w_pol * w * g + w_kl * kw * dkl);
    acc[0] += mk * w * loss;
    acc[1] += mk * (clipped ? 1.f : 0.f);
    acc[2] += mk * kw * kl;
    acc[3] += mk;
    acc[4] += mk * r;
    acc[5] += mk * (dual ? 1.f : 0.f);
    acc[6] += mk * (old_logp[i] - lp);
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const float t = block_sum_f(acc[k], red);
    if (threadIdx.x == 0 && t != 0.f) atomicAdd(stats + k, t);
  }
}

// One CTA per group: adv = (score - mean_g) / (std_g + eps) (unbiased std; singleton group: mean 0, std 1);
// mode 0 = GRPO, 1 = GRPO without std (Dr.GRPO), 2 = RLOO ((s - mean) * n / (n - 1)).
__global__ void group_advantage_kernel(const float* __restrict__ scores, const int* __restrict__ group_ids, int B,
                                       int mode, float eps, float* __restrict__ out) {
  __shared__ float red[32];
  const int g = blockIdx.x;
  float s = 0.f, c = 0.f;
  for (int i = threadIdx.x; i < B; i += blockDim.x)
    if (group_ids[i] == g) {
      s += scores[i];
      c += 1.f;
    }
  const float n = block_sum_f(c, red);
  const float sum = block_sum_f(s, red);
  if (n == 0.f) return;
  const float mean = (n > 1.f) ? sum / n : 0.f;
  float v = 0.f;
  for (int i = threadIdx.x; i < B; i += blockDim.x)
    if (group_ids[i] == g) {
      const float d = scores[i] - mean;
      v += d * d;
    }
  const float var = block_sum_f(v, red);
  const float stdv = (n > 1.f) ? sqrtf(var / (n - 1.f)) : 1.f;
  for (int i = threadIdx.x; i < B; i += blockDim.x)
    if (group_ids[i] == g) {
      const float d = scores[i] - mean;
      float a;
      if (mode == 0)
        a = d / (stdv + eps);
      else if (mode == 1)
        a = d;
      else
        a = (n > 1.f) ? d * n / (n - 1.f) : d;
      out[i] = a;
    }
}

// GAE: one thread per sequence, plain reverse scan over the R response positions of [B, R] tensors.  Like the
// reference's scan (ppo_utils.py:1331-1336) it runs over every position, padded ones included (their rewards and
// values are zero by construction); the response mask only enters the whitening that follows on the caller's side:
//   delta_t = r_t + gamma * V_{t+1} - V_t ;  A_t = delta_t + gamma * lambda * A_{t+1} ;  ret_t = A_t + V_t
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values, int B, int R,
                           float gamma, float lam, float* __restrict__ adv, float* __restrict__ ret) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const size_t o = static_cast<size_t>(b) * R;
  float last = 0.f;
  for (int t = R - 1; t >= 0; --t) {
    const float v = values[o + t];
    const float nv = (t + 1 < R) ? values[o + t + 1] : 0.f;
    const float delta = rewards[o + t] + gamma * nv - v;
    last = delta + gamma * lam * last;
    adv[o + t] = last;
    ret[o + t] = last + v;
  }
}

}  // namespace sb

extern "C" {

int sb_policy_loss(const float* logp, const float* old_logp, const float* adv, const float* mask, const float* ref_logp,
                   const float* tis, const float* klw, long long n, float eps_low, float eps_high, float clip_c, int loss_type,
                   int kl_type, float w_pol, float w_kl, float* dlogp, float* stats, void* stream) {
  if (n <= 0) return SB_OK;
  long long blocks = (n + 255) / 256;
  const long long cap = static_cast<long long>(sb::sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  sb::policy_loss_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logp, old_logp, adv, mask, ref_logp, tis, klw, n, eps_low, eps_high, clip_c, loss_type, kl_type, w_pol, w_kl, dlogp,
      stats);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_group_advantage(const float* scores, const int* group_ids, int B, int num_groups, int mode, float eps, float* out,
                       void* stream) {
  if (B <= 0 || num_groups <= 0) return SB_OK;
  sb::group_advantage_kernel<<<num_groups, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(scores, group_ids, B, mode,
                                                                                            eps, out);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

int sb_gae(const float* rewards, const float* values, const float* mask, int B, int R, float gamma, float lam,
           float* adv, float* ret, void* stream) {
  if (B <= 0 || R <= 0) return SB_OK;
  (void)mask;  // kept in the signature for callers that pass one; the scan itself is unmasked (see gae_kernel)
  sb::gae_kernel<<<(B + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(rewards, values, B, R, gamma, lam,
                                                                                      adv, ret);
  return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA;
}

}  // extern "C"
