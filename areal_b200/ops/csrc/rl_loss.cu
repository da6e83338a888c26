// Reinforcement-learning losses as single bandwidth-bound kernels.
//
//   ppo_token_loss   decoupled PPO / GRPO clipped surrogate at token level with the token-level
//                    rejection sampling between proximal and behaviour policy folded in: one pass
//                    over the per-token inputs produces the loss sum, its gradient with respect to
//                    the new log-probs, and every per-token statistic the trainer logs. Replaces the
//                    ~40 elementwise launches (and three host synchronisations) of the eager
//                    statement (reference: areal/utils/functional/functional.py:185-437, 452-596).
//   gae_scan         token-level generalised advantage estimation: one thread per sequence walks its
//                    row from the end (reference: the Python loop over T in areal/trainer/ppo/gae.py:10-36).
//
// Sequence-level variants (GSPO ratios, sequence-level rejection) need per-sequence reductions
// first and stay on the eager path.
#include "common.cuh"

namespace ab2 {

struct PPOLossParams {
  float eps_lo;      // ratio is clipped to [1 - eps_lo, 1 + eps_hi]
  float eps_hi;
  float c_clip;      // dual clip constant, <= 0: off
  int rs_action;     // 0 none, 1 mask, 2 clamp
  int rs_metric;     // 0 ratio, 1 kl_k1, 2 kl_k2, 3 kl_k3, 4 binary_kl
  float rs_lower;
  float rs_upper;
  int rs_has_lower;
  int rs_has_upper;
  int prox_is_logp;  // 1: the proximal policy is the current one (ratio == 1, gradient of exp(logp - sg(logp)))
};

enum PPOFlags : int { F_CLIP = 1, F_DUAL = 2, F_BEHAVE = 4, F_KEPT = 8 };

__device__ __forceinline__ float bern_kl(float lp, float lq) {
  const float eps = 1e-8f;
  const float p = fminf(fmaxf(expf(lp), eps), 1.f - eps), q = fminf(fmaxf(expf(lq), eps), 1.f - eps);
  return p * logf(p / q) + (1.f - p) * logf((1.f - p) / (1.f - q));
}

// sums (double, 8 entries): 0 loss over kept tokens, 1 valid tokens before rejection, 2 kept tokens,
// 3 filtered / clamped tokens, 4 clipped, 5 dual clipped, 6 behave tokens.
__global__ void ppo_token_loss_kernel(const float* __restrict__ logp, const float* __restrict__ prox,
                                      const float* __restrict__ old, const float* __restrict__ adv,
                                      const uint8_t* __restrict__ mask, long long n, PPOLossParams P,
                                      float* __restrict__ dlogp, float* __restrict__ loss_tok,
                                      float* __restrict__ ratio_out, float* __restrict__ behave_w,
                                      uint8_t* __restrict__ flags, double* __restrict__ sums) {
  double acc[7] = {0, 0, 0, 0, 0, 0, 0};
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const bool valid = mask[i] != 0;
    const float lp = logp[i];
    const float px = P.prox_is_logp ? lp : prox[i];
    const float ol = old[i];
    const float a = adv[i];
    // ---- rejection sampling between proximal and behaviour policy (token level)
    bool kept = valid;
    float w = 1.f;
    int fl = 0;
    if (P.rs_action != 0) {
      float lr = px - ol;
      if (!isfinite(lr)) lr = 0.f;
      float metric;
      switch (P.rs_metric) {
        case 0: metric = expf(lr); break;
        case 1: metric = lr; break;
        case 2: metric = 0.5f * lr * lr; break;
        case 3: metric = expf(-lr) - 1.f + lr; break;
        default: metric = fmaxf(bern_kl(px, ol), bern_kl(ol, px)); break;
      }
      const float raw = expf(lr);
      w = raw;
      if (P.rs_action == 1) {
        bool inb = true;
        if (P.rs_has_upper) inb = inb && (metric <= P.rs_upper);
        if (P.rs_has_lower) inb = inb && (metric >= P.rs_lower);
        kept = valid && inb;
        if (valid && !inb) acc[3] += 1.0;
      } else {
        const float lo = P.rs_has_lower ? P.rs_lower : 0.f;
        w = fmaxf(w, lo);
        if (P.rs_has_upper) w = fminf(w, P.rs_upper);
        if (valid && w != raw) acc[3] += 1.0;
      }
      if (!kept) w = 0.f;
      if (w > 0.f && kept) fl |= F_BEHAVE;
    }
    // ---- clipped surrogate
    const float ratio = valid ? expf(lp - px) : 0.f;
    const float clipped = fminf(fmaxf(ratio, 1.f - P.eps_lo), 1.f + P.eps_hi);
    const float l1 = -a * ratio, l2 = -a * clipped;
    float loss = fmaxf(l1, l2);
    // d loss / d logp: through `ratio` only where the unclipped branch is the maximum (ties go to it,
    // like torch.max) or the clip is not active
    float g = (l1 >= l2) ? (-a * ratio) : ((ratio == clipped) ? (-a * ratio) : 0.f);
    if (l1 < l2 && valid) fl |= F_CLIP;
    if (P.c_clip > 0.f) {
      const float sgn = (a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f);
      const float l3 = sgn * P.c_clip * a;
      if (l3 < loss) {
        if (valid) fl |= F_DUAL;
        loss = l3;
        g = 0.f;
      }
    }
    if (P.rs_action != 0) {
      loss *= w;
      g *= w;
    }
    if (!kept) g = 0.f;
    if (kept) fl |= F_KEPT;
    dlogp[i] = g;
    loss_tok[i] = loss;
    ratio_out[i] = ratio;
    behave_w[i] = w;
    flags[i] = (uint8_t)fl;
    if (kept) acc[0] += (double)loss;
    if (valid) acc[1] += 1.0;
    if (kept) acc[2] += 1.0;
    if (fl & F_CLIP) acc[4] += 1.0;
    if (fl & F_DUAL) acc[5] += 1.0;
    if (fl & F_BEHAVE) acc[6] += 1.0;
  }
  __shared__ double red[7][8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    double v = acc[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[k][wid] = v;
  }
  __syncthreads();
  if (threadIdx.x < 7) {
    double v = 0;
    for (int wq = 0; wq < (blockDim.x >> 5); ++wq) v += red[threadIdx.x][wq];
    if (v != 0) atomicAdd(&sums[threadIdx.x], v);
  }
}

// One thread per sequence. rewards / values / mask / adv / ret: [B, L] row-major; lambda: [B].
// delta_t = r_t + gamma * V_next - V_t, A_t = delta_t + gamma * lambda * A_next on loss positions;
// masked positions carry the running advantage and the next value; A[:, L-1] = 0.
__global__ void gae_scan_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                                const uint8_t* __restrict__ mask, const uint8_t* __restrict__ no_eos,
                                const float* __restrict__ lam, float gamma, int B, int L,
                                float* __restrict__ adv, float* __restrict__ ret) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const size_t base = (size_t)b * L;
  const float dl = gamma * lam[b];
  float last = 0.f;
  float nextv = no_eos[b] ? values[base + L - 1] : 0.f;
  adv[base + L - 1] = 0.f;
  ret[base + L - 1] = values[base + L - 1];
  for (int t = L - 2; t >= 0; --t) {
    const float v = values[base + t];
    const float delta = rewards[base + t] + gamma * nextv - v;
    const float nw = delta + dl * last;
    if (mask[base + t]) {
      nextv = v;
      last = nw;
    }
    adv[base + t] = last;
    ret[base + t] = last + v;
  }
}

}  // namespace ab2

extern "C" {

// All per-token arrays have n elements; mask / flags are bytes; sums: 8 doubles, zeroed by the caller.
// params: 10 x 4 bytes in the order of PPOLossParams.
int ab2_ppo_token_loss(const float* logp, const float* prox, const float* old, const float* adv, const void* mask, long long n,
                       const void* params, float* dlogp, float* loss_tok, float* ratio, float* behave_w, void* flags, double* sums,
                       void* stream) {
  using namespace ab2;
  if (n <= 0) return 0;
  PPOLossParams P = *reinterpret_cast<const PPOLossParams*>(params);
  if (!P.prox_is_logp && !prox) return 10;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ppo_token_loss_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(logp, prox, old, adv, (const uint8_t*)mask, n, P, dlogp, loss_tok,
                                                                       ratio, behave_w, (uint8_t*)flags, sums);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_gae_scan(const float* rewards, const float* values, const void* mask, const void* no_eos, const float* lam, float gamma, int B,
                 int L, float* adv, float* ret, void* stream) {
  using namespace ab2;
  if (B <= 0 || L <= 0) return 0;
  gae_scan_kernel<<<(B + 63) / 64, 64, 0, (cudaStream_t)stream>>>(rewards, values, (const uint8_t*)mask, (const uint8_t*)no_eos, lam, gamma,
                                                                  B, L, adv, ret);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
