// Fused per-head RMSNorm (Qwen3 QK-norm) + rotary embedding for the q and k heads of a fused
// QKV projection, forward and backward, reading and writing the projection buffer's layout
// directly:
//
//   forward : qkv [T, (nq + 2 nkv) * D] bf16  ->  qk [T, (nq + nkv), D] bf16 (normed, rotated)
//             (+ rstd [T, nq + nkv] fp32 when norm weights are given); v is consumed in place
//             by the attention kernel through its row stride.
//   backward: dq fp32 [T, nq, D] (the attention backward's reduction buffer) and dk bf16 already
//             sitting in the k region of dqkv  ->  dqkv q / k regions bf16 (un-rotated, norm
//             backward applied), dw_q / dw_k accumulated in fp32.
//
// One warp per token at a time (its heads share the position, so cos / sin are fetched once per
// token), one (token, head) row per step with every lane holding D / 32 contiguous elements,
// the rotate-half partner lives in lane ^ 16. Rows are processed four at a time so that four
// independent loads are in flight per warp. Weight gradients are reduced in registers, then across the
// CTA in shared memory, and reach global memory as one atomic per column per CTA.
//
// Replaces the separate slice / RMSNorm / RoPE launches (and their backward slice-copies) of
// the reference's attention block (areal/experimental/models/archon/qwen3/model/model.py,
// apply_rotary_emb in areal/experimental/models/archon/qwen2/model/rope.py).
#include "common.cuh"

namespace ab2 {

template <int VEC>
__device__ __forceinline__ void load_bf16_vec(const __nv_bfloat16* p, float* out) {
  if (VEC == 4) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y);
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
  } else {
    const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(p));
    out[0] = a.x; out[1] = a.y;
  }
}
template <int VEC>
__device__ __forceinline__ void store_bf16_vec(__nv_bfloat16* p, const float* v) {
  if (VEC == 4) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  } else {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16(v[0], v[1]);
  }
}
template <int VEC>
__device__ __forceinline__ void load_f32_vec(const float* p, float* out) {
  if (VEC == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
    const float2 v = *reinterpret_cast<const float2*>(p);
    out[0] = v.x; out[1] = v.y;
  }
}

constexpr int QK_UNROLL = 4;
constexpr int QK_UNROLL_BWD = 2;  // the backward keeps three vectors per row live: two rows keep it at 3+ CTAs per SM

// D = 32 * VEC. wq / wk may be null (no norm: rotation only).
template <int VEC>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                       const __nv_bfloat16* __restrict__ wk, const int* __restrict__ pos,
                       const float* __restrict__ cosb, const float* __restrict__ sinb,
                       __nv_bfloat16* __restrict__ qk, float* __restrict__ rstd_out, int T, int nq, int nkv,
                       long long qkv_stride, float eps, int hsplit) {
  constexpr int D = 32 * VEC;
  constexpr int HALF = D / 2;
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int heads = nq + nkv;
  const int warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  const int e0 = lane * VEC;               // first element of this lane
  const int f0 = e0 & (HALF - 1);          // frequency index of that element
  const bool upper = lane >= 16;
  float wqv[VEC], wkv[VEC];
  const bool has_norm = wq != nullptr;
  if (has_norm) {
    load_bf16_vec<VEC>(wq + e0, wqv);
    load_bf16_vec<VEC>(wk + e0, wkv);
  }
  // One token per warp at a time: its heads share the position, so cos / sin are fetched once
  // per token and the per-row work is a single independent load -> reduce -> store chain.
  // With few tokens (decode) a token's heads are split over ``hsplit`` warps so the launch is
  // not one long serial walk per token.
  const int hps = ((heads + hsplit - 1) / hsplit + QK_UNROLL - 1) / QK_UNROLL * QK_UNROLL;
  for (long long w = warp0; w < (long long)T * hsplit; w += nwarps) {
    const int tok = (int)(w / hsplit);
    const int hbeg = (int)(w - (long long)tok * hsplit) * hps;
    const int hend = min(heads, hbeg + hps);
    const int p = pos[tok];
    float c[VEC], s[VEC];
    load_f32_vec<VEC>(cosb + (size_t)p * HALF + f0, c);
    load_f32_vec<VEC>(sinb + (size_t)p * HALF + f0, s);
    const __nv_bfloat16* src = qkv + (size_t)tok * qkv_stride + e0;
    __nv_bfloat16* dst = qk + (size_t)tok * heads * D + e0;
    for (int h0 = hbeg; h0 < hend; h0 += QK_UNROLL) {
      float x[QK_UNROLL][VEC];
#pragma unroll
      for (int u = 0; u < QK_UNROLL; ++u)
        if (h0 + u < hend) load_bf16_vec<VEC>(src + (size_t)(h0 + u) * D, x[u]);
#pragma unroll
      for (int u = 0; u < QK_UNROLL; ++u) {
        const int h = h0 + u;
        if (h >= hend) break;
        float y[VEC];
        if (has_norm) {
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < VEC; ++e) ss += x[u][e] * x[u][e];
          ss = warp_sum(ss);
          const float rstd = rsqrtf(ss / (float)D + eps);
          if (lane == 0) rstd_out[(size_t)tok * heads + h] = rstd;
          const bool isq = h < nq;
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            // the normalised value is rounded to bf16 like the unfused op's output
            y[e] = __bfloat162float(__float2bfloat16(x[u][e] * rstd * (isq ? wqv[e] : wkv[e])));
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) y[e] = x[u][e];
        }
        float o[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float partner = __shfl_xor_sync(0xffffffffu, y[e], 16);
          o[e] = upper ? (y[e] * c[e] + partner * s[e]) : (y[e] * c[e] - partner * s[e]);
        }
        store_bf16_vec<VEC>(dst + (size_t)h * D, o);
      }
    }
  }
}

// dq32: [T, nq, D] fp32. dqkv: [T, (nq + 2 nkv) * D] bf16 whose k region holds dk on entry; q and
// k regions are overwritten with the gradient w.r.t. the projection output.
template <int VEC>
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                       const __nv_bfloat16* __restrict__ wk, const int* __restrict__ pos,
                       const float* __restrict__ cosb, const float* __restrict__ sinb,
                       const float* __restrict__ rstd_in, const float* __restrict__ dq32,
                       __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dwq, float* __restrict__ dwk, int T,
                       int nq, int nkv, long long qkv_stride, long long dqkv_stride) {
  constexpr int D = 32 * VEC;
  constexpr int HALF = D / 2;
  __shared__ float red[2][8][D];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int heads = nq + nkv;
  const int warp0 = blockIdx.x * (blockDim.x >> 5) + wib;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  const int e0 = lane * VEC;
  const int f0 = e0 & (HALF - 1);
  const bool upper = lane >= 16;
  const bool has_norm = wq != nullptr;
  float wqv[VEC], wkv[VEC], aq[VEC], ak[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) { aq[e] = 0.f; ak[e] = 0.f; wqv[e] = 1.f; wkv[e] = 1.f; }
  if (has_norm) {
    load_bf16_vec<VEC>(wq + e0, wqv);
    load_bf16_vec<VEC>(wk + e0, wkv);
  }
  for (int tok = warp0; tok < T; tok += nwarps) {
    const int p = pos[tok];
    float c[VEC], s[VEC];
    load_f32_vec<VEC>(cosb + (size_t)p * HALF + f0, c);
    load_f32_vec<VEC>(sinb + (size_t)p * HALF + f0, s);
    const __nv_bfloat16* xsrc = qkv + (size_t)tok * qkv_stride + e0;
    __nv_bfloat16* gdst = dqkv + (size_t)tok * dqkv_stride + e0;
    const float* qsrc = dq32 + (size_t)tok * nq * D + e0;
    const float* rs = rstd_in + (size_t)tok * heads;
    for (int h0 = 0; h0 < heads; h0 += QK_UNROLL_BWD) {
      float g[QK_UNROLL_BWD][VEC], x[QK_UNROLL_BWD][VEC], rstd[QK_UNROLL_BWD];
#pragma unroll
      for (int u = 0; u < QK_UNROLL_BWD; ++u) {
        const int h = h0 + u;
        if (h < heads) {
          if (h < nq) load_f32_vec<VEC>(qsrc + (size_t)h * D, g[u]);
          else load_bf16_vec<VEC>(gdst + (size_t)h * D, g[u]);
          if (has_norm) {
            load_bf16_vec<VEC>(xsrc + (size_t)h * D, x[u]);
            rstd[u] = rs[h];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < QK_UNROLL_BWD; ++u) {
        const int h = h0 + u;
        if (h >= heads) break;
        float gy[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          // transpose of the rotation: gy_lo = g_lo c + g_hi s ; gy_hi = g_hi c - g_lo s
          const float partner = __shfl_xor_sync(0xffffffffu, g[u][e], 16);
          gy[e] = upper ? (g[u][e] * c[e] - partner * s[e]) : (g[u][e] * c[e] + partner * s[e]);
        }
        float dx[VEC];
        if (has_norm) {
          const bool isq = h < nq;
          float xh[VEC], gw[VEC];
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            xh[e] = x[u][e] * rstd[u];
            gw[e] = gy[e] * (isq ? wqv[e] : wkv[e]);
            dot += gw[e] * xh[e];
            if (isq) aq[e] += gy[e] * xh[e]; else ak[e] += gy[e] * xh[e];
          }
          dot = warp_sum(dot) / (float)D;
#pragma unroll
          for (int e = 0; e < VEC; ++e) dx[e] = rstd[u] * (gw[e] - xh[e] * dot);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) dx[e] = gy[e];
        }
        store_bf16_vec<VEC>(gdst + (size_t)h * D, dx);
      }
    }
  }
  if (has_norm) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      red[0][wib][e0 + e] = aq[e];
      red[1][wib][e0 + e] = ak[e];
    }
    __syncthreads();
    const int nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
      const int which = i / D, col = i - which * D;
      float sum = 0.f;
      for (int w = 0; w < nw; ++w) sum += red[which][w][col];
      atomicAdd((which ? dwk : dwq) + col, sum);
    }
  }
}

}  // namespace ab2

extern "C" {

// Forward. qkv: [T, qkv_stride] bf16 (q heads, then k heads, then v heads, D each); qk: contiguous
// [T, nq + nkv, D] bf16; rstd: [T * (nq + nkv)] fp32 (written only with norm weights).
// wq / wk: [D] bf16 or null together. D must be 64 or 128.
int ab2_qknorm_rope_fwd(const void* qkv, const void* wq, const void* wk, const int* pos, const float* cosb,
                        const float* sinb, void* qk, float* rstd, int T, int nq, int nkv, int D,
                        long long qkv_stride, float eps, void* stream) {
  if (T <= 0) return 0;
  if (D != 64 && D != 128) return 10;
  if ((wq == nullptr) != (wk == nullptr)) return 11;
  if (qkv_stride & 3) return 12;
  // few tokens (decode): split each token's heads over several warps until the GPU is covered
  const int max_split = (nq + nkv + ab2::QK_UNROLL - 1) / ab2::QK_UNROLL;
  int hsplit = 1;
  if ((long long)T < 148 * 8) {
    hsplit = (int)((148 * 8 * 2) / (long long)T);
    if (hsplit > max_split) hsplit = max_split;
    if (hsplit < 1) hsplit = 1;
  }
  const long long want = ((long long)T * hsplit + 7) / 8;   // 8 warps per CTA, one (token, head range) per warp step
  const int grid = (int)(want < 148 * 8 ? want : 148 * 8);
  auto s = (cudaStream_t)stream;
  if (D == 128)
    ab2::launch_pdl(ab2::qknorm_rope_fwd_kernel<4>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq,
                    (const __nv_bfloat16*)wk, pos, cosb, sinb, (__nv_bfloat16*)qk, rstd, T, nq, nkv, qkv_stride, eps, hsplit);
  else
    ab2::launch_pdl(ab2::qknorm_rope_fwd_kernel<2>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq,
                    (const __nv_bfloat16*)wk, pos, cosb, sinb, (__nv_bfloat16*)qk, rstd, T, nq, nkv, qkv_stride, eps, hsplit);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// Backward (see the kernel comment for the buffer contract). dwq / dwk: [D] fp32, accumulated.
int ab2_qknorm_rope_bwd(const void* qkv, const void* wq, const void* wk, const int* pos, const float* cosb,
                        const float* sinb, const float* rstd, const float* dq32, void* dqkv, float* dwq, float* dwk,
                        int T, int nq, int nkv, int D, long long qkv_stride, long long dqkv_stride, void* stream) {
  if (T <= 0) return 0;
  if (D != 64 && D != 128) return 10;
  if ((wq == nullptr) != (wk == nullptr)) return 11;
  if ((qkv_stride | dqkv_stride) & 3) return 12;
  if (wq && (!dwq || !dwk || !rstd)) return 13;
  const long long want = ((long long)T + 7) / 8;
  const int grid = (int)(want < 148 * 4 ? want : 148 * 4);
  auto s = (cudaStream_t)stream;
  if (D == 128)
    ab2::qknorm_rope_bwd_kernel<4><<<grid, 256, 0, s>>>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq,
                                                        (const __nv_bfloat16*)wk, pos, cosb, sinb, rstd, dq32,
                                                        (__nv_bfloat16*)dqkv, dwq, dwk, T, nq, nkv, qkv_stride, dqkv_stride);
  else
    ab2::qknorm_rope_bwd_kernel<2><<<grid, 256, 0, s>>>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq,
                                                        (const __nv_bfloat16*)wk, pos, cosb, sinb, rstd, dq32,
                                                        (__nv_bfloat16*)dqkv, dwq, dwk, T, nq, nkv, qkv_stride, dqkv_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
