// Bandwidth-bound kernels of the transformer block and the optimizer: RMSNorm (+residual,
// fwd/bwd), rotary embedding, SwiGLU (fwd/bwd), embedding gather / scatter-add, fused
// AdamW on flat shards with device-side clip coefficient, squared-norm reduction.
// All use 16-byte vector accesses and grid-stride persistence sized from the SM count.
//
// Reference call sites these replace: RMSNorm/RoPE/SwiGLU eager ops in
// areal/experimental/models/archon/qwen3/model/model.py and qwen2/model/rope.py,
// torch.optim.AdamW(fused=True) in areal/engine/fsdp_engine.py, multi_tensor_l2norm /
// multi_tensor_scale in areal/engine/fsdp_utils/grad.py.
#include "common.cuh"

namespace ab2 {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------ RMSNorm
// One CTA of TPR threads per row; each thread keeps up to VPT 16-byte vectors in registers.
// y = x * rstd * w, optionally x = x + residual first (the sum is written back to `resid_out`).
template <int TPR, int VPT>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ resid,
                                   const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ resid_out, float* __restrict__ rstd_out,
                                   int rows, int H, float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int nvec = H >> 3;
  // TPR == 32: every warp of the CTA owns its own row (blockDim.x / 32 rows per CTA step)
  const int rows_per_cta = (TPR == 32) ? (blockDim.x >> 5) : 1;
  const int sub = (TPR == 32) ? (threadIdx.x >> 5) : 0;
  const int tid = (TPR == 32) ? (threadIdx.x & 31) : threadIdx.x;
  for (int row = blockIdx.x * rows_per_cta + sub; row < rows; row += gridDim.x * rows_per_cta) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* rr = resid ? reinterpret_cast<const uint4*>(resid + (size_t)row * H) : nullptr;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * TPR;
      if (idx < nvec) {
        uint4 a = xr[idx];
        const uint32_t aa[4] = {a.x, a.y, a.z, a.w};
        uint32_t bb[4] = {0, 0, 0, 0};
        if (rr) {
          uint4 b = rr[idx];
          bb[0] = b.x; bb[1] = b.y; bb[2] = b.z; bb[3] = b.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = unpack_bf16(aa[e]);
          if (rr) {
            const float2 g = unpack_bf16(bb[e]);
            f.x += g.x; f.y += g.y;
            // The residual stream is stored in bf16: normalise what is stored.
            const uint32_t pk = pack_bf16(f.x, f.y);
            bb[e] = pk;
            f = unpack_bf16(pk);
          }
          v[i][2 * e] = f.x; v[i][2 * e + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
        if (rr && resid_out)
          reinterpret_cast<uint4*>(resid_out + (size_t)row * H)[idx] = make_uint4(bb[0], bb[1], bb[2], bb[3]);
      }
    }
    ss = (TPR == 32) ? warp_sum(ss) : block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (tid == 0 && rstd_out) rstd_out[row] = rstd;
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * TPR;
      if (idx < nvec) {
        const uint4 ww = wr[idx];
        const uint32_t wa[4] = {ww.x, ww.y, ww.z, ww.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16(wa[e]);
          o[e] = pack_bf16(v[i][2 * e] * rstd * f.x, v[i][2 * e + 1] * rstd * f.y);
        }
        yr[idx] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dresid), dw[col] += sum_rows dy * xhat.
// Each CTA walks many rows and keeps its dw partial in registers; one atomicAdd per column
// per CTA at the end.
template <int TPR, int VPT>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ dresid,
                                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw, int rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  const int rows_per_cta = (TPR == 32) ? (blockDim.x >> 5) : 1;
  const int sub = (TPR == 32) ? (threadIdx.x >> 5) : 0;
  const int tid = (TPR == 32) ? (threadIdx.x & 31) : threadIdx.x;
  float dwacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
  for (int row = blockIdx.x * rows_per_cta + sub; row < rows; row += gridDim.x * rows_per_cta) {
    const float rstd = rstd_in[row];
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    float xh[VPT][8], gw[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * TPR;
      if (idx < nvec) {
        const uint4 a = xr[idx], g = gr[idx], ww = wr[idx];
        const uint32_t aa[4] = {a.x, a.y, a.z, a.w}, ga[4] = {g.x, g.y, g.z, g.w},
                       wa[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 xf = unpack_bf16(aa[e]), gf = unpack_bf16(ga[e]), wf = unpack_bf16(wa[e]);
          const float h0 = xf.x * rstd, h1 = xf.y * rstd;
          xh[i][2 * e] = h0; xh[i][2 * e + 1] = h1;
          gw[i][2 * e] = gf.x * wf.x; gw[i][2 * e + 1] = gf.y * wf.y;
          dwacc[i][2 * e] += gf.x * h0; dwacc[i][2 * e + 1] += gf.y * h1;
          dot += gw[i][2 * e] * h0 + gw[i][2 * e + 1] * h1;
        }
      }
    }
    dot = (TPR == 32) ? warp_sum(dot) : block_sum(dot, red);
    const float c = dot / (float)H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
    const uint4* drr = dresid ? reinterpret_cast<const uint4*>(dresid + (size_t)row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * TPR;
      if (idx < nvec) {
        uint32_t o[4];
        uint32_t da[4] = {0, 0, 0, 0};
        if (drr) {
          const uint4 d = drr[idx];
          da[0] = d.x; da[1] = d.y; da[2] = d.z; da[3] = d.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float r0 = rstd * (gw[i][2 * e] - xh[i][2 * e] * c);
          float r1 = rstd * (gw[i][2 * e + 1] - xh[i][2 * e + 1] * c);
          if (drr) {
            const float2 d = unpack_bf16(da[e]);
            r0 += d.x; r1 += d.y;
          }
          o[e] = pack_bf16(r0, r1);
        }
        dxr[idx] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = tid + i * TPR;
    if (idx < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(dw + idx * 8 + e, dwacc[i][e]);
    }
  }
}

// ------------------------------------------------------------------ RoPE (rotate-half form)
// x: [T, heads, D] bf16 with row stride `stride_t` elements; cos/sin: [max_pos, D/2] fp32.
// sign = +1 forward, -1 backward (inverse rotation). In place.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos,
                            const float* __restrict__ cosb, const float* __restrict__ sinb, int T,
                            int heads, int D, long long stride_t, float sign) {
  const int half = D >> 1;
  const int pairs_per_tok = heads * (half >> 1);  // two adjacent freq indices per thread
  const long long total = (long long)T * pairs_per_tok;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / pairs_per_tok);
    const int r = (int)(i - (long long)t * pairs_per_tok);
    const int h = r / (half >> 1);
    const int j = (r - h * (half >> 1)) * 2;
    const int p = pos[t];
    const float2 c = *reinterpret_cast<const float2*>(cosb + (size_t)p * half + j);
    float2 s = *reinterpret_cast<const float2*>(sinb + (size_t)p * half + j);
    s.x *= sign; s.y *= sign;
    __nv_bfloat16* base = x + (size_t)t * stride_t + (size_t)h * D;
    uint32_t* lo = reinterpret_cast<uint32_t*>(base + j);
    uint32_t* hi = reinterpret_cast<uint32_t*>(base + half + j);
    const float2 a = unpack_bf16(*lo), b = unpack_bf16(*hi);
    *lo = pack_bf16(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
    *hi = pack_bf16(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
  }
}

// ------------------------------------------------------------------ SwiGLU
// gu: [T, 2I] (gate | up); out[T, I] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long long T, int I) {
  pdl_wait();
  pdl_trigger();
  const int vec_per_row = I >> 3;
  const long long total = T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = (int)(i - t * vec_per_row);
    const uint4 g = reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I)[c];
    const uint4 u = reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I + I)[c];
    const uint32_t ga[4] = {g.x, g.y, g.z, g.w}, ua[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gf = unpack_bf16(ga[e]), uf = unpack_bf16(ua[e]);
      o[e] = pack_bf16(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
    }
    reinterpret_cast<uint4*>(out + (size_t)t * I)[c] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dgu[T, 2I] from dout[T, I] and the saved gu.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const int vec_per_row = I >> 3;
  const long long total = T * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = (int)(i - t * vec_per_row);
    const uint4 g = reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I)[c];
    const uint4 u = reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I + I)[c];
    const uint4 d = reinterpret_cast<const uint4*>(dout + (size_t)t * I)[c];
    const uint32_t ga[4] = {g.x, g.y, g.z, g.w}, ua[4] = {u.x, u.y, u.z, u.w}, da[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gf = unpack_bf16(ga[e]), uf = unpack_bf16(ua[e]), df = unpack_bf16(da[e]);
      const float s0 = 1.f / (1.f + __expf(-gf.x)), s1 = 1.f / (1.f + __expf(-gf.y));
      const float silu0 = gf.x * s0, silu1 = gf.y * s1;
      og[e] = pack_bf16(df.x * uf.x * (s0 + silu0 * (1.f - s0)), df.y * uf.y * (s1 + silu1 * (1.f - s1)));
      ou[e] = pack_bf16(df.x * silu0, df.y * silu1);
    }
    reinterpret_cast<uint4*>(dgu + (size_t)t * 2 * I)[c] = make_uint4(og[0], og[1], og[2], og[3]);
    reinterpret_cast<uint4*>(dgu + (size_t)t * 2 * I + I)[c] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// ------------------------------------------------------------------ embedding
// A token id outside [0, V) is clamped (the kernel stays inside W) and reported in the error word, which the
// engines read once per optimizer step / decode iteration: a bad id is a loud failure, not a silent row 0.
__global__ void embed_fwd_kernel(const __nv_bfloat16* __restrict__ W, const int* __restrict__ ids,
                                 __nv_bfloat16* __restrict__ out, int T, int H, int V, int* __restrict__ err) {
  pdl_wait();
  pdl_trigger();
  const int vec = H >> 3;
  const long long total = (long long)T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec), c = (int)(i - (long long)t * vec);
    int id = ids[t];
    if (id < 0 || id >= V) {
      if (c == 0 && err != nullptr) set_error(err, ERR_BOUNDS);
      id = id < 0 ? 0 : V - 1;
    }
    reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = reinterpret_cast<const uint4*>(W + (size_t)id * H)[c];
  }
}
// dW[ids[t]] += dy[t]  (fp32 gradient buffer)
__global__ void embed_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const int* __restrict__ ids,
                                 float* __restrict__ dW, int T, int H, int V) {
  const int pairs = H >> 1;
  const long long total = (long long)T * pairs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / pairs), c = (int)(i - (long long)t * pairs);
    int id = ids[t];
    if (id < 0 || id >= V) continue;
    const float2 f = unpack_bf16(reinterpret_cast<const uint32_t*>(dy + (size_t)t * H)[c]);
    atomicAdd(dW + (size_t)id * H + 2 * c, f.x);
    atomicAdd(dW + (size_t)id * H + 2 * c + 1, f.y);
  }
}

// ------------------------------------------------------------------ norms / AdamW
// out[0] += sum(x^2); x fp32.
__global__ void sqnorm_f32_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = x4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) acc += x[i] * x[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// state[0] = sum of squares (input); writes state[1] = clip coefficient, state[2] = 1 if the
// norm is finite (update allowed) else 0, state[3] = norm. inv_scale folds loss scaling /
// gradient averaging into the coefficient.
__global__ void clip_coef_kernel(float* __restrict__ state, float max_norm, float inv_scale) {
  const float ss = state[0];
  const float norm = sqrtf(ss) * inv_scale;
  const bool finite = isfinite(norm);
  float coef = inv_scale;
  if (max_norm > 0.f && finite && norm > max_norm) coef = inv_scale * max_norm / (norm + 1e-6f);
  state[1] = finite ? coef : 0.f;
  state[2] = finite ? 1.f : 0.f;
  state[3] = norm;
}

// Decoupled-weight-decay Adam on a flat shard. g may be fp32 or bf16 (G_BF16). The clip
// coefficient and the skip flag are read from device memory (state[1], state[2]) so the
// step needs no host synchronisation. Writes the bf16 compute copy in the same pass.
template <bool G_BF16>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const void* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16,
                             const float* __restrict__ state, long long n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2) {
  const float coef = state ? state[1] : 1.f;
  const bool go = state ? (state[2] != 0.f) : true;
  if (!go) return;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float gi = G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])
                      : reinterpret_cast<const float*>(g)[i];
    gi *= coef;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    float pi = p[i];
    pi -= lr * wd * pi;
    pi -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    p[i] = pi;
    if (p_bf16) p_bf16[i] = __float2bfloat16(pi);
  }
}

static int grid_for(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace ab2

extern "C" {
using namespace ab2;

// RMSNorm forward. H must be a multiple of 8 and <= 8192. resid/resid_out/rstd may be null.
int ab2_rmsnorm_fwd(const void* x, const void* resid, const void* w, void* y, void* resid_out,
                    float* rstd, int rows, int H, float eps, void* stream) {
  if (H % 8 || H > 8192) return 10;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  if (rows <= 0) return 0;
  auto X = (const __nv_bfloat16*)x; auto R = (const __nv_bfloat16*)resid; auto W = (const __nv_bfloat16*)w;
  auto Y = (__nv_bfloat16*)y; auto RO = (__nv_bfloat16*)resid_out;
  if (H <= 256) launch_pdl(rmsnorm_fwd_kernel<32, 1>, dim3((rows + 7) / 8 < 148 * 16 ? (rows + 7) / 8 : 148 * 16), dim3(256), 0, s, X, R, W, Y, RO, rstd, rows, H, eps);
  else if (H <= 2048) launch_pdl(rmsnorm_fwd_kernel<128, 2>, dim3(grid), dim3(128), 0, s, X, R, W, Y, RO, rstd, rows, H, eps);
  else if (H <= 4096) launch_pdl(rmsnorm_fwd_kernel<128, 4>, dim3(grid), dim3(128), 0, s, X, R, W, Y, RO, rstd, rows, H, eps);
  else launch_pdl(rmsnorm_fwd_kernel<256, 4>, dim3(grid), dim3(256), 0, s, X, R, W, Y, RO, rstd, rows, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// RMSNorm backward; dw (fp32, [H]) is accumulated into. dresid may be null.
int ab2_rmsnorm_bwd(const void* x, const void* w, const void* dy, const void* dresid, const float* rstd,
                    void* dx, float* dw, int rows, int H, void* stream) {
  if (H % 8 || H > 8192) return 10;
  if (rows <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = rows < 148 * 4 ? rows : 148 * 4;
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto DY = (const __nv_bfloat16*)dy;
  auto DR = (const __nv_bfloat16*)dresid; auto DX = (__nv_bfloat16*)dx;
  if (H <= 256) rmsnorm_bwd_kernel<32, 1><<<(rows + 7) / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8, 256, 0, s>>>(X, W, DY, DR, rstd, DX, dw, rows, H);
  else if (H <= 2048) rmsnorm_bwd_kernel<128, 2><<<grid, 128, 0, s>>>(X, W, DY, DR, rstd, DX, dw, rows, H);
  else if (H <= 4096) rmsnorm_bwd_kernel<128, 4><<<grid, 128, 0, s>>>(X, W, DY, DR, rstd, DX, dw, rows, H);
  else rmsnorm_bwd_kernel<256, 4><<<grid, 256, 0, s>>>(X, W, DY, DR, rstd, DX, dw, rows, H);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// In-place rotary embedding on [T, heads, D] (row stride stride_t elements). D % 4 == 0.
int ab2_rope(void* x, const int* pos, const float* cosb, const float* sinb, int T, int heads, int D,
             long long stride_t, int backward, void* stream) {
  if (D % 4) return 10;
  if (T <= 0) return 0;
  const long long total = (long long)T * heads * (D / 4);
  rope_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)x, pos, cosb, sinb, T, heads, D, stride_t, backward ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_swiglu_fwd(const void* gu, void* out, long long T, int I, void* stream) {
  if (I % 8) return 10;
  if (T <= 0) return 0;
  launch_pdl(swiglu_fwd_kernel, dim3(grid_for(T * (I / 8), 256)), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)gu,
             (__nv_bfloat16*)out, T, I);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
int ab2_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int I, void* stream) {
  if (I % 8) return 10;
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, I);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_embed_fwd(const void* W, const int* ids, void* out, int T, int H, int V, void* stream) {
  if (H % 8) return 10;
  if (T <= 0) return 0;
  launch_pdl(embed_fwd_kernel, dim3(grid_for((long long)T * (H / 8), 256)), dim3(256), 0, (cudaStream_t)stream,
             (const __nv_bfloat16*)W, ids, (__nv_bfloat16*)out, T, H, V, ab2host::error_flag());
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
int ab2_embed_bwd(const void* dy, const int* ids, float* dW, int T, int H, int V, void* stream) {
  if (H % 2) return 10;
  if (T <= 0) return 0;
  embed_bwd_kernel<<<grid_for((long long)T * (H / 2), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, ids, dW, T, H, V);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// state: 4 floats on the device. sqnorm accumulates into state[0] (zero it first).
int ab2_sqnorm_f32(const float* x, long long n, float* state, void* stream) {
  if (n <= 0) return 0;
  sqnorm_f32_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, (cudaStream_t)stream>>>(x, n, state);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
int ab2_clip_coef(float* state, float max_norm, float inv_scale, void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(state, max_norm, inv_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
int ab2_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p_bf16,
              const float* state, long long n, float lr, float beta1, float beta2, float eps, float wd,
              int step, void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  const int grid = grid_for(n, 256);
  if (g_is_bf16)
    adamw_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(p, m, v, g, (__nv_bfloat16*)p_bf16, state, n,
                                                              lr, beta1, beta2, eps, wd, bc1, bc2);
  else
    adamw_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(p, m, v, g, (__nv_bfloat16*)p_bf16, state, n,
                                                               lr, beta1, beta2, eps, wd, bc1, bc2);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
