// Kernels that fuse compute with cross-GPU data movement over NVLink peer memory.
// Every rank maps every peer's symmetric buffers, so a kernel can load from / store to a
// peer with plain ld/st (no TMA multicast, no library collective in between).
//
//   signal_barrier     all-to-all flag exchange with a bounded wait (error status, no trap)
//   rs_sumsq           gradient reduce-scatter by peer loads + squared-norm partial of the shard
//   rs_sumsq_multimem  the same through the NVLink switch: multimem.ld_reduce on the multicast address
//   norm_allreduce     exchanges the per-shard partials through peer stores -> global sum
//   adamw_push         sharded AdamW whose bf16 result is written straight into every
//                      destination buffer (trainer peers = parameter all-gather, rollout
//                      replicas = weight update)
//   push_copy          shard-direct copy of a bf16 range to several destinations (weight push)
//   push_plan          a whole FSDP-shard -> tensor-parallel re-shard plan (row / column slices of
//                      q/k/v/o, gate/up/down) in ONE launch, bf16 or cast to block-scaled e4m3
//
// These replace: FSDP2's NCCL reduce-scatter / all-gather (areal/engine/fsdp_utils/parallel.py:388),
// the grad-norm all-reduces of areal/engine/fsdp_utils/grad.py:112-190, and the all-gather +
// NCCL broadcast weight update of areal/engine/fsdp_engine.py:1596-1692.
#include <cuda_fp8.h>

#include "common.cuh"

namespace ab2 {

static constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// One CTA. Thread r publishes `epoch` into slot [channel][my_rank] of rank r's signal pad and
// then waits until slot [channel][r] of the local pad reaches `epoch`. The wait is bounded.
__global__ void signal_barrier_kernel(PeerPtrs pads, int my_rank, int world, int channel, int epoch,
                                      long long limit_cycles, int* err) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    int* remote = reinterpret_cast<int*>(pads.p[r]) + channel * MAX_PEERS + my_rank;
    st_release_sys(remote, epoch);
    const int* local = reinterpret_cast<const int*>(pads.p[my_rank]) + channel * MAX_PEERS + r;
    const long long t0 = clock64();
    while (ld_acquire_sys(local) < epoch) {
      if (clock64() - t0 > limit_cycles) {
        set_error(err, ERR_WAIT_PEER_FLAG);
        break;
      }
    }
  }
}

// out[i] = sum_r grads[r][lo + i] for i in [0, n); state[0] += sum(out^2).
__global__ void rs_sumsq_kernel(PeerPtrs grads, int world, long long lo, long long n, float* __restrict__ out,
                                float* __restrict__ state, float scale) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = acc;
  __syncthreads();
  if (w == 0) {
    float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
    t = warp_sum(t);
    if (l == 0) atomicAdd(state, t);
  }
}

// The same reduce-scatter through the NVLink switch (NVLS): `mc` is the MULTICAST address of the
// symmetric gradient buffer; one multimem.ld_reduce returns the sum over all ranks of 16 bytes, so a
// rank issues one load per element group instead of one per peer and the addition happens in the
// switch. Ordering is the caller's: a barrier after every rank's gradient writes, before this kernel.
__global__ void rs_sumsq_multimem_kernel(const float* __restrict__ mc, long long lo, long long n, float* __restrict__ out,
                                         float* __restrict__ state, float scale) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 s;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w)
                 : "l"(mc + lo + 4 * i)
                 : "memory");
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = acc;
  __syncthreads();
  if (w == 0) {
    float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
    t = warp_sum(t);
    if (l == 0) atomicAdd(state, t);
  }
}

// Every rank writes its partial (state[0]) into slot my_rank of every peer's float pad, raises
// the flag, waits (bounded) for all peers and replaces state[0] by the global sum.
__global__ void norm_allreduce_kernel(PeerPtrs pads, PeerPtrs fpads, int my_rank, int world, int channel, int epoch,
                                      float* __restrict__ state, long long limit_cycles, int* err) {
  __shared__ float vals[MAX_PEERS];
  const int r = threadIdx.x;
  if (r < world) {
    const float mine = state[0];
    float* rf = reinterpret_cast<float*>(fpads.p[r]) + my_rank;
    *reinterpret_cast<volatile float*>(rf) = mine;
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(pads.p[r]) + channel * MAX_PEERS + my_rank, epoch);
    const int* local = reinterpret_cast<const int*>(pads.p[my_rank]) + channel * MAX_PEERS + r;
    const long long t0 = clock64();
    bool ok = true;
    while (ld_acquire_sys(local) < epoch) {
      if (clock64() - t0 > limit_cycles) { set_error(err, ERR_WAIT_PEER_FLAG); ok = false; break; }
    }
    vals[r] = ok ? *reinterpret_cast<volatile float*>(reinterpret_cast<float*>(fpads.p[my_rank]) + r) : 0.f;
  }
  __syncthreads();
  if (r == 0) {
    float s = 0.f;
    for (int i = 0; i < world; ++i) s += vals[i];
    state[0] = s;
  }
}

// AdamW on the local shard; the refreshed bf16 values go to dst[k] + lo for every k < ndst.
__global__ void adamw_push_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                  const float* __restrict__ g, PeerPtrs dst, int ndst, long long lo,
                                  const float* __restrict__ state, long long n, float lr, float beta1, float beta2,
                                  float eps, float wd, float bc1, float bc2) {
  const float coef = state[1];
  const bool go = state[2] != 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    if (go) {
      const float4 gv = reinterpret_cast<const float4*>(g)[i];
      float4 mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
      float* pp = reinterpret_cast<float*>(&pv);
      float* mm = reinterpret_cast<float*>(&mv);
      float* vq = reinterpret_cast<float*>(&vv);
      const float* gg = reinterpret_cast<const float*>(&gv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float gi = gg[e] * coef;
        mm[e] = beta1 * mm[e] + (1.f - beta1) * gi;
        vq[e] = beta2 * vq[e] + (1.f - beta2) * gi * gi;
        float x = pp[e];
        x -= lr * wd * x;
        x -= lr * (mm[e] / bc1) / (sqrtf(vq[e] / bc2) + eps);
        pp[e] = x;
      }
      reinterpret_cast<float4*>(p)[i] = pv;
      reinterpret_cast<float4*>(m)[i] = mv;
      reinterpret_cast<float4*>(v)[i] = vv;
    }
    uint2 pk;
    pk.x = pack_bf16(pv.x, pv.y);
    pk.y = pack_bf16(pv.z, pv.w);
    for (int k = 0; k < ndst; ++k)
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(dst.p[k]) + lo)[i] = pk;
  }
}

// dst[k][dst_off + i] = src[i] for a bf16 range (16-byte vectors).
__global__ void push_copy_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, int ndst, long long dst_off,
                                 long long n) {
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(src)[i];
    for (int k = 0; k < ndst; ++k) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[k]) + dst_off)[i] = v;
  }
}

// One launch for a whole re-shard plan (tensor-parallel rollout replicas). Every op is a 2-D strided
// copy of bf16 (rows x cols, 16-byte vectors) from this rank's flat parameter buffer into the flat
// buffer of TP rank `dst` of EVERY replica: the source vector is loaded once and stored n_rep times.
// Work is cut into chunks of PLAN_CHUNK vectors; chunk_start[] is the exclusive prefix sum of the
// ops' chunk counts, so a CTA finds its op by bisection. With fp8 != 0 the copy casts instead:
// 128-element blocks (16 consecutive threads, 8 values each) become e4m3 values plus
// one fp32 scale per block, written to the q / s destination tables.
struct PushOp {
  long long src_off;   // elements, in the source flat buffer
  long long dst_off;   // elements, in the destination flat buffer
  int dst;             // TP rank inside a replica
  int rows, cols;      // cols % 8 == 0
  int ld_src, ld_dst;  // elements
  int pad;
};
static constexpr int PLAN_CHUNK = 4096;  // 16-byte vectors per work item (64 KiB)

__global__ void push_plan_kernel(const __nv_bfloat16* __restrict__ src, const PushOp* __restrict__ ops, int n_ops,
                                 const int* __restrict__ chunk_start, int total_chunks,
                                 void* const* __restrict__ dst_ptrs, int n_rep, int tp) {
  for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    int lo = 0, hi = n_ops - 1;
    while (lo < hi) {              // last op whose first chunk is <= chunk
      const int mid = (lo + hi + 1) >> 1;
      if (chunk_start[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    const PushOp op = ops[lo];
    const int c8 = op.cols >> 3;
    const long long total = (long long)op.rows * c8;
    const long long base = (long long)(chunk - chunk_start[lo]) * PLAN_CHUNK;
    const long long end = min(total, base + PLAN_CHUNK);
    for (long long i = base + threadIdx.x; i < end; i += blockDim.x) {
      const int r = (int)(i / c8), c = (int)(i - (long long)r * c8);
      const uint4 v = reinterpret_cast<const uint4*>(src + op.src_off + (size_t)r * op.ld_src)[c];
      for (int k = 0; k < n_rep; ++k) {
        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst_ptrs[k * tp + op.dst]);
        reinterpret_cast<uint4*>(d + op.dst_off + (size_t)r * op.ld_dst)[c] = v;
      }
    }
  }
}

// Same plan, casting to block-scaled e4m3 on the way: every row of an op is cut into 1 x 128 blocks
// (cols % 128 == 0, dst_off % 128 == 0, ld_dst % 128 == 0); 16 threads share a block (8 values each),
// take its amax with shuffles inside their half-warp, and write 8 e4m3 bytes each plus one fp32 scale
// per block at (element offset / 128) of the scale buffer.
__global__ void push_plan_fp8_kernel(const __nv_bfloat16* __restrict__ src, const PushOp* __restrict__ ops, int n_ops,
                                     const int* __restrict__ chunk_start, int total_chunks,
                                     void* const* __restrict__ dstq, void* const* __restrict__ dsts, int n_rep, int tp,
                                     int pow2) {
  for (int chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    int lo = 0, hi = n_ops - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (chunk_start[mid] <= chunk) lo = mid; else hi = mid - 1;
    }
    const PushOp op = ops[lo];
    const int c8 = op.cols >> 3;
    const long long total = (long long)op.rows * c8;
    const long long base = (long long)(chunk - chunk_start[lo]) * PLAN_CHUNK;
    const long long end = min(total, base + PLAN_CHUNK);
    // total and PLAN_CHUNK are multiples of 16 vectors, so the 16 threads of a block stay together
    for (long long i0 = base; i0 < end; i0 += blockDim.x) {
      const long long i = i0 + threadIdx.x;
      const bool live = i < end;
      const long long ii = live ? i : base;
      const int r = (int)(ii / c8), c = (int)(ii - (long long)r * c8);
      const uint4 v = reinterpret_cast<const uint4*>(src + op.src_off + (size_t)r * op.ld_src)[c];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      float f[8];
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 t = unpack_bf16(w[e]);
        f[2 * e] = t.x; f[2 * e + 1] = t.y;
        amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      float scale = fmaxf(amax, 1e-12f) / 448.f;
      if (pow2) scale = exp2f(ceilf(log2f(scale)));
      const float inv = 1.f / scale;
      __nv_fp8x4_e4m3 q0(make_float4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv));
      __nv_fp8x4_e4m3 q1(make_float4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv));
      if (!live) continue;
      const size_t e_off = (size_t)op.dst_off + (size_t)r * op.ld_dst + (size_t)c * 8;
      for (int k = 0; k < n_rep; ++k) {
        uint8_t* dq = reinterpret_cast<uint8_t*>(dstq[k * tp + op.dst]);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&q0);
        pk.y = *reinterpret_cast<uint32_t*>(&q1);
        *reinterpret_cast<uint2*>(dq + e_off) = pk;
        if ((c & 15) == 0) reinterpret_cast<float*>(dsts[k * tp + op.dst])[e_off >> 7] = scale;
      }
    }
  }
}

static int grid_of(long long work) {
  long long b = (work + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace ab2

extern "C" {
using namespace ab2;

static PeerPtrs make_ptrs(void* const* ptrs, int n) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.p[i] = i < n ? ptrs[i] : nullptr;
  return pp;
}

// pads: device pointers of every rank's signal pad (int32[channels][16]), indexed by rank.
// timeout_ms bounds the wait; on expiry the kernel records ERR_WAIT_PEER_FLAG and returns.
int ab2_signal_barrier(void* const* pads, int my_rank, int world, int channel, int epoch, int timeout_ms,
                       void* stream) {
  if (world > MAX_PEERS) return 10;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  const long long limit = (long long)timeout_ms * 1900000LL;
  signal_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_ptrs(pads, world), my_rank, world, channel, epoch,
                                                            limit, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_rs_sumsq(void* const* grads, int world, long long lo, long long n, float* out, float* state, float scale,
                 void* stream) {
  if (world > MAX_PEERS || (n & 3) || (lo & 3)) return 10;
  if (n <= 0) return 0;
  rs_sumsq_kernel<<<grid_of(n / 4), 256, 0, (cudaStream_t)stream>>>(make_ptrs(grads, world), world, lo, n, out, state,
                                                                    scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// mc_grads: multicast (NVLS) address of the symmetric fp32 gradient buffer.
int ab2_rs_sumsq_multimem(const void* mc_grads, long long lo, long long n, float* out, float* state, float scale, void* stream) {
  if (!mc_grads || (n & 3) || (lo & 3)) return 10;
  if (n <= 0) return 0;
  rs_sumsq_multimem_kernel<<<grid_of(n / 4), 256, 0, (cudaStream_t)stream>>>((const float*)mc_grads, lo, n, out, state, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_norm_allreduce(void* const* pads, void* const* fpads, int my_rank, int world, int channel, int epoch,
                       float* state, int timeout_ms, void* stream) {
  if (world > MAX_PEERS) return 10;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  norm_allreduce_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_ptrs(pads, world), make_ptrs(fpads, world), my_rank,
                                                            world, channel, epoch, state,
                                                            (long long)timeout_ms * 1900000LL, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_adamw_push(float* p, float* m, float* v, const float* g, void* const* dst, int ndst, long long lo,
                   const float* state, long long n, float lr, float beta1, float beta2, float eps, float wd, int step,
                   void* stream) {
  if (ndst > MAX_PEERS || (n & 3) || (lo & 3)) return 10;
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  adamw_push_kernel<<<grid_of(n / 4), 256, 0, (cudaStream_t)stream>>>(p, m, v, g, make_ptrs(dst, ndst), ndst, lo, state,
                                                                      n, lr, beta1, beta2, eps, wd, bc1, bc2);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_push_copy(const void* src, void* const* dst, int ndst, long long dst_off, long long n, void* stream) {
  if (ndst > MAX_PEERS || (n & 7) || (dst_off & 7)) return 10;
  if (n <= 0 || ndst <= 0) return 0;
  push_copy_kernel<<<grid_of(n / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, make_ptrs(dst, ndst),
                                                                     ndst, dst_off, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// Executes a re-shard plan in one launch. ops / chunk_start / dst tables live in device memory:
// ops[n_ops] (PushOp, 40 bytes each), chunk_start[n_ops] (int32, exclusive prefix sum of
// ceil(rows * cols / 8 / 4096)), dst_ptrs[n_rep * tp] (destination flat buffers, replica-major).
// fp8 == 0: bf16 copy into dst_ptrs. fp8 != 0: block-scaled e4m3 cast into dst_ptrs (values) and
// scale_ptrs (fp32, one per 128 elements); then every op needs cols, dst_off and ld_dst to be multiples of 128.
int ab2_push_plan(const void* src, const void* ops, int n_ops, const void* chunk_start, int total_chunks,
                  const void* dst_ptrs, const void* scale_ptrs, int n_rep, int tp, int fp8, int pow2_scales, void* stream) {
  if (n_ops <= 0 || total_chunks <= 0 || n_rep <= 0) return 0;
  if (tp <= 0 || !src || !ops || !chunk_start || !dst_ptrs) return 10;
  const int grid = total_chunks < 148 * 8 ? total_chunks : 148 * 8;
  if (fp8) {
    if (!scale_ptrs) return 10;
    push_plan_fp8_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, (const PushOp*)ops, n_ops,
                                                                  (const int*)chunk_start, total_chunks,
                                                                  (void* const*)dst_ptrs, (void* const*)scale_ptrs, n_rep,
                                                                  tp, pow2_scales);
  } else {
    push_plan_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, (const PushOp*)ops, n_ops,
                                                              (const int*)chunk_start, total_chunks,
                                                              (void* const*)dst_ptrs, n_rep, tp);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

}
