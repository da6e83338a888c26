// Tensor-parallel inference: the sum over the ranks of a row-parallel product, fused with the
// residual add and the RMSNorm that follow it.
//
// A row-parallel projection (o_proj, down_proj) of a tensor-parallel layer leaves every rank with a
// PARTIAL [M, H] result. Its GEMM (ab2_gemm_bf16_bcast, gemm.cu) stores that partial from inside its
// epilogue into slot `source rank` of the receive buffer of EVERY rank of the group (peer stores over
// NVLink) and then adds to each receiver's arrival counter. The kernel below is the consumer: it
// waits (bounded) until its own counter shows that all P partials of this product have landed, sums
// them in fp32, adds the residual stream, writes the new residual and the normalised activations.
// Together the pair replaces  GEMM -> NCCL all-reduce -> residual add + RMSNorm  (three kernels and a
// library collective) by two kernels whose communication is plain peer memory traffic, so a decode
// step of a tensor-parallel replica can be captured in a CUDA graph.
//
// Counters only grow. `state[0]` holds the count this rank has already consumed; a launch waits for
// state[0] + expected and its last CTA stores that value back, so graph replays need no host-side
// argument updates. Two buffer / counter sets alternate between consecutive products: a rank can run
// ahead of a peer by at most one product (it blocks in the next consumer until that peer has
// produced), so the set written by product k + 2 is no longer read by anybody's consumer of product k.
//
// Role in the reference: the tensor-parallel all-reduce inside the SGLang / vLLM servers behind
// areal/engine/sglang_remote.py.
#include "common.cuh"

namespace ab2 {

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float block_sum_tp(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// slots: [P][M][H] bf16 (this rank's receive buffer of the current set), one CTA of TPR threads per
// row. H % 8 == 0 and H <= 8 * VEC_PER_THREAD * TPR. The thread-to-column mapping and the order of
// the sum of squares are those of rmsnorm_fwd_kernel (elementwise.cu) for the same H, so the result
// is bit-identical to  all-reduce in bf16 -> residual add + RMSNorm  with the unfused kernels.
template <int TPR, int VEC_PER_THREAD>
__global__ void __launch_bounds__(TPR)
tp_reduce_rmsnorm_kernel(const __nv_bfloat16* __restrict__ slots, int P, long long slot_stride,
                         const __nv_bfloat16* __restrict__ resid_in, __nv_bfloat16* __restrict__ resid_out,
                         __nv_bfloat16* __restrict__ x_out, const __nv_bfloat16* __restrict__ w, float eps, int M, int H,
                         const unsigned long long* __restrict__ counter, unsigned long long* __restrict__ state,
                         unsigned long long expected, long long limit_cycles, int* err) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  __shared__ int proceed;
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    const unsigned long long target = state[0] + expected;
    int ok = 1;
    if (ld_acquire_sys_u64(counter) < target) {
      const long long t0 = clock64();
      while (ld_acquire_sys_u64(counter) < target) {
        if (clock64() - t0 > limit_cycles) {
          set_error(err, ERR_WAIT_PEER_FLAG);
          ok = 0;
          break;
        }
      }
    }
    proceed = ok;
  }
  __syncthreads();
  // after a give-up the row is still written (from whatever has arrived) so that nothing downstream
  // reads uninitialised memory; the host sees the error word and drops the step
  const int nvec = H >> 3;
  float v[VEC_PER_THREAD][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int c = threadIdx.x + i * TPR;
#pragma unroll
    for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
    if (c < nvec) {
      for (int p = 0; p < P; ++p) {
        const uint4 raw = reinterpret_cast<const uint4*>(slots + (size_t)p * slot_stride + (size_t)row * H)[c];
        const uint32_t q[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16(q[e]);
          v[i][2 * e] += f.x;
          v[i][2 * e + 1] += f.y;
        }
      }
      // the sum of the partials is rounded to bf16 first: bit-identical to an all-reduce in bf16
      // followed by the unfused residual + norm kernel (for two ranks)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16(pack_bf16(v[i][2 * e], v[i][2 * e + 1]));
        v[i][2 * e] = f.x;
        v[i][2 * e + 1] = f.y;
      }
      if (resid_in != nullptr) {
        const uint4 raw = reinterpret_cast<const uint4*>(resid_in + (size_t)row * H)[c];
        const uint32_t q[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16(q[e]);
          v[i][2 * e] += f.x;
          v[i][2 * e + 1] += f.y;
        }
      }
      // the residual stream is kept in bf16: normalise what is stored, as the unfused kernels do
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pk[e] = pack_bf16(v[i][2 * e], v[i][2 * e + 1]);
        const float2 f = unpack_bf16(pk[e]);
        v[i][2 * e] = f.x;
        v[i][2 * e + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      reinterpret_cast<uint4*>(resid_out + (size_t)row * H)[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
  const float tot = (TPR == 32) ? warp_sum(ss) : block_sum_tp(ss, red);
  const float rs = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; ++i) {
    const int c = threadIdx.x + i * TPR;
    if (c < nvec) {
      const uint4 wr = reinterpret_cast<const uint4*>(w)[c];
      const uint32_t q[4] = {wr.x, wr.y, wr.z, wr.w};
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16(q[e]);
        pk[e] = pack_bf16(v[i][2 * e] * rs * f.x, v[i][2 * e + 1] * rs * f.y);
      }
      reinterpret_cast<uint4*>(x_out + (size_t)row * H)[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
  // the last CTA to finish publishes the consumed count for the next launch on this set
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned long long done = atomicAdd(&state[1], 1ULL) + 1ULL;
    if (done == (unsigned long long)gridDim.x) {
      state[1] = 0ULL;
      if (proceed) state[0] = state[0] + expected;
      else state[0] = ld_acquire_sys_u64(counter);   // resynchronise on what did arrive
      __threadfence();
    }
  }
}

}  // namespace ab2

extern "C" {

// x_out, resid_out [M, H] bf16 = RMSNorm / sum of (the P partials in `slots` + resid_in).
// slots: this rank's receive buffer [P][slot_stride elements], rows dense with H columns.
// counter / state: this rank's arrival counter and {consumed count, CTA ticket} pair of the set.
// expected = P * M * ceil(H / 32) (what P producers add for one product).
int ab2_tp_reduce_rmsnorm(const void* slots, int P, long long slot_stride, const void* resid_in, void* resid_out, void* x_out,
                          const void* w, float eps, int M, int H, const void* counter, void* state, int timeout_ms, void* stream) {
  using namespace ab2;
  if (M <= 0) return 0;
  if (P < 1 || (H & 7) || H > 8192) return 10;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  const unsigned long long expected = (unsigned long long)P * (unsigned long long)M * (unsigned long long)((H + 31) / 32);
  const long long limit = (long long)timeout_ms * 1900000LL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // same (threads per row, vectors per thread) as ab2_rmsnorm_fwd picks for this H
  if (H <= 256) {
    launch_pdl(tp_reduce_rmsnorm_kernel<32, 1>, dim3(M), dim3(32), 0, s, (const __nv_bfloat16*)slots, P, slot_stride,
               (const __nv_bfloat16*)resid_in, (__nv_bfloat16*)resid_out, (__nv_bfloat16*)x_out, (const __nv_bfloat16*)w, eps, M, H,
               (const unsigned long long*)counter, (unsigned long long*)state, expected, limit, err);
  } else if (H <= 2048) {
    launch_pdl(tp_reduce_rmsnorm_kernel<128, 2>, dim3(M), dim3(128), 0, s, (const __nv_bfloat16*)slots, P, slot_stride,
               (const __nv_bfloat16*)resid_in, (__nv_bfloat16*)resid_out, (__nv_bfloat16*)x_out, (const __nv_bfloat16*)w, eps, M, H,
               (const unsigned long long*)counter, (unsigned long long*)state, expected, limit, err);
  } else if (H <= 4096) {
    launch_pdl(tp_reduce_rmsnorm_kernel<128, 4>, dim3(M), dim3(128), 0, s, (const __nv_bfloat16*)slots, P, slot_stride,
               (const __nv_bfloat16*)resid_in, (__nv_bfloat16*)resid_out, (__nv_bfloat16*)x_out, (const __nv_bfloat16*)w, eps, M, H,
               (const unsigned long long*)counter, (unsigned long long*)state, expected, limit, err);
  } else {
    launch_pdl(tp_reduce_rmsnorm_kernel<256, 4>, dim3(M), dim3(256), 0, s, (const __nv_bfloat16*)slots, P, slot_stride,
               (const __nv_bfloat16*)resid_in, (__nv_bfloat16*)resid_out, (__nv_bfloat16*)x_out, (const __nv_bfloat16*)w, eps, M, H,
               (const unsigned long long*)counter, (unsigned long long*)state, expected, limit, err);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
