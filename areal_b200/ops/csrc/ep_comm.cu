// Expert-parallel token dispatch and combine as two peer-memory kernels.
//
// A mixture-of-experts layer under expert parallelism moves every routed token copy to the
// rank that owns its expert and moves the expert outputs back. Done with a library all-to-all
// this is: gather rows by token -> all-to-all -> regroup by local expert -> experts ->
// inverse regroup -> all-to-all -> scale by the gate weight -> scatter-add by token.
// Here each direction is ONE kernel over NVLink peer memory:
//
//   ep_dispatch   row i of the expert-sorted list is src[token_of[i]] (optionally times
//                 scale[i]); the warp stores it straight into rank drank[i]'s receive
//                 buffer at row drow[i], which is its final position in that rank's
//                 (local expert, source rank) order: gather + transfer + regroup in one pass.
//                 With `ys` given it also returns dw[i] = <src[token_of[i]], ys[i]>, the gate
//                 weight gradient needed by the combine backward.
//   ep_combine    out[t] = sum_j w[i] * buf[drank[i]][drow[i]] with i = inv[t*k + j]: the warp
//                 of token t pulls its k expert outputs from the owning ranks, weights and
//                 sums them in fp32: transfer + inverse regroup + weighting + scatter-add in
//                 one pass. Optionally keeps the pulled rows (ys_save) for the backward.
//
// The backward of a dispatch is a combine with unit weights and vice versa, so the same two
// kernels serve both directions. Ordering between ranks comes from the bounded flag barrier
// of comm.cu, launched between the writes and the reads of a phase; these kernels never wait.
//
// Replaces the NCCL all-to-all token dispatcher of
// areal/experimental/models/archon/expert_parallel.py:163-240 and the permute / unpermute
// steps of areal/experimental/models/archon/moe/moe.py.
#include "common.cuh"

namespace ab2 {

static constexpr int EP_MAX_PEERS = 16;

struct EpPeerPtrs {
  void* p[EP_MAX_PEERS];
};

// One warp per sorted row. H is a multiple of 8 (16-byte vectors).
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src,
                                   const int* __restrict__ token_of, const int* __restrict__ drank,
                                   const int* __restrict__ drow, const float* __restrict__ scale,
                                   const __nv_bfloat16* __restrict__ ys, float* __restrict__ dw, EpPeerPtrs dst,
                                   long long dst_off, int n_rows, int H, int world, long long capacity_rows, int* err) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H >> 3;
  for (int i = warp; i < n_rows; i += nwarps) {
    const int rk = drank[i];
    const long long row = drow[i];
    if (rk < 0 || rk >= world || row < 0 || row >= capacity_rows) {  // a bad plan must not become a bad store
      if (lane == 0) set_error(err, ERR_BOUNDS);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)token_of[i] * ld_src);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[rk]) + dst_off + (size_t)row * H);
    const float sc = scale ? scale[i] : 1.f;
    const uint4* y = ys ? reinterpret_cast<const uint4*>(ys + (size_t)i * H) : nullptr;
    float dot = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      uint4 v = s[c];
      if (y) {
        const uint4 yv = y[c];
        const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
        const uint32_t* b = reinterpret_cast<const uint32_t*>(&yv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 fa = unpack_bf16(a[q]), fb = unpack_bf16(b[q]);
          dot += fa.x * fb.x + fa.y * fb.y;
        }
      }
      if (scale) {
        uint32_t* a = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16(a[q]);
          a[q] = pack_bf16(f.x * sc, f.y * sc);
        }
      }
      d[c] = v;
    }
    if (y) {
      dot = warp_sum(dot);
      if (lane == 0) dw[i] = dot;
    }
  }
}

// One warp per token; lane j < k resolves the address and weight of slot j once into the
// warp's shared-memory slots, the row loop reads them from there (broadcast). k <= 32.
__global__ void ep_combine_kernel(EpPeerPtrs srcbuf, long long src_off, const int* __restrict__ inv,
                                  const int* __restrict__ drank, const int* __restrict__ drow,
                                  const float* __restrict__ w, __nv_bfloat16* __restrict__ out, long long ld_out,
                                  __nv_bfloat16* __restrict__ ys_save, int T, int k, int H, int world,
                                  long long capacity_rows, int* err) {
  __shared__ unsigned long long s_ptr[8][32];
  __shared__ float s_w[8][32];
  __shared__ int s_i[8][32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H >> 3;
  for (int t = warp; t < T; t += nwarps) {
    __syncwarp();  // the previous token's slots are no longer read
    if (lane < k) {
      const int i = inv[(size_t)t * k + lane];
      const int rk = drank[i];
      const long long row = drow[i];
      unsigned long long ptr = 0;
      float wt = 0.f;
      if (rk < 0 || rk >= world || row < 0 || row >= capacity_rows) {
        set_error(err, ERR_BOUNDS);  // the slot contributes nothing
      } else {
        ptr = reinterpret_cast<unsigned long long>(reinterpret_cast<const __nv_bfloat16*>(srcbuf.p[rk]) + src_off +
                                                   (size_t)row * H);
        wt = w ? w[i] : 1.f;
      }
      s_ptr[wib][lane] = ptr;
      s_w[wib][lane] = wt;
      s_i[wib][lane] = i;
    }
    __syncwarp();
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * ld_out);
    for (int c = lane; c < nvec; c += 32) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int j = 0; j < k; ++j) {
        const unsigned long long pj = s_ptr[wib][j];
        if (pj == 0) continue;
        const float wj = s_w[wib][j];
        const uint4 v = reinterpret_cast<const uint4*>(pj)[c];
        if (ys_save) reinterpret_cast<uint4*>(ys_save + (size_t)s_i[wib][j] * H)[c] = v;
        const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16(a[q]);
          acc[2 * q] += wj * f.x;
          acc[2 * q + 1] += wj * f.y;
        }
      }
      uint4 r;
      r.x = pack_bf16(acc[0], acc[1]);
      r.y = pack_bf16(acc[2], acc[3]);
      r.z = pack_bf16(acc[4], acc[5]);
      r.w = pack_bf16(acc[6], acc[7]);
      o[c] = r;
    }
  }
}

static int ep_grid(long long warps) {
  long long b = (warps + 7) / 8;  // 8 warps per CTA
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace ab2

extern "C" {
using namespace ab2;

static EpPeerPtrs ep_ptrs(void* const* ptrs, int n) {
  EpPeerPtrs pp;
  for (int i = 0; i < EP_MAX_PEERS; ++i) pp.p[i] = i < n ? ptrs[i] : nullptr;
  return pp;
}

// src [*, ld_src] bf16; token_of / drank / drow int32 [n_rows]; scale fp32 [n_rows] or null;
// ys bf16 [n_rows, H] with dw fp32 [n_rows], or both null. dst: every rank's receive buffer
// (bf16), rows of H elements starting dst_off elements into the buffer.
int ab2_ep_dispatch(const void* src, long long ld_src, const void* token_of, const void* drank, const void* drow,
                    const void* scale, const void* ys, void* dw, void* const* dst, int world, long long dst_off,
                    int n_rows, int H, long long capacity_rows, void* stream) {
  if (world > EP_MAX_PEERS || world < 1 || (H & 7) || (ld_src & 7) || (dst_off & 7)) return 10;
  if ((ys == nullptr) != (dw == nullptr)) return 11;
  if (n_rows <= 0) return 0;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  ep_dispatch_kernel<<<ep_grid(n_rows), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, ld_src, (const int*)token_of, (const int*)drank, (const int*)drow, (const float*)scale,
      (const __nv_bfloat16*)ys, (float*)dw, ep_ptrs(dst, world), dst_off, n_rows, H, world, capacity_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// srcbuf: every rank's buffer of expert outputs (bf16 rows of H). inv int32 [T*k] maps slot
// (t, j) to its sorted row; w fp32 [T*k] indexed by sorted row, or null for unit weights.
// out bf16 [T, ld_out]; ys_save bf16 [T*k, H] or null.
int ab2_ep_combine(void* const* srcbuf, int world, long long src_off, const void* inv, const void* drank,
                   const void* drow, const void* w, void* out, long long ld_out, void* ys_save, int T, int k, int H,
                   long long capacity_rows, void* stream) {
  if (world > EP_MAX_PEERS || world < 1 || (H & 7) || (ld_out & 7) || (src_off & 7) || k < 1 || k > 32) return 10;
  if (T <= 0) return 0;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  ep_combine_kernel<<<ep_grid(T), 256, 0, (cudaStream_t)stream>>>(
      ep_ptrs(srcbuf, world), src_off, (const int*)inv, (const int*)drank, (const int*)drow, (const float*)w,
      (__nv_bfloat16*)out, ld_out, (__nv_bfloat16*)ys_save, T, k, H, world, capacity_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
