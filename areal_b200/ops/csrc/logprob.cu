// Per-token log-probability / entropy from fp32 logits (one vocabulary shard or the full
// vocabulary), and the matching backward that emits bf16 dlogits for the LM-head GEMMs.
// Also the vocab-parallel partial form: (max, sum-exp, sum exp*z, target logit) per row so
// that tensor-parallel ranks can combine their shards with one small reduction.
//
// Semantics follow areal/utils/functional/vocab_parallel.py:16-82 (log_softmax of
// logits/temperature gathered at the label, entropy = -sum p log p) and the sharded form
// at :120-195 of the same file.
#include "common.cuh"

namespace ab2 {

struct RowStat {
  float m;  // running max of z
  float s;  // sum exp(z - m)
  float a;  // sum exp(z - m) * z
};

__device__ __forceinline__ void stat_add(RowStat& st, float z) {
  if (z > st.m) {
    const float r = __expf(st.m - z);
    st.s = st.s * r + 1.f;
    st.a = st.a * r + z;
    st.m = z;
  } else {
    const float e = __expf(z - st.m);
    st.s += e;
    st.a += e * z;
  }
}
__device__ __forceinline__ void stat_merge(RowStat& x, const RowStat& y) {
  const float m = fmaxf(x.m, y.m);
  const float rx = (x.m == -INFINITY) ? 0.f : __expf(x.m - m);
  const float ry = (y.m == -INFINITY) ? 0.f : __expf(y.m - m);
  x.s = x.s * rx + y.s * ry;
  x.a = x.a * rx + y.a * ry;
  x.m = m;
}

__device__ __forceinline__ RowStat block_stat(RowStat st, RowStat* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    RowStat y;
    y.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    y.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    y.a = __shfl_xor_sync(0xffffffffu, st.a, o);
    stat_merge(st, y);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = st;
  __syncthreads();
  RowStat t;
  t.m = -INFINITY; t.s = 0.f; t.a = 0.f;
  if (l < nw) t = red[l];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    RowStat y;
    y.m = __shfl_xor_sync(0xffffffffu, t.m, o);
    y.s = __shfl_xor_sync(0xffffffffu, t.s, o);
    y.a = __shfl_xor_sync(0xffffffffu, t.a, o);
    stat_merge(t, y);
  }
  return t;
}

// One CTA per row. logits: [rows, ld] fp32 (V valid columns). labels are global vocabulary
// ids; this shard covers [vocab_start, vocab_start + V).
//   partial == 0: writes logp[row], entropy[row], lse[row] (lse of z = logits * inv_temp).
//   partial == 1: writes part[row*4 + {0,1,2,3}] = {max, sumexp, sum exp*z, target z or 0}.
__global__ void logprob_fwd_kernel(const float* __restrict__ logits, const int* __restrict__ labels,
                                   float* __restrict__ logp, float* __restrict__ entropy,
                                   float* __restrict__ lse, float* __restrict__ part, int rows, int V,
                                   long long ld, float inv_temp, int vocab_start, int partial) {
  __shared__ RowStat red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* z = logits + (size_t)row * ld;
    RowStat st;
    st.m = -INFINITY; st.s = 0.f; st.a = 0.f;
    const int V4 = V >> 2;
    const float4* z4 = reinterpret_cast<const float4*>(z);
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
      const float4 v = z4[i];
      stat_add(st, v.x * inv_temp);
      stat_add(st, v.y * inv_temp);
      stat_add(st, v.z * inv_temp);
      stat_add(st, v.w * inv_temp);
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) stat_add(st, z[i] * inv_temp);
    st = block_stat(st, red);
    if (threadIdx.x == 0) {
      const int lab = labels[row] - vocab_start;
      const bool mine = lab >= 0 && lab < V;
      const float zt = mine ? z[lab] * inv_temp : 0.f;
      if (partial) {
        part[(size_t)row * 4 + 0] = st.m;
        part[(size_t)row * 4 + 1] = st.s;
        part[(size_t)row * 4 + 2] = st.a;
        part[(size_t)row * 4 + 3] = zt;
      } else {
        const float l = st.m + __logf(st.s);
        logp[row] = zt - l;
        entropy[row] = l - st.a / st.s;
        lse[row] = l;
      }
    }
  }
}

// dlogits[row, j] = inv_temp * ( g_logp * (1[j==label] - p_j) - g_ent * p_j * (log p_j + H) )
// with p_j = exp(z_j - lse). lse / entropy are the *global* row values (after any
// vocab-parallel reduction). Output bf16 [rows, ld_out].
__global__ void logprob_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ labels,
                                   const float* __restrict__ lse, const float* __restrict__ entropy,
                                   const float* __restrict__ g_logp, const float* __restrict__ g_ent,
                                   __nv_bfloat16* __restrict__ dlogits, int rows, int V, long long ld,
                                   long long ld_out, float inv_temp, int vocab_start) {
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* z = logits + (size_t)row * ld;
    __nv_bfloat16* d = dlogits + (size_t)row * ld_out;
    const float l = lse[row];
    const float gl = g_logp ? g_logp[row] : 0.f;
    const float ge = g_ent ? g_ent[row] : 0.f;
    const float H = entropy ? entropy[row] : 0.f;
    const int lab = labels[row] - vocab_start;
    const int V4 = V >> 2;
    const float4* z4 = reinterpret_cast<const float4*>(z);
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
      const float4 v = z4[i];
      const float zz[4] = {v.x * inv_temp, v.y * inv_temp, v.z * inv_temp, v.w * inv_temp};
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lp = zz[e] - l;
        const float p = __expf(lp);
        float g = -gl * p;
        if (ge != 0.f) g -= ge * p * (lp + H);
        if (i * 4 + e == lab) g += gl;
        o[e] = g * inv_temp;
      }
      uint2 pk;
      pk.x = pack_bf16(o[0], o[1]);
      pk.y = pack_bf16(o[2], o[3]);
      reinterpret_cast<uint2*>(d)[i] = pk;
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) {
      const float lp = z[i] * inv_temp - l;
      const float p = __expf(lp);
      float g = -gl * p;
      if (ge != 0.f) g -= ge * p * (lp + H);
      if (i == lab) g += gl;
      d[i] = __float2bfloat16(g * inv_temp);
    }
  }
}

// Combines vocab-parallel partials: parts[r][row][4] for r in [0, nparts) -> logp, entropy, lse.
__global__ void logprob_combine_kernel(const float* __restrict__ parts, int nparts, long long part_stride,
                                       float* __restrict__ logp, float* __restrict__ entropy,
                                       float* __restrict__ lse, int rows) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  RowStat st;
  st.m = -INFINITY; st.s = 0.f; st.a = 0.f;
  float zt = 0.f;
  for (int r = 0; r < nparts; ++r) {
    const float* p = parts + (size_t)r * part_stride + (size_t)row * 4;
    RowStat y;
    y.m = p[0]; y.s = p[1]; y.a = p[2];
    stat_merge(st, y);
    zt += p[3];
  }
  const float l = st.m + __logf(st.s);
  logp[row] = zt - l;
  entropy[row] = l - st.a / st.s;
  lse[row] = l;
}

}  // namespace ab2

extern "C" {
using namespace ab2;

int ab2_logprob_fwd(const float* logits, const int* labels, float* logp, float* entropy, float* lse,
                    float* part, int rows, int V, long long ld, float temperature, int vocab_start,
                    int partial, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 4) return 10;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  logprob_fwd_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(logits, labels, logp, entropy, lse, part, rows,
                                                             V, ld, 1.f / temperature, vocab_start, partial);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_logprob_bwd(const float* logits, const int* labels, const float* lse, const float* entropy,
                    const float* g_logp, const float* g_ent, void* dlogits, int rows, int V, long long ld,
                    long long ld_out, float temperature, int vocab_start, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 4 || ld_out % 4) return 10;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  logprob_bwd_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(logits, labels, lse, entropy, g_logp, g_ent,
                                                             (__nv_bfloat16*)dlogits, rows, V, ld, ld_out,
                                                             1.f / temperature, vocab_start);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ab2_logprob_combine(const float* parts, int nparts, long long part_stride, float* logp, float* entropy,
                        float* lse, int rows, void* stream) {
  if (rows <= 0) return 0;
  logprob_combine_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(parts, nparts, part_stride,
                                                                               logp, entropy, lse, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
