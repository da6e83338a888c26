// Rollout-engine kernels: paged KV-cache append, paged decode attention (split-KV with a
// combine pass), and fused temperature / Gumbel-max sampling that also returns the
// log-probability of the sampled token.
//
// These take the place of the SGLang / vLLM (FlashInfer, sgl_kernel) kernels that the
// reference reaches through areal/engine/sglang_remote.py and areal/engine/vllm_remote.py.
#include <cstdlib>
#include <mutex>

#include "ab2_noalloc.h"
#include "common.cuh"

namespace ab2 {

// ------------------------------------------------------------------ KV append
// k, v: [n, Hkv, D] (token stride given) -> cache[slot[n]] where the cache is
// [num_slots, Hkv, D] (slot = page * page_size + offset). slot < 0 skips the token.
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                 const int* __restrict__ slots, int n, int row_elems, long long k_stride,
                                 long long v_stride) {
  pdl_wait();
  pdl_trigger();
  const int vec = row_elems >> 3;
  const long long total = (long long)n * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec), c = (int)(i - (long long)t * vec);
    const int s = slots[t];
    if (s < 0) continue;
    reinterpret_cast<uint4*>(kc + (size_t)s * row_elems)[c] = reinterpret_cast<const uint4*>(k + (size_t)t * k_stride)[c];
    reinterpret_cast<uint4*>(vc + (size_t)s * row_elems)[c] = reinterpret_cast<const uint4*>(v + (size_t)t * v_stride)[c];
  }
}

// ------------------------------------------------------------------ paged decode attention
// One CTA = (sequence b, kv head h, split s), 128 threads. The split's tokens are walked in chunks
// of 64: the chunk's K and V rows are brought into shared memory with 16-byte asynchronous copies
// (two stages, so one chunk is in flight while the other is consumed; three CTAs per SM keep about
// 100 KB of loads in flight), then every warp works on its own 16 rows of the chunk:
//   scores:  8 lanes per token, each lane 2 x 8 dims (conflict-free 128-byte reads of a row), the
//            query heads of the group in registers four at a time;
//   softmax: running (max, sum) per warp and query head, no block-wide exchange;
//   output:  lane = D/32 dims, probabilities broadcast from shared memory.
// The four warps' states are merged once at the end and the CTA writes an (m, l, o) partial.
constexpr int DEC_CHUNK = 64;

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D, int G>
__global__ void __launch_bounds__(128, 3)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ page_table,
                    const int* __restrict__ seq_lens, float* __restrict__ part_o, float* __restrict__ part_ml,
                    int Hq, int Hkv, int page_size, int max_pages, int num_splits, float scale, long long q_stride) {
  constexpr int NC = D / 64;            // 8-dim pieces per lane in the score phase
  constexpr int DPL = D / 32;           // dims per lane in the output phase
  constexpr int GH = G < 4 ? G : 4;     // query heads held in registers at a time
  constexpr int ROW_BYTES = D * 2;
  constexpr int STAGE_BYTES = 2 * DEC_CHUNK * ROW_BYTES;   // K rows then V rows
  constexpr int PIECES = DEC_CHUNK * ROW_BYTES / 16;       // 16-byte pieces per operand and chunk
  extern __shared__ __align__(128) unsigned char dsm[];
  float* sq = reinterpret_cast<float*>(dsm + 2 * STAGE_BYTES);      // [G][D] scaled queries
  float* sp = sq + G * D;                                           // [DEC_CHUNK][G] probabilities
  const int b = blockIdx.x, h = blockIdx.y, spl = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = tid >> 3, lg = tid & 7;
  const int len = seq_lens[b];
  const int per = (len + num_splits - 1) / num_splits;
  const int t0 = spl * per, t1 = min(len, t0 + per);
  const int n_chunks = t1 > t0 ? (t1 - t0 + DEC_CHUNK - 1) / DEC_CHUNK : 0;
  const int* pt = page_table + (size_t)b * max_pages;
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(dsm);
  const float sl2 = scale * 1.4426950408889634f;

  auto issue = [&](int c, int stage) {
    const int base = t0 + c * DEC_CHUNK;
#pragma unroll
    for (int i = 0; i < PIECES / 128; ++i) {
      const int idx = tid + i * 128;
      const int row = idx / (ROW_BYTES / 16), piece = idx % (ROW_BYTES / 16);
      const int t = base + row;
      const bool ok = t < t1;
      size_t off = 0;
      if (ok) {
        const int page = pt[t / page_size];
        off = (((size_t)page * page_size + (t % page_size)) * Hkv + h) * D + piece * 8;
      }
      const uint32_t dst = smem0 + stage * STAGE_BYTES + row * ROW_BYTES + piece * 16;
      cp_async16(dst, kc + off, ok);
      cp_async16(dst + DEC_CHUNK * ROW_BYTES, vc + off, ok);
    }
    cp_async_commit();
  };

  if (n_chunks > 0) issue(0, 0);
  for (int i = tid; i < G * D; i += 128)
    sq[i] = __bfloat162float(q[(size_t)b * q_stride + (size_t)h * G * D + i]) * sl2;
  __syncthreads();

  float m_run[G], l_run[G], o[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[g][e] = 0.f;
  }
  float qr[GH][NC * 8];
  if constexpr (G <= 4) {
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) qr[g][c * 8 + e] = sq[g * D + c * 64 + lg * 8 + e];
  }

  for (int c = 0; c < n_chunks; ++c) {
    const int stage = c & 1;
    if (c + 1 < n_chunks) {
      issue(c + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned char* ks = dsm + stage * STAGE_BYTES;
    const unsigned char* vs = ks + DEC_CHUNK * ROW_BYTES;
    const int base = t0 + c * DEC_CHUNK;
    // ---- scores of this warp's 16 rows: row = grp + 16 * i (grp = 4 * warp + 0..3)
    float sc[4][G];
#pragma unroll
    for (int g0 = 0; g0 < G; g0 += GH) {
      if constexpr (G > 4) {
#pragma unroll
        for (int g = 0; g < GH; ++g) {
          if (g0 + g >= G) break;            // G need not be a multiple of GH (e.g. 6 query heads per kv head)
#pragma unroll
          for (int cc = 0; cc < NC; ++cc)
#pragma unroll
            for (int e = 0; e < 8; ++e) qr[g][cc * 8 + e] = sq[(g0 + g) * D + cc * 64 + lg * 8 + e];
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = grp + 16 * i;
        float kf[NC * 8];
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) {
          const uint4 kk = *reinterpret_cast<const uint4*>(ks + row * ROW_BYTES + cc * 128 + lg * 16);
          const uint32_t ka[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 a = unpack_bf16(ka[j]);
            kf[cc * 8 + 2 * j] = a.x;
            kf[cc * 8 + 2 * j + 1] = a.y;
          }
        }
#pragma unroll
        for (int g = 0; g < GH; ++g) {
          if (g0 + g >= G) break;
          float s = 0.f;
#pragma unroll
          for (int e = 0; e < NC * 8; ++e) s += qr[g][e] * kf[e];
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          s += __shfl_xor_sync(0xffffffffu, s, 4);
          sc[i][g0 + g] = (base + row < t1) ? s : -INFINITY;
        }
      }
    }
    // ---- running max per warp, probabilities to shared memory, partial sums per group
    float alpha[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = fmaxf(fmaxf(sc[0][g], sc[1][g]), fmaxf(sc[2][g], sc[3][g]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float mn = fmaxf(m_run[g], mx);
      const float mref = (mn == -INFINITY) ? 0.f : mn;
      alpha[g] = fast_exp2(m_run[g] - mref);
      m_run[g] = mn;
      float ps = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float p = fast_exp2(sc[i][g] - mref);
        sc[i][g] = p;
        ps += p;
      }
      l_run[g] = l_run[g] * alpha[g] + ps;     // the group's rows (same value in its 8 lanes)
    }
    if (lg == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g) sp[(grp + 16 * i) * G + g] = sc[i][g];
    }
    __syncwarp();
    // ---- output: the same 16 rows, lane = DPL dims
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < DPL; ++e) o[g][e] *= alpha[g];
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
      const int row = 4 * warp + (j & 3) + 16 * (j >> 2);
      float vf[DPL];
      if constexpr (DPL == 4) {
        const uint2 vv = *reinterpret_cast<const uint2*>(vs + row * ROW_BYTES + lane * 8);
        const float2 a = unpack_bf16(vv.x), c2 = unpack_bf16(vv.y);
        vf[0] = a.x; vf[1] = a.y; vf[2] = c2.x; vf[3] = c2.y;
      } else {
        const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(vs + row * ROW_BYTES + lane * 4));
        vf[0] = a.x; vf[1] = a.y;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float p = sp[row * G + g];
#pragma unroll
        for (int e = 0; e < DPL; ++e) o[g][e] += p * vf[e];
      }
    }
    __syncthreads();   // every warp is done with this stage before the next copies land in it
  }

  // ---- merge the four warps (stage memory is free now)
#pragma unroll
  for (int g = 0; g < G; ++g) {
    l_run[g] += __shfl_xor_sync(0xffffffffu, l_run[g], 8);
    l_run[g] += __shfl_xor_sync(0xffffffffu, l_run[g], 16);
  }
  float* mo = reinterpret_cast<float*>(dsm);          // [4][G][D]
  float* mm = mo + 4 * G * D;                         // [4][G]
  float* ml = mm + 4 * G;                             // [4][G]
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int e = 0; e < DPL; ++e) mo[(warp * G + g) * D + lane * DPL + e] = o[g][e];
    if (lane == 0) {
      mm[warp * G + g] = m_run[g];
      ml[warp * G + g] = l_run[g];
    }
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i - g * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mm[w * G + g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mm[w * G + g];
      const float wt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mx);
      ll += ml[w * G + g] * wt;
      oo += mo[(w * G + g) * D + d] * wt;
    }
    const size_t pidx = ((size_t)b * Hq + (size_t)h * G + g) * num_splits + spl;
    part_o[pidx * D + d] = oo;
    if (d == 0) {
      part_ml[pidx * 2] = mx;
      part_ml[pidx * 2 + 1] = ll;
    }
  }
}

// ------------------------------------------------------------------ paged decode attention, tensor-core form
// Same decomposition as above (CTA = sequence x kv head x split, 64-token chunks staged by
// asynchronous copies, one warp per 16 tokens of the chunk), but the two products run on
// mma.sync m16n8k16 (bf16 in, fp32 out): the G query heads of the group are the rows of a
// 16-row tile (rows >= G are zero), S = Q K^T takes D/16 steps per 8 tokens, and the
// probabilities feed O += P V straight from the accumulator registers. About eight times fewer
// issued instructions than the scalar form, so the kernel follows the memory system instead of
// the issue slots. Rows of K / V / Q in shared memory are padded by 16 bytes so that the 8 x 8
// matrix loads touch distinct banks.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int D>
struct DecodeMmaCfg {
  static constexpr int STRIDE = D * 2 + 16;                       // bytes per staged row
  static constexpr int OPERAND_BYTES = DEC_CHUNK * STRIDE;
  static constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;           // K rows then V rows
  static constexpr int Q_BYTES = 16 * STRIDE;
  static constexpr int SLOT_BYTES = 2 * DEC_CHUNK * 8;               // row -> element offset of its K/V row, two chunks
  static constexpr int SMEM_BYTES = 2 * STAGE_BYTES + Q_BYTES + SLOT_BYTES;
};

template <int D>
__global__ void __launch_bounds__(128, 3)
paged_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                        const __nv_bfloat16* __restrict__ vc, const int* __restrict__ page_table,
                        const int* __restrict__ seq_lens, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int Hq, int Hkv, int G, int page_size, int max_pages, int num_splits, float scale, long long q_stride) {
  using Cfg = DecodeMmaCfg<D>;
  constexpr int STRIDE = Cfg::STRIDE;
  constexpr int KS = D / 16;                 // k-steps of S = Q K^T; also 16-dim column pairs of O
  pdl_wait();
  pdl_trigger();
  constexpr int PIECES = DEC_CHUNK * D * 2 / 16;
  extern __shared__ __align__(128) unsigned char dsm[];
  const int b = blockIdx.x, h = blockIdx.y, spl = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;    // row group / column pair inside a fragment
  const int len = seq_lens[b];
  const int per = (len + num_splits - 1) / num_splits;
  const int t0 = spl * per, t1 = min(len, t0 + per);
  const int n_chunks = t1 > t0 ? (t1 - t0 + DEC_CHUNK - 1) / DEC_CHUNK : 0;
  const int* pt = page_table + (size_t)b * max_pages;
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(dsm);
  const uint32_t sq_addr = smem0 + 2 * Cfg::STAGE_BYTES;
  const float sl2 = scale * 1.4426950408889634f;

  // Row offsets of a chunk are worked out once (64 threads, one row each: page lookup + the only
  // integer divisions of the copy path) and kept in shared memory, one chunk ahead of the copies.
  long long* s_off = reinterpret_cast<long long*>(dsm + 2 * Cfg::STAGE_BYTES + Cfg::Q_BYTES);   // [2][DEC_CHUNK], -1 = past the end
  auto plan = [&](int c) {
    if (tid < DEC_CHUNK) {
      const int t = t0 + c * DEC_CHUNK + tid;
      long long off = -1;
      if (t < t1) {
        const int page = pt[t / page_size];
        off = (((long long)page * page_size + (t % page_size)) * Hkv + h) * D;
      }
      s_off[(c & 1) * DEC_CHUNK + tid] = off;
    }
  };
  auto issue = [&](int c, int stage) {
#pragma unroll
    for (int i = 0; i < PIECES / 128; ++i) {
      const int idx = tid + i * 128;
      const int row = idx / (D / 8), piece = idx % (D / 8);
      const long long off = s_off[(c & 1) * DEC_CHUNK + row];
      const bool ok = off >= 0;
      const size_t src = ok ? (size_t)off + piece * 8 : 0;
      const uint32_t dst = smem0 + stage * Cfg::STAGE_BYTES + row * STRIDE + piece * 16;
      cp_async16(dst, kc + src, ok);
      cp_async16(dst + Cfg::OPERAND_BYTES, vc + src, ok);
    }
    cp_async_commit();
  };

  if (n_chunks > 0) plan(0);
  if (n_chunks > 1) plan(1);
  __syncthreads();
  if (n_chunks > 0) issue(0, 0);
  // queries of the group as a 16-row tile (rows >= G zero)
  for (int i = tid; i < 16 * (D / 8); i += 128) {
    const int row = i / (D / 8), piece = i % (D / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < G) v = *reinterpret_cast<const uint4*>(q + (size_t)b * q_stride + ((size_t)h * G + row) * D + piece * 8);
    *reinterpret_cast<uint4*>(dsm + 2 * Cfg::STAGE_BYTES + row * STRIDE + piece * 16) = v;
  }
  __syncthreads();
  uint32_t qa[KS][4];
  {
    const int mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
      ldsm_x4(sq_addr + ((mat & 1) * 8 + r) * STRIDE + (ks * 16 + (mat >> 1) * 8) * 2, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};     // rows gq and gq + 8

  for (int c = 0; c < n_chunks; ++c) {
    const int stage = c & 1;
    if (c + 1 < n_chunks) {
      issue(c + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (c + 2 < n_chunks) plan(c + 2);      // table slot (c & 1) is free: chunk c's copies have been issued from it
    const uint32_t ks_addr = smem0 + stage * Cfg::STAGE_BYTES + (warp * 16) * STRIDE;   // this warp's 16 tokens
    const uint32_t vs_addr = ks_addr + Cfg::OPERAND_BYTES;
    const int mat = lane >> 3, r = lane & 7;
    // ---- S[16 heads, 16 tokens] = Q K^T
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b0, b1, b2, b3;   // tokens 0-7: dims lo / hi; tokens 8-15: dims lo / hi
      ldsm_x4(ks_addr + ((mat >> 1) * 8 + r) * STRIDE + (ks * 16 + (mat & 1) * 8) * 2, b0, b1, b2, b3);
      mma_bf16_16816(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      mma_bf16_16816(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
    }
    // ---- mask, running max per row over this warp's tokens
    const int tok = t0 + c * DEC_CHUNK + warp * 16 + 2 * tq;
    const bool v00 = tok < t1, v01 = tok + 1 < t1, v10 = tok + 8 < t1, v11 = tok + 9 < t1;
    s0[0] = v00 ? s0[0] * sl2 : -INFINITY; s0[1] = v01 ? s0[1] * sl2 : -INFINITY;
    s0[2] = v00 ? s0[2] * sl2 : -INFINITY; s0[3] = v01 ? s0[3] * sl2 : -INFINITY;
    s1[0] = v10 ? s1[0] * sl2 : -INFINITY; s1[1] = v11 ? s1[1] * sl2 : -INFINITY;
    s1[2] = v10 ? s1[2] * sl2 : -INFINITY; s1[3] = v11 ? s1[3] * sl2 : -INFINITY;
    float alpha[2];
    uint32_t pa[4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {           // hh = 0: row gq (elements 0, 1); 1: row gq + 8 (elements 2, 3)
      float mx = fmaxf(fmaxf(s0[2 * hh], s0[2 * hh + 1]), fmaxf(s1[2 * hh], s1[2 * hh + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(m_run[hh], mx);
      const float mref = (mn == -INFINITY) ? 0.f : mn;
      alpha[hh] = fast_exp2(m_run[hh] - mref);
      m_run[hh] = mn;
      const float p00 = fast_exp2(s0[2 * hh] - mref), p01 = fast_exp2(s0[2 * hh + 1] - mref);
      const float p10 = fast_exp2(s1[2 * hh] - mref), p11 = fast_exp2(s1[2 * hh + 1] - mref);
      l_run[hh] = l_run[hh] * alpha[hh] + (p00 + p01 + p10 + p11);   // this thread's columns; summed over the quad at the end
      pa[hh] = pack_bf16(p00, p01);            // A fragment: tokens 0-7
      pa[2 + hh] = pack_bf16(p10, p11);        //             tokens 8-15
    }
    // ---- O[16 heads, D] = O * alpha + P V
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }
#pragma unroll
    for (int jj = 0; jj < KS; ++jj) {          // 16 output dims per step
      uint32_t b0, b1, b2, b3;   // dims lo: tokens 0-7 / 8-15; dims hi: tokens 0-7 / 8-15
      ldsm_x4_trans(vs_addr + ((mat & 1) * 8 + r) * STRIDE + (jj * 16 + (mat >> 1) * 8) * 2, b0, b1, b2, b3);
      mma_bf16_16816(o[2 * jj], pa[0], pa[1], pa[2], pa[3], b0, b1);
      mma_bf16_16816(o[2 * jj + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
    }
    __syncthreads();   // every warp is done with this stage before the next copies land in it
  }

  // ---- merge the four warps (stage memory is free now): mo [4][16][D], mm / ml [4][16]
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
  float* mo = reinterpret_cast<float*>(dsm);
  float* mm = mo + 4 * 16 * D;
  float* ml = mm + 4 * 16;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int col = j * 8 + 2 * tq;
    *reinterpret_cast<float2*>(mo + ((warp * 16 + gq) * D + col)) = make_float2(o[j][0], o[j][1]);
    *reinterpret_cast<float2*>(mo + ((warp * 16 + gq + 8) * D + col)) = make_float2(o[j][2], o[j][3]);
  }
  if (tq == 0) {
    mm[warp * 16 + gq] = m_run[0]; mm[warp * 16 + gq + 8] = m_run[1];
    ml[warp * 16 + gq] = l_run[0]; ml[warp * 16 + gq + 8] = l_run[1];
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i - g * D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mm[w * 16 + g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mm[w * 16 + g];
      const float wt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mx);
      ll += ml[w * 16 + g] * wt;
      oo += mo[(w * 16 + g) * D + d] * wt;
    }
    const size_t pidx = ((size_t)b * Hq + (size_t)h * G + g) * num_splits + spl;
    part_o[pidx * D + d] = oo;
    if (d == 0) {
      part_ml[pidx * 2] = mx;
      part_ml[pidx * 2 + 1] = ll;
    }
  }
}

template <int D>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int num_splits);

template <int D>
static int launch_decode_mma(const void* q, const void* kc, const void* vc, const int* pt, const int* lens,
                             float* part_o, float* part_ml, void* out, int B, int Hq, int Hkv, int page_size,
                             int max_pages, int splits, float scale, long long q_stride, cudaStream_t s) {
  using Cfg = DecodeMmaCfg<D>;
  static_assert(2 * Cfg::STAGE_BYTES >= (4 * 16 * D + 8 * 16) * 4, "the merge buffers alias the stage memory");
  dim3 grid(B, Hkv, splits);
  auto kern = paged_decode_mma_kernel<D>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, dev_state, &num_sms)) return 2;
  (void)num_sms;
  launch_pdl(kern, grid, dim3(128), (size_t)Cfg::SMEM_BYTES, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, pt, lens,
             part_o, part_ml, Hq, Hkv, Hq / Hkv, page_size, max_pages, splits, scale, q_stride);
  launch_pdl(decode_combine_kernel<D>, dim3(B * Hq), dim3(D), 0, s, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, splits);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

template <int D, int G>
constexpr int decode_smem_bytes() {
  return 2 * (2 * DEC_CHUNK * D * 2) + (G * D + DEC_CHUNK * G) * 4;
}

// out[b, hq, :] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
template <int D>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int num_splits) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;  // b * Hq + hq
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(row * num_splits + s) * 2]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(row * num_splits + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
    L += part_ml[(row * num_splits + s) * 2 + 1] * w;
    acc += part_o[(row * num_splits + s) * D + d] * w;
  }
  out[row * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
}

// ------------------------------------------------------------------ sampling
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float uniform01(uint32_t seed, uint32_t row, uint32_t idx, uint32_t step) {
  uint32_t h = mix32(seed ^ 0x9e3779b9U);
  h = mix32(h ^ (row * 0x85ebca6bU + 0x165667b1U));
  h = mix32(h ^ (step * 0xc2b2ae35U + 0x27d4eb2fU));
  h = mix32(h ^ idx);
  return ((h >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
}

struct SampleState {
  float m, s;      // online max / sum-exp of z
  float best;      // best perturbed score
  int best_idx;
  float best_z;
};
__device__ __forceinline__ void sample_merge(SampleState& a, const SampleState& b) {
  const float mm = fmaxf(a.m, b.m);
  const float ra = (a.m == -INFINITY) ? 0.f : __expf(a.m - mm);
  const float rb = (b.m == -INFINITY) ? 0.f : __expf(b.m - mm);
  a.s = a.s * ra + b.s * rb;
  a.m = mm;
  if (b.best > a.best || (b.best == a.best && b.best_idx < a.best_idx && b.best_idx >= 0)) {
    a.best = b.best; a.best_idx = b.best_idx; a.best_z = b.best_z;
  }
}

// One CTA per row. z = logits * inv_temp[row]; token = argmax(z + Gumbel) (argmax z when
// greedy[row]); logprob = z_token - logsumexp(z). Per-row temperature / seed / greedy flags.
__global__ void sample_kernel(const float* __restrict__ logits, long long ld, int V,
                              const float* __restrict__ inv_temp, const int* __restrict__ greedy,
                              const unsigned int* __restrict__ seeds, unsigned int step,
                              int* __restrict__ out_tok, float* __restrict__ out_logp) {
  __shared__ SampleState red[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const float it = inv_temp[row];
  const bool gr = greedy[row] != 0;
  const uint32_t seed = seeds[row];
  const float* z = logits + (size_t)row * ld;
  SampleState st;
  st.m = -INFINITY; st.s = 0.f; st.best = -INFINITY; st.best_idx = -1; st.best_z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float zi = z[i] * it;
    if (zi > st.m) { st.s = st.s * __expf(st.m - zi) + 1.f; st.m = zi; } else { st.s += __expf(zi - st.m); }
    float score = zi;
    if (!gr) {
      const float u = uniform01(seed, (uint32_t)row, (uint32_t)i, step);
      score = zi - __logf(-__logf(u));
    }
    if (score > st.best) { st.best = score; st.best_idx = i; st.best_z = zi; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    SampleState y;
    y.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    y.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    y.best = __shfl_xor_sync(0xffffffffu, st.best, o);
    y.best_idx = __shfl_xor_sync(0xffffffffu, st.best_idx, o);
    y.best_z = __shfl_xor_sync(0xffffffffu, st.best_z, o);
    sample_merge(st, y);
  }
  const int w = threadIdx.x >> 5, ln = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (ln == 0) red[w] = st;
  __syncthreads();
  if (w == 0) {
    SampleState t;
    t.m = -INFINITY; t.s = 0.f; t.best = -INFINITY; t.best_idx = -1; t.best_z = 0.f;
    if (ln < nw) t = red[ln];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      SampleState y;
      y.m = __shfl_xor_sync(0xffffffffu, t.m, o);
      y.s = __shfl_xor_sync(0xffffffffu, t.s, o);
      y.best = __shfl_xor_sync(0xffffffffu, t.best, o);
      y.best_idx = __shfl_xor_sync(0xffffffffu, t.best_idx, o);
      y.best_z = __shfl_xor_sync(0xffffffffu, t.best_z, o);
      sample_merge(t, y);
    }
    if (ln == 0) {
      out_tok[row] = t.best_idx;
      out_logp[row] = t.best_z - (t.m + __logf(t.s));
    }
  }
}

template <int D, int G>
static int launch_decode(const void* q, const void* kc, const void* vc, const int* pt, const int* lens,
                         float* part_o, float* part_ml, void* out, int B, int Hq, int Hkv, int page_size,
                         int max_pages, int splits, float scale, long long q_stride, cudaStream_t s) {
  dim3 grid(B, Hkv, splits);
  constexpr int SMEM = decode_smem_bytes<D, G>();
  static_assert(SMEM >= (4 * G * D + 8 * G) * 4, "the merge buffers alias the stage memory");
  auto kern = paged_decode_kernel<D, G>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, SMEM, dev_state, &num_sms)) return 2;
  (void)num_sms;
  kern<<<grid, 128, SMEM, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, pt, lens, part_o, part_ml,
                               Hq, Hkv, page_size, max_pages, splits, scale, q_stride);
  decode_combine_kernel<D><<<B * Hq, D, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, splits);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

}  // namespace ab2

extern "C" {
using namespace ab2;

int ab2_kv_append(const void* k, const void* v, void* kc, void* vc, const int* slots, int n, int Hkv, int D,
                  long long k_stride, long long v_stride, void* stream) {
  if (n <= 0) return 0;
  const int row = Hkv * D;
  if (row % 8) return 10;
  long long work = (long long)n * (row / 8);
  int grid = (int)((work + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  launch_pdl(kv_append_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                           (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, slots, n, row,
                                                           k_stride, v_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// Workspace sizes (floats) for ab2_paged_decode: part_o = B*Hq*splits*D, part_ml = B*Hq*splits*2.
// q_stride: elements between consecutive rows of q (Hq * D when q is dense; larger when q is the query part
// of a fused [q | k] buffer). out is dense [B, Hq, D].
int ab2_paged_decode_strided(const void* q, const void* kc, const void* vc, const int* page_table, const int* seq_lens,
                             float* part_o, float* part_ml, void* out, int B, int Hq, int Hkv, int D, int page_size,
                             int max_pages, int num_splits, float scale, long long q_stride, void* stream) {
  if (B <= 0) return 0;
  if (Hq % Hkv || num_splits < 1 || (q_stride & 7)) return 10;
  const int G = Hq / Hkv;
  cudaStream_t s = (cudaStream_t)stream;
  // tensor-core form for every group size up to 16; AB2_DECODE_SIMT=1 selects the scalar form
  static const bool simt = [] { const char* e = getenv("AB2_DECODE_SIMT"); return e && e[0] == '1'; }();
  if (!simt && G <= 16 && (D == 64 || D == 128)) {
    if (D == 128) return launch_decode_mma<128>(q, kc, vc, page_table, seq_lens, part_o, part_ml, out, B, Hq, Hkv, page_size, max_pages, num_splits, scale, q_stride, s);
    return launch_decode_mma<64>(q, kc, vc, page_table, seq_lens, part_o, part_ml, out, B, Hq, Hkv, page_size, max_pages, num_splits, scale, q_stride, s);
  }
#define AB2_DEC(DD, GG)                                                                                   \
  if (D == DD && G == GG)                                                                                 \
    return launch_decode<DD, GG>(q, kc, vc, page_table, seq_lens, part_o, part_ml, out, B, Hq, Hkv,       \
                                 page_size, max_pages, num_splits, scale, q_stride, s);
  AB2_DEC(128, 1) AB2_DEC(128, 2) AB2_DEC(128, 4) AB2_DEC(128, 6) AB2_DEC(128, 8)
  AB2_DEC(64, 1) AB2_DEC(64, 2) AB2_DEC(64, 4) AB2_DEC(64, 8)
#undef AB2_DEC
  return 11;
}

int ab2_paged_decode(const void* q, const void* kc, const void* vc, const int* page_table, const int* seq_lens,
                     float* part_o, float* part_ml, void* out, int B, int Hq, int Hkv, int D, int page_size,
                     int max_pages, int num_splits, float scale, void* stream) {
  return ab2_paged_decode_strided(q, kc, vc, page_table, seq_lens, part_o, part_ml, out, B, Hq, Hkv, D, page_size, max_pages,
                                  num_splits, scale, (long long)Hq * D, stream);
}

int ab2_sample(const float* logits, long long ld, int B, int V, const float* inv_temp, const int* greedy,
               const unsigned int* seeds, unsigned int step, int* out_tok, float* out_logp, void* stream) {
  if (B <= 0) return 0;
  launch_pdl(sample_kernel, dim3(B), dim3(1024), 0, (cudaStream_t)stream, logits, ld, V, inv_temp, greedy, seeds, step, out_tok, out_logp);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}

// ------------------------------------------------------------------ allocation-free variant
// Workspace of ab2_paged_decode_noalloc(): partial outputs first, then the (max, sum) pairs.
// In host code this name is only a stand-in for the symbol, not a device address; the address
// each device uses is resolved with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[AB2_NOALLOC_MAX_ROWS * (128 + 2)];

static float* g_noalloc_ptr[64] = {nullptr};
static std::mutex g_noalloc_mu;

// Resolves (once per device, with that device current) where the built-in workspace lives.
static float* noalloc_workspace() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch) != cudaSuccess) return nullptr;
    g_noalloc_ptr[dev] = p;
  }
  return g_noalloc_ptr[dev];
}

extern "C" int ab2_paged_decode_noalloc(const void* q, const void* kc, const void* vc, const int* page_table,
                                        const int* seq_lens, void* out, int B, int Hq, int Hkv, int D,
                                        int page_size, int max_pages, int num_splits, float scale, void* stream) {
  if (B <= 0) return 0;
  if (num_splits < 1 || Hkv <= 0 || Hq % Hkv) return 10;
  const long long rows = (long long)B * Hq * num_splits;
  if (rows > AB2_NOALLOC_MAX_ROWS || D > 128) return 20;  // beyond the built-in workspace
  float* ws = noalloc_workspace();
  if (!ws) return 21;
  float* part_o = ws;
  float* part_ml = ws + (size_t)AB2_NOALLOC_MAX_ROWS * 128;
  return ab2_paged_decode(q, kc, vc, page_table, seq_lens, part_o, part_ml, out, B, Hq, Hkv, D, page_size,
                          max_pages, num_splits, scale, stream);
}
