// Variable-length (packed) causal / full flash-attention backward for sm_100a.
//
// One CTA owns a 128-key block of one KV head and walks every query block (of every query
// head of the GQA group) that attends to it, so dK and dV accumulate in TMEM for the whole
// kernel and are written once, without atomics. Per query block:
//   S  = Q K^T, dP = dO V^T          tcgen05.mma into TMEM (two 128-column accumulators)
//   P  = exp(S*scale - lse)          4 warps, one query row per thread (tcgen05.ld)
//   dS = P * (dP - delta) * scale    written with P as bf16 into swizzled shared memory
//   dV += P^T dO, dK += dS^T Q       P / dS consumed as MN-major A operands (no transpose copy)
//   dQ  = dS K                       into the (now free) S accumulator, then added to the
//                                    fp32 dQ buffer in global memory with vector reductions
// TMEM: S | dP | dV | dK = 512 columns at head dim 128. Shared memory: K, V resident, one Q and
// one dO tile, P and dS tiles (192 KB at head dim 128).
// CTA = 192 threads: warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2..5 compute.
//
// Replaces the FlashAttention-2 backward reached through
// areal/experimental/models/archon/attention/varlen.py (aten._flash_attention_backward).
#include "common.cuh"

namespace ab2 {

static constexpr int BQ = 128;
static constexpr int BKV = 128;
static constexpr int CHUNK = 128 * 128;  // bytes of one 64-column swizzled chunk with 128 rows

template <int HD>
struct BwdCfg {
  static constexpr int DCH = HD / 64;
  static constexpr int TILE = DCH * CHUNK;          // a [128, HD] bf16 tile
  static constexpr int PS = 2 * CHUNK;              // a [128, 128] bf16 tile (P or dS)
  static constexpr int SMEM_BYTES = 4 * TILE + 2 * PS + 1024 + 256;
  static constexpr int S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + HD;
  static constexpr int TMEM_COLS = 512;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int T, int Hq, int D, long long o_stride,
                                  long long do_stride) {
  const int warps_per_block = blockDim.x >> 5;
  const long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);  // t * Hq + h
  if (row >= (long long)T * Hq) return;
  const int t = (int)(row / Hq), h = (int)(row - (long long)t * Hq);
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* op = o + (size_t)t * o_stride + (size_t)h * D;
  const __nv_bfloat16* dp = dout + (size_t)t * do_stride + (size_t)h * D;
  float acc = 0.f;
  for (int e = lane * 2; e < D; e += 64) {
    const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(op + e));
    const float2 b = unpack_bf16(*reinterpret_cast<const uint32_t*>(dp + e));
    acc += a.x * b.x + a.y * b.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[(size_t)h * T + t] = acc;
}

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const float* __restrict__ LSE, const float* __restrict__ DELTA, float* __restrict__ dQ,
                __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dV, const int* __restrict__ cu_seqlens,
                const int* __restrict__ tile_info, int T, int Hq, int Hkv, long long dk_stride, long long dv_stride,
                float scale, int causal, int* err) {
  using Cfg = BwdCfg<HD>;
  const int tile = blockIdx.x;
  const int seq = tile_info[2 * tile];
  if (seq < 0) return;
  const int jb = tile_info[2 * tile + 1];  // key block inside the sequence
  const int kvh = blockIdx.y;
  const int G = Hq / Hkv;
  const int seq_start = cu_seqlens[seq];
  const int seq_len = cu_seqlens[seq + 1] - seq_start;
  const int kv_row0 = seq_start + jb * BKV;
  const int nq_total = (seq_len + BQ - 1) / BQ;
  const int i_first = causal ? jb : 0;
  const int n_i = nq_total - i_first;      // query blocks per head
  const int n_iter = n_i * G;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = sK + Cfg::TILE, sQ = sV + Cfg::TILE, sDO = sQ + Cfg::TILE;
  const uint32_t sP = sDO + Cfg::TILE, sDS = sP + Cfg::PS;
  const uint32_t bar = sDS + Cfg::PS;
  const uint32_t kv_full = bar, qdo_full = bar + 8, qdo_free = bar + 16, s_full = bar + 24;
  const uint32_t pds_ready = bar + 32, dq_full = bar + 40, s_free = bar + 48, tmem_slot = bar + 56;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_free, 1);
    mbar_init(s_full, 1);
    mbar_init(pds_ready, 128);
    mbar_init(dq_full, 1);
    mbar_init(s_free, 128);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * Cfg::TILE);
#pragma unroll
      for (int c = 0; c < Cfg::DCH; ++c) {
        tma_load_2d(sK + c * CHUNK, &tmK, kv_full, kvh * HD + c * 64, kv_row0);
        tma_load_2d(sV + c * CHUNK, &tmV, kv_full, kvh * HD + c * 64, kv_row0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int g = it / n_i, i = i_first + (it - g * n_i);
        const int hq = kvh * G + g;
        if (!mbar_wait(qdo_free, (static_cast<uint32_t>(it) & 1u) ^ 1u, err, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(qdo_full, 2 * Cfg::TILE);
        const int q_row0 = seq_start + i * BQ;
#pragma unroll
        for (int c = 0; c < Cfg::DCH; ++c) {
          tma_load_2d(sQ + c * CHUNK, &tmQ, qdo_full, hq * HD + c * 64, q_row0);
          tma_load_2d(sDO + c * CHUNK, &tmDO, qdo_full, hq * HD + c * 64, q_row0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t id_kk = make_idesc(128, 128, 1, 1, 0, 0);   // S, dP: both K-major
      constexpr uint32_t id_mm = make_idesc(128, HD, 1, 1, 1, 1);    // dV, dK: both MN-major
      constexpr uint32_t id_km = make_idesc(128, HD, 1, 1, 0, 1);    // dQ: A K-major, B MN-major
      bool ok = mbar_wait(kv_full, 0, err, ERR_WAIT_FULL);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = static_cast<uint32_t>(it) & 1u;
        if (!mbar_wait(qdo_full, ph, err, ERR_WAIT_FULL)) { ok = false; break; }
        if (!mbar_wait(s_free, ph ^ 1u, err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        // S = Q K^T ; dP = dO V^T   (reduction over the head dim)
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t co = (kk >> 2) * CHUNK;
          const uint64_t off = (uint64_t)((kk & 3) * 2);
          umma_f16(tmem_base + Cfg::S_COL, make_smem_desc_sw128(sQ + co, 16, 1024) + off,
                   make_smem_desc_sw128(sK + co, 16, 1024) + off, id_kk, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t co = (kk >> 2) * CHUNK;
          const uint64_t off = (uint64_t)((kk & 3) * 2);
          umma_f16(tmem_base + Cfg::DP_COL, make_smem_desc_sw128(sDO + co, 16, 1024) + off,
                   make_smem_desc_sw128(sV + co, 16, 1024) + off, id_kk, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(pds_ready, ph, err, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q   (reduction over the 128 query rows, 16 per step)
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint64_t off = (uint64_t)(kk * (16 * 128 >> 4));
          umma_f16(tmem_base + Cfg::DV_COL, make_smem_desc_sw128(sP, CHUNK, 1024) + off,
                   make_smem_desc_sw128(sDO, CHUNK, 1024) + off, id_mm, (it | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint64_t off = (uint64_t)(kk * (16 * 128 >> 4));
          umma_f16(tmem_base + Cfg::DK_COL, make_smem_desc_sw128(sDS, CHUNK, 1024) + off,
                   make_smem_desc_sw128(sQ, CHUNK, 1024) + off, id_mm, (it | kk) != 0 ? 1u : 0u);
        }
        umma_commit(qdo_free);
        // dQ = dS K   (reduction over the 128 keys) into the S accumulator
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t aoff = (uint64_t)((kk & 3) * 2);
          const uint64_t boff = (uint64_t)(kk * (16 * 128 >> 4));
          umma_f16(tmem_base + Cfg::S_COL, make_smem_desc_sw128(sDS + (kk >> 2) * CHUNK, 16, 1024) + aoff,
                   make_smem_desc_sw128(sK, CHUNK, 1024) + boff, id_km, kk != 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
      }
    }
  } else {
    // ------------------------------------------------ compute warps (2..5)
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const float sl2 = scale * 1.4426950408889634f;
    const uint32_t row_off = (row >> 3) * 1024 + (row & 7) * 128;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t ph = static_cast<uint32_t>(it) & 1u;
      const int g = it / n_i, i = i_first + (it - g * n_i);
      const int hq = kvh * G + g;
      const int q_local = i * BQ + row;
      const bool q_valid = q_local < seq_len;
      const size_t vec_idx = (size_t)hq * T + seq_start + q_local;
      const float lse2 = q_valid ? LSE[vec_idx] * 1.4426950408889634f : 0.f;
      const float dlt = q_valid ? DELTA[vec_idx] : 0.f;
      if (!mbar_wait(s_full, ph, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const bool diag = causal && (i == jb);
      const bool tail = (jb * BKV + BKV > seq_len);
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t s[32], dp[32];
        tmem_ld32(tmem_base + lane_off + Cfg::S_COL + c * 32, s);
        tmem_ld32(tmem_base + lane_off + Cfg::DP_COL + c * 32, dp);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float p0 = fast_exp2(__uint_as_float(s[2 * e]) * sl2 - lse2);
          float p1 = fast_exp2(__uint_as_float(s[2 * e + 1]) * sl2 - lse2);
          const int kv = jb * BKV + c * 32 + 2 * e;
          if (!q_valid || (tail && kv >= seq_len) || (diag && kv > q_local)) p0 = 0.f;
          if (!q_valid || (tail && kv + 1 >= seq_len) || (diag && kv + 1 > q_local)) p1 = 0.f;
          const float d0 = p0 * (__uint_as_float(dp[2 * e]) - dlt) * scale;
          const float d1 = p1 * (__uint_as_float(dp[2 * e + 1]) - dlt) * scale;
          pp[e] = pack_bf16(p0, p1);
          dd[e] = pack_bf16(d0, d1);
        }
        const uint32_t cb = (c >> 1) * CHUNK + row_off;
        const int u0 = (c & 1) * 4;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t sw = static_cast<uint32_t>((u0 + u) ^ (row & 7)) << 4;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sP + cb + sw), "r"(pp[4 * u]),
                       "r"(pp[4 * u + 1]), "r"(pp[4 * u + 2]), "r"(pp[4 * u + 3]) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sDS + cb + sw), "r"(dd[4 * u]),
                       "r"(dd[4 * u + 1]), "r"(dd[4 * u + 2]), "r"(dd[4 * u + 3]) : "memory");
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_ready);
      // dQ block -> global fp32 accumulation
      if (!mbar_wait(dq_full, ph, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = dQ + ((size_t)(seq_start + q_local) * Hq + hq) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_off + Cfg::S_COL + c * 32, r);
        tmem_ld_wait();
        if (q_valid) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            red_add_v4(dq_row + c * 32 + 4 * e, __uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                       __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
        }
      }
      tc_fence_before();
      mbar_arrive(s_free);
    }
    // ---- epilogue: dK, dV rows of this key block (the last dq_full covers every earlier MMA)
    if (ok) {
      const int kv_local = jb * BKV + row;
      const bool kv_valid = kv_local < seq_len;
      __nv_bfloat16* dk_row = dK + (size_t)(kv_row0 + row) * dk_stride + (size_t)kvh * HD;
      __nv_bfloat16* dv_row = dV + (size_t)(kv_row0 + row) * dv_stride + (size_t)kvh * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t a[32], b[32];
        if (n_iter > 0) {
          tmem_ld32(tmem_base + lane_off + Cfg::DK_COL + c * 32, a);
          tmem_ld32(tmem_base + lane_off + Cfg::DV_COL + c * 32, b);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) { a[e] = 0u; b[e] = 0u; }
        }
        if (kv_valid) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 x, y;
            x.x = pack_bf16(__uint_as_float(a[8 * u]), __uint_as_float(a[8 * u + 1]));
            x.y = pack_bf16(__uint_as_float(a[8 * u + 2]), __uint_as_float(a[8 * u + 3]));
            x.z = pack_bf16(__uint_as_float(a[8 * u + 4]), __uint_as_float(a[8 * u + 5]));
            x.w = pack_bf16(__uint_as_float(a[8 * u + 6]), __uint_as_float(a[8 * u + 7]));
            y.x = pack_bf16(__uint_as_float(b[8 * u]), __uint_as_float(b[8 * u + 1]));
            y.y = pack_bf16(__uint_as_float(b[8 * u + 2]), __uint_as_float(b[8 * u + 3]));
            y.z = pack_bf16(__uint_as_float(b[8 * u + 4]), __uint_as_float(b[8 * u + 5]));
            y.w = pack_bf16(__uint_as_float(b[8 * u + 6]), __uint_as_float(b[8 * u + 7]));
            reinterpret_cast<uint4*>(dk_row + c * 32)[u] = x;
            reinterpret_cast<uint4*>(dv_row + c * 32)[u] = y;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab2

namespace ab2 {

template <int HD>
static int launch_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                           const float* delta, float* dq, void* dk, void* dv, const int* cu_seqlens,
                           const int* tile_info, int num_tiles, int T, int Hq, int Hkv, long long q_stride,
                           long long k_stride, long long v_stride, long long do_stride, long long dk_stride,
                           long long dv_stride, float scale, int causal, cudaStream_t stream) {
  using Cfg = BwdCfg<HD>;
  CUtensorMap tq, tk, tv, tdo;
  if (ab2host::encode_tmap_2d(&tq, q, 2, (uint64_t)Hq * HD, (uint64_t)T, (uint64_t)q_stride * 2, 64, BQ, true, 0)) return 100;
  if (ab2host::encode_tmap_2d(&tk, k, 2, (uint64_t)Hkv * HD, (uint64_t)T, (uint64_t)k_stride * 2, 64, BKV, true, 0)) return 101;
  if (ab2host::encode_tmap_2d(&tv, v, 2, (uint64_t)Hkv * HD, (uint64_t)T, (uint64_t)v_stride * 2, 64, BKV, true, 0)) return 102;
  if (ab2host::encode_tmap_2d(&tdo, dout, 2, (uint64_t)Hq * HD, (uint64_t)T, (uint64_t)do_stride * 2, 64, BQ, true, 0)) return 103;
  auto kern = attn_bwd_kernel<HD>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, dev_state, &num_sms)) return 300;
  (void)num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  dim3 grid(num_tiles, Hkv);
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, lse, delta, dq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv,
                                               cu_seqlens, tile_info, T, Hq, Hkv, dk_stride, dv_stride, scale, causal, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

}  // namespace ab2

extern "C" {
// delta[Hq, T] = rowsum(dO * O); o / dout: [T, Hq, D] bf16 with the given token strides.
int ab2_attn_delta(const void* o, const void* dout, float* delta, int T, int Hq, int D, long long o_stride,
                   long long do_stride, void* stream) {
  if (T <= 0) return 0;
  const long long rows = (long long)T * Hq;
  const int wpb = 8;
  ab2::attn_delta_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, T, Hq, D, o_stride, do_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// Packed varlen attention backward. q/dout: [T, Hq, D], k/v: [T, Hkv, D] bf16 (token strides
// given); lse, delta: [Hq, T] fp32; dq: [T, Hq, D] fp32, must be zero on entry (accumulated
// with reductions); dk, dv: [T, Hkv, D] bf16 (fully overwritten for valid tokens).
// tile_info: [num_tiles, 2] (sequence | -1, key block) on device. D in {64, 128}.
int ab2_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                 float* dq, void* dk, void* dv, const int* cu_seqlens, const int* tile_info, int num_tiles, int T,
                 int Hq, int Hkv, int D, long long q_stride, long long k_stride, long long v_stride,
                 long long do_stride, long long dk_stride, long long dv_stride, float scale, int causal, void* stream) {
  if (num_tiles <= 0 || T <= 0) return 0;
  if (Hq % Hkv) return 10;
  if ((q_stride | k_stride | v_stride | do_stride | dk_stride | dv_stride) & 7) return 11;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 128)
    return ab2::launch_attn_bwd<128>(q, k, v, dout, lse, delta, dq, dk, dv, cu_seqlens, tile_info, num_tiles, T, Hq,
                                     Hkv, q_stride, k_stride, v_stride, do_stride, dk_stride, dv_stride, scale, causal, s);
  if (D == 64)
    return ab2::launch_attn_bwd<64>(q, k, v, dout, lse, delta, dq, dk, dv, cu_seqlens, tile_info, num_tiles, T, Hq,
                                    Hkv, q_stride, k_stride, v_stride, do_stride, dk_stride, dv_stride, scale, causal, s);
  return 12;
}
}
