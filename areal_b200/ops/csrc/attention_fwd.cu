// Variable-length (packed) causal / full flash-attention forward for sm_100a.
//
// One CTA handles a 128-query tile of one head. Per 128-key block:
//   S = Q K^T      tcgen05.mma, both operands K-major from TMA-filled swizzled smem, S in TMEM
//   softmax        4 warps, one query row per thread, reads S with tcgen05.ld, online max/sum,
//                  writes P (bf16) into swizzled smem, rescales O in TMEM when the max moved
//   O += P V       tcgen05.mma, P K-major from smem, V MN-major ([kv, d] row-major) from smem
// S is double-buffered in TMEM so the next block's QK^T overlaps this block's softmax.
// CTA = 192 threads: warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2..5 softmax.
//
// Replaces the FlashAttention-2 varlen call behind
// areal/experimental/models/archon/attention/varlen.py and the HF flash-attn integration
// used by areal/engine/fsdp_engine.py; also serves prefill in the rollout engine.
#include "common.cuh"

namespace ab2 {

static constexpr int QT = 128;   // query rows per CTA
static constexpr int KT = 128;   // keys per block
static constexpr int CHUNK_BYTES = 128 * 128;  // 128 rows x 128 B (one swizzled 64-column chunk)

template <int HD>
struct AttnCfg {
  static constexpr int DCH = HD / 64;                 // 64-wide chunks of the head dim
  static constexpr int Q_BYTES = DCH * CHUNK_BYTES;
  static constexpr int KV_BYTES = DCH * CHUNK_BYTES;  // K tile and V tile have the same size
  static constexpr int P_BYTES = 2 * CHUNK_BYTES;
  static constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;               // S0 | S1 | O
  static constexpr int S_COL0 = 0, S_COL1 = 128, O_COL = 256;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ O,
                float* __restrict__ LSE, const int* __restrict__ cu_seqlens,
                const int* __restrict__ tile_info, int T, int Hq, int Hkv, long long o_stride_t,
                float scale, int causal, int* err) {
  using Cfg = AttnCfg<HD>;
  const int tile = blockIdx.x;
  const int seq = tile_info[2 * tile];
  if (seq < 0) return;  // padding entry of the tile table (uniform for the CTA)
  const int qb = tile_info[2 * tile + 1];
  const int head = blockIdx.y;
  const int kvh = head / (Hq / Hkv);
  const int seq_start = cu_seqlens[seq];
  const int seq_len = cu_seqlens[seq + 1] - seq_start;
  const int q_row0 = seq_start + qb * QT;
  const int nkv_total = (seq_len + KT - 1) / KT;
  const int nkv = causal ? min(qb + 1, nkv_total) : nkv_total;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sK0 = sQ + Cfg::Q_BYTES;
  const uint32_t sV0 = sK0 + 2 * Cfg::KV_BYTES;
  const uint32_t sP = sV0 + 2 * Cfg::KV_BYTES;
  const uint32_t bar = sP + Cfg::P_BYTES;
  const uint32_t q_full = bar;
  auto k_full = [&](int s) { return bar + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar + 8u * (3 + s); };
  auto kv_empty = [&](int s) { return bar + 8u * (5 + s); };
  auto s_full = [&](int b) { return bar + 8u * (7 + b); };
  const uint32_t p_ready = bar + 8u * 9;
  const uint32_t o_ready = bar + 8u * 10;
  const uint32_t tmem_slot = bar + 8u * 11;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(kv_empty(s), 1);
      mbar_init(s_full(s), 1);
    }
    mbar_init(p_ready, 128);
    mbar_init(o_ready, 1);
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
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::DCH; ++c)
        tma_load_2d(sQ + c * CHUNK_BYTES, &tmQ, q_full, head * HD + c * 64, q_row0);
      for (int j = 0; j < nkv; ++j) {
        const int s = j & 1;
        const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
        if (!mbar_wait(kv_empty(s), ph ^ 1u, err, ERR_WAIT_EMPTY)) break;
        const int kv_row0 = seq_start + j * KT;
        mbar_expect_tx(k_full(s), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::DCH; ++c)
          tma_load_2d(sK0 + s * Cfg::KV_BYTES + c * CHUNK_BYTES, &tmK, k_full(s), kvh * HD + c * 64, kv_row0);
        mbar_expect_tx(v_full(s), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::DCH; ++c)
          tma_load_2d(sV0 + s * Cfg::KV_BYTES + c * CHUNK_BYTES, &tmV, v_full(s), kvh * HD + c * 64, kv_row0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc(QT, KT, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(QT, HD, 1, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, err, ERR_WAIT_FULL);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t d = tmem_base + (s ? Cfg::S_COL1 : Cfg::S_COL0);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = make_smem_desc_sw128(sQ + (kk >> 2) * CHUNK_BYTES, 16, 1024) + (uint64_t)((kk & 3) * 2);
          const uint64_t bd = make_smem_desc_sw128(sK0 + s * Cfg::KV_BYTES + (kk >> 2) * CHUNK_BYTES, 16, 1024) +
                              (uint64_t)((kk & 3) * 2);
          umma_f16(d, ad, bd, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full(s));
      };
      if (ok && nkv > 0) {
        ok = mbar_wait(k_full(0), 0, err, ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
      }
      for (int j = 0; j < nkv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
        if (j + 1 < nkv) {
          const int s1 = (j + 1) & 1;
          const uint32_t ph1 = static_cast<uint32_t>((j + 1) >> 1) & 1u;
          if (!mbar_wait(k_full(s1), ph1, err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(p_ready, static_cast<uint32_t>(j) & 1u, err, ERR_WAIT_MISC)) { ok = false; break; }
        if (!mbar_wait(v_full(s), ph, err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + Cfg::O_COL;
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint64_t ad = make_smem_desc_sw128(sP + (kk >> 2) * CHUNK_BYTES, 16, 1024) + (uint64_t)((kk & 3) * 2);
          const uint64_t bd = make_smem_desc_sw128(sV0 + s * Cfg::KV_BYTES, CHUNK_BYTES, 1024) +
                              (uint64_t)(kk * (16 * 128 >> 4));
          umma_f16(d, ad, bd, idesc_o, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(kv_empty(s));
        umma_commit(o_ready);
      }
    }
  } else {
    // ------------------------------------------------ softmax + epilogue (warps 2..5)
    const int q = warp & 3;
    const int row = q * 32 + lane;         // row inside the tile == TMEM lane
    const int q_local = qb * QT + row;     // position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const float sl2 = scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int sb = j & 1;
      const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
      if (!mbar_wait(s_full(sb), ph, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_s = tmem_base + lane_off + (sb ? Cfg::S_COL1 : Cfg::S_COL0);
      const int kv0 = j * KT;
      const bool edge = (kv0 + KT > seq_len) || (causal && (kv0 + KT - 1 > qb * QT));
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < KT / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_s + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]);
          if (edge) {
            const int kv = kv0 + c * 32 + i;
            if (kv >= seq_len || (causal && kv > q_local)) v = -INFINITY;
          }
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m_run, mx * sl2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use);
      // P smem (and O) may only be touched once the previous PV has retired.
      if (j > 0) {
        if (!mbar_wait(o_ready, static_cast<uint32_t>(j - 1) & 1u, err, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
      }
      // pass 2: probabilities -> bf16 P in swizzled smem, row sum
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < KT / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_s + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float v0 = __uint_as_float(r[2 * i]), v1 = __uint_as_float(r[2 * i + 1]);
          float p0 = fast_exp2(v0 * sl2 - m_use), p1 = fast_exp2(v1 * sl2 - m_use);
          if (edge) {
            const int kv = kv0 + c * 32 + 2 * i;
            if (kv >= seq_len || (causal && kv > q_local)) p0 = 0.f;
            if (kv + 1 >= seq_len || (causal && kv + 1 > q_local)) p1 = 0.f;
          }
          sum += p0 + p1;
          pk[i] = pack_bf16(p0, p1);
        }
        // columns [c*32, c*32+32) of row `row`: chunk = c/2, 16-byte units u0..u0+3
        const uint32_t chunk_base = sP + (c >> 1) * CHUNK_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
        const int u0 = (c & 1) * 4;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t addr = chunk_base + (((u0 + u) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * u]),
                       "r"(pk[4 * u + 1]), "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3])
                       : "memory");
        }
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      // rescale O when any row of this warp moved its maximum
      if (j > 0) {
        const bool need = __any_sync(0xffffffffu, alpha != 1.f);
        if (need) {
          const uint32_t t_o = tmem_base + lane_off + Cfg::O_COL;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(t_o + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(t_o + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    // ---- epilogue: O / l -> global, log-sum-exp
    if (ok && nkv > 0) {
      if (mbar_wait(o_ready, static_cast<uint32_t>(nkv - 1) & 1u, err, ERR_WAIT_MISC)) {
        tc_fence_after();
        const bool valid = q_local < seq_len;
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        const uint32_t t_o = tmem_base + lane_off + Cfg::O_COL;
        __nv_bfloat16* out = O + (size_t)(q_row0 + row) * o_stride_t + (size_t)head * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_o + c * 32, r);
          tmem_ld_wait();
          if (valid) {
            uint4* o4 = reinterpret_cast<uint4*>(out + c * 32);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[8 * u]) * inv_l, __uint_as_float(r[8 * u + 1]) * inv_l);
              v.y = pack_bf16(__uint_as_float(r[8 * u + 2]) * inv_l, __uint_as_float(r[8 * u + 3]) * inv_l);
              v.z = pack_bf16(__uint_as_float(r[8 * u + 4]) * inv_l, __uint_as_float(r[8 * u + 5]) * inv_l);
              v.w = pack_bf16(__uint_as_float(r[8 * u + 6]) * inv_l, __uint_as_float(r[8 * u + 7]) * inv_l);
              o4[u] = v;
            }
          }
        }
        if (valid && LSE) LSE[(size_t)head * T + q_row0 + row] = (m_run + log2f(l_run)) * 0.6931471805599453f;
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

template <int HD>
static int launch_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                           const int* cu_seqlens, const int* tile_info, int num_tiles, int T, int Hq,
                           int Hkv, long long q_stride, long long k_stride, long long v_stride,
                           long long o_stride, float scale, int causal, cudaStream_t stream) {
  using Cfg = AttnCfg<HD>;
  CUtensorMap tq, tk, tv;
  if (ab2host::encode_tmap_2d(&tq, q, 2, (uint64_t)Hq * HD, (uint64_t)T, (uint64_t)q_stride * 2, 64, QT, true, 0)) return 100;
  if (ab2host::encode_tmap_2d(&tk, k, 2, (uint64_t)Hkv * HD, (uint64_t)T, (uint64_t)k_stride * 2, 64, KT, true, 0)) return 101;
  if (ab2host::encode_tmap_2d(&tv, v, 2, (uint64_t)Hkv * HD, (uint64_t)T, (uint64_t)v_stride * 2, 64, KT, true, 0)) return 102;
  auto kern = attn_fwd_kernel<HD>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, dev_state, &num_sms)) return 300;
  (void)num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  dim3 grid(num_tiles, Hq);
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, (__nv_bfloat16*)o, lse, cu_seqlens, tile_info, T,
                                               Hq, Hkv, o_stride, scale, causal, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

}  // namespace ab2

extern "C" {
// Packed varlen attention forward.
//   q: [T, Hq, D], k/v: [T, Hkv, D] bf16; *_stride = elements between consecutive tokens
//   (so q/k/v may be slices of one fused projection output). o: [T, Hq, D] with o_stride.
//   lse: [Hq, T] fp32 (natural log) or null. cu_seqlens: [B+1] int32 on device.
//   tile_info: [num_tiles, 2] int32 on device = (sequence index or -1, query block index).
//   D in {64, 128}. Strides must be multiples of 8 elements, pointers 16-byte aligned.
int ab2_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens,
                 const int* tile_info, int num_tiles, int T, int Hq, int Hkv, int D, long long q_stride,
                 long long k_stride, long long v_stride, long long o_stride, float scale, int causal,
                 void* stream) {
  if (num_tiles <= 0 || T <= 0) return 0;
  if (Hq % Hkv) return 10;
  if ((q_stride | k_stride | v_stride | o_stride) & 7) return 11;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 128)
    return ab2::launch_attn_fwd<128>(q, k, v, o, lse, cu_seqlens, tile_info, num_tiles, T, Hq, Hkv, q_stride,
                                     k_stride, v_stride, o_stride, scale, causal, s);
  if (D == 64)
    return ab2::launch_attn_fwd<64>(q, k, v, o, lse, cu_seqlens, tile_info, num_tiles, T, Hq, Hkv, q_stride,
                                    k_stride, v_stride, o_stride, scale, causal, s);
  return 12;
}
}
