// Decode-shaped GEMM ("skinny": at most 256 tokens against a large weight matrix):
//
//   Y[M_tok, N_out] = X[M_tok, K] * W[N_out, K]^T (+ R)
//
// The product is bound by streaming W from HBM once, so the kernel is laid out around that
// stream instead of around the output: W tiles (128 output features x 64 K) are the M-side
// operand of tcgen05.mma, the few tokens are the N-side operand (swap-AB), the accumulator
// D[128 features, tokens] lives in TMEM, and K is split across CTAs so that even a
// 4096 x 4096 projection keeps ~200 CTAs pulling on HBM at once.
//
// Split-K partial sums are reduced in L2 with `red.global.add.f32` into a zeroed fp32
// workspace; the CTA that arrives last at a tile (arrival counter, no waiting anywhere)
// converts the tile to the output type, adds the residual, and re-zeroes workspace and
// counter for the next launch. With split_k == 1 the epilogue stores directly.
//
// CTA layout (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5
// epilogue. One output tile and one K range per CTA; shared memory is kept under ~100 KB so
// two CTAs share an SM.
//
// Takes the place of the cuBLAS/cuBLASLt GEMV-like calls inside the reference's inference
// servers (SGLang / vLLM decode path; areal/engine/sglang_remote.py drives them remotely).
#include "common.cuh"

namespace ab2 {

static constexpr int SK_BM = 128;  // output features per tile (MMA M)
static constexpr int SK_BK = 64;
static constexpr int SK_UMMA_K = 16;

template <int MT>
struct SkinnyCfg {
  static constexpr int A_BYTES = SK_BM * SK_BK * 2;
  static constexpr int B_BYTES = MT * SK_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // up to 128 tokens: <= 98 KB so two CTAs share an SM; 256 tokens: one CTA with 4 stages
  static constexpr int STAGES_RAW = (MT > 128 ? 196 * 1024 : 98 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);
  static constexpr int TMEM_COLS = MT < 32 ? 32 : MT;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 128;
};

template <int MT>
__global__ void __launch_bounds__(192, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   void* __restrict__ Yptr, const __nv_bfloat16* __restrict__ Rptr,
                   float* __restrict__ ws, int* __restrict__ counters, int M_tok, int N_out, int K,
                   int ldy, int out_f32, int split_k, int kb_per_split, int* err) {
  using Cfg = SkinnyCfg<MT>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_last;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x;
  const int split = blockIdx.y;
  const int n0 = tile_n * SK_BM;
  const int num_kb_total = (K + SK_BK - 1) / SK_BK;
  const int kb0 = split * kb_per_split;
  const int kb1 = min(num_kb_total, kb0 + kb_per_split);
  const int num_kb = kb1 - kb0;  // >= 1 by construction of the grid

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmX);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    fence_mbar_init();
    s_last = 0;
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
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, err, ERR_WAIT_EMPTY)) { ok = false; break; }
        const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sB = sA + Cfg::A_BYTES;
        mbar_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
        tma_load_2d(sA, &tmW, full_bar(stage), kb * SK_BK, n0);
        tma_load_2d(sB, &tmX, full_bar(stage), kb * SK_BK, 0);
        ++issued;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) {
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) { /* bounded grace for copies in flight */ }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(SK_BM, MT, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sB = sA + Cfg::A_BYTES;
        const uint64_t adesc = make_smem_desc_sw128(sA, 16, 1024);
        const uint64_t bdesc = make_smem_desc_sw128(sB, 16, 1024);
#pragma unroll
        for (int k = 0; k < SK_BK / SK_UMMA_K; ++k)
          umma_f16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(empty_bar(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
    }
  } else {
    // epilogue: thread <-> one output feature (TMEM lane), loop over token columns
    const int q = warp & 3;
    const int n = n0 + q * 32 + lane;
    if (mbar_wait(tfull_bar, 0u, err, ERR_WAIT_TMEM_FULL)) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < MT / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        if (n < N_out) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = c * 32 + j;
            if (tok < M_tok) {
              const float v = __uint_as_float(r[j]);
              if (split_k > 1) {
                atomicAdd(ws + (size_t)tok * N_out + n, v);  // result unused -> red.global.add.f32
              } else if (out_f32) {
                reinterpret_cast<float*>(Yptr)[(size_t)tok * ldy + n] =
                    v + (Rptr ? __bfloat162float(Rptr[(size_t)tok * ldy + n]) : 0.f);
              } else {
                reinterpret_cast<__nv_bfloat16*>(Yptr)[(size_t)tok * ldy + n] =
                    __float2bfloat16(v + (Rptr ? __bfloat162float(Rptr[(size_t)tok * ldy + n]) : 0.f));
              }
            }
          }
        }
      }
      if (split_k > 1) __threadfence();  // partial sums visible before this CTA is counted
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (split_k > 1) {
    if (threadIdx.x == 0) {
      const int old = atomicAdd(counters + tile_n, 1);
      s_last = (old == split_k - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      const int rows = min(SK_BM, N_out - n0);
      const bool vec_ok = rows == SK_BM && (N_out & 3) == 0 && (ldy & 3) == 0;
      if (vec_ok) {
        // 4 features per thread and 4 independent loads in flight: the tile sits in L2 and
        // this loop would otherwise pay one L2 round trip per element
        const int items = M_tok * (SK_BM / 4);
        for (int base = threadIdx.x; base < items; base += blockDim.x * 4) {
          float4 v[4];
          int idxs[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            idxs[u] = base + u * blockDim.x;
            if (idxs[u] < items) {
              const int tok = idxs[u] / (SK_BM / 4);
              const int nn = (idxs[u] - tok * (SK_BM / 4)) * 4;
              v[u] = __ldcg(reinterpret_cast<const float4*>(ws + (size_t)tok * N_out + n0 + nn));
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (idxs[u] < items) {
              const int tok = idxs[u] / (SK_BM / 4);
              const int nn = (idxs[u] - tok * (SK_BM / 4)) * 4;
              __stcg(reinterpret_cast<float4*>(ws + (size_t)tok * N_out + n0 + nn), make_float4(0.f, 0.f, 0.f, 0.f));
              const size_t o = (size_t)tok * ldy + n0 + nn;
              float4 a = v[u];
              if (Rptr) {
                const uint2 rr = *reinterpret_cast<const uint2*>(Rptr + o);
                const float2 r0 = unpack_bf16(rr.x), r1 = unpack_bf16(rr.y);
                a.x += r0.x; a.y += r0.y; a.z += r1.x; a.w += r1.y;
              }
              if (out_f32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(Yptr) + o) = a;
              else *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(Yptr) + o) =
                  make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
            }
          }
        }
      } else {
        for (int idx = threadIdx.x; idx < M_tok * SK_BM; idx += blockDim.x) {
          const int tok = idx / SK_BM;
          const int nn = idx - tok * SK_BM;
          if (nn < rows) {
            float* p = ws + (size_t)tok * N_out + n0 + nn;
            float v = __ldcg(p);
            __stcg(p, 0.f);
            const size_t o = (size_t)tok * ldy + n0 + nn;
            if (Rptr) v += __bfloat162float(Rptr[o]);
            if (out_f32) reinterpret_cast<float*>(Yptr)[o] = v;
            else reinterpret_cast<__nv_bfloat16*>(Yptr)[o] = __float2bfloat16(v);
          }
        }
      }
      if (threadIdx.x == 0) counters[tile_n] = 0;
    }
  }
}

template <int MT>
static int launch_skinny(const void* X, const void* W, void* Y, const void* R, float* ws, int* counters,
                         int M_tok, int N_out, int K, int ldx, int ldw, int ldy, int out_f32, int split_k,
                         cudaStream_t stream) {
  using Cfg = SkinnyCfg<MT>;
  CUtensorMap tmW, tmX;
  int rc = ab2host::encode_tmap_2d(&tmW, W, 2, (uint64_t)K, (uint64_t)N_out, (uint64_t)ldw * 2, SK_BK, SK_BM, true, 0);
  if (rc) return 100 + rc;
  rc = ab2host::encode_tmap_2d(&tmX, X, 2, (uint64_t)K, (uint64_t)M_tok, (uint64_t)ldx * 2, SK_BK, MT, true, 0);
  if (rc) return 200 + rc;
  auto kern = gemm_skinny_kernel<MT>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, dev_state, &num_sms)) return 300;
  (void)num_sms;
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  const int kb_per = (num_kb + split_k - 1) / split_k;
  const int splits = (num_kb + kb_per - 1) / kb_per;  // every launched split owns >= 1 k-block
  int* err = ab2host::error_flag();
  if (!err) return 301;
  dim3 grid((N_out + SK_BM - 1) / SK_BM, splits);
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tmW, tmX, Y, reinterpret_cast<const __nv_bfloat16*>(R), ws, counters,
                                               M_tok, N_out, K, ldy, out_f32, splits, kb_per, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

}  // namespace ab2

extern "C" {

// Y[M_tok, N_out] = X[M_tok, K] W[N_out, K]^T (+ R), bf16 inputs, fp32 accumulation, for
// M_tok <= 256. `ws` (fp32, at least M_tok * N_out, all zero) and `counters` (int32, at least
// ceil(N_out / 128), all zero) are only touched when split_k != 1 and are left zeroed again.
// split_k = 0 chooses a split that gives at least ~1.25 CTAs per SM. out_f32 selects the type
// of Y; R (optional, bf16) has Y's layout. Overlapping launches must not share ws/counters.
int ab2_gemm_skinny(const void* X, const void* W, void* Y, const void* R, void* ws, void* counters, int M_tok,
                    int N_out, int K, int ldx, int ldw, int ldy, int out_f32, int split_k, void* stream) {
  using namespace ab2;
  if (M_tok <= 0 || N_out <= 0 || K <= 0) return 0;
  if (M_tok > 256) return 20;
  if ((ldx & 7) || (ldw & 7)) return 10;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15) return 11;
  const int tiles = (N_out + SK_BM - 1) / SK_BM;
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  int num_sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (split_k <= 0) {
    split_k = 1;
    while (tiles * split_k * 4 < num_sms * 5 && split_k < 16 && num_kb / (split_k * 2) >= 4) split_k *= 2;
  }
  if (split_k > num_kb) split_k = num_kb;
  if (split_k > 1 && (!ws || !counters)) return 12;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* w = reinterpret_cast<float*>(ws);
  int* c = reinterpret_cast<int*>(counters);
  if (M_tok <= 32) return launch_skinny<32>(X, W, Y, R, w, c, M_tok, N_out, K, ldx, ldw, ldy, out_f32, split_k, s);
  if (M_tok <= 64) return launch_skinny<64>(X, W, Y, R, w, c, M_tok, N_out, K, ldx, ldw, ldy, out_f32, split_k, s);
  if (M_tok <= 128) return launch_skinny<128>(X, W, Y, R, w, c, M_tok, N_out, K, ldx, ldw, ldy, out_f32, split_k, s);
  return launch_skinny<256>(X, W, Y, R, w, c, M_tok, N_out, K, ldx, ldw, ldy, out_f32, split_k, s);
}
}
