// FP8 (e4m3) GEMM on tcgen05 tensor cores with fp32 accumulation, plus the quantisation kernels
// that produce its operands.
//
//   C[M, N] = (A[M, K] * B[N, K]^T) with scales, both operands K-major, one byte per element.
//
// Two scaling schemes:
//   * row-wise: one fp32 scale per row of A and per row of B; the whole K range accumulates in
//     tensor memory and the epilogue multiplies by sa[m] * sb[n];
//   * block-wise (the DeepSeek-V3 recipe the reference's fp8 paths follow): A carries a scale per
//     (row, 128-wide K block), B per (128 x 128) block. Each K block accumulates into its own
//     tensor-memory buffer (two buffers, ping-pong), and the epilogue warps promote it into fp32
//     registers with the block's scale product while the tensor cores work on the next block.
//
// Pipeline (one CTA per SM, persistent over output tiles): warp 0 = TMA producer, warp 1 = MMA
// issuer (one elected thread, kind::f8f6f4, 128 x 128 x 32 per instruction), warps 2..5 =
// epilogue. Every wait is bounded and reports through the kernel error word.
//
// Takes the place of the Triton fp8 cast / dequant kernels and the DeepGEMM / torchao block-wise
// GEMMs the reference reaches through areal/engine/megatron_utils/fp8/ and
// areal/experimental/models/archon/fp8.py.
#include <cuda_fp8.h>

#include "common.cuh"

namespace ab2 {

static constexpr int F8_BM = 128;
static constexpr int F8_BK = 128;      // one 128-byte swizzle row of fp8
static constexpr int F8_UMMA_K = 32;
static constexpr int F8_A_BYTES = F8_BM * F8_BK;

// BN = 128 for the block-wise recipe (the weight scale blocks are 128 wide and the promoted
// accumulators live in registers); 256 for row-wise scales, where a wider tile halves the
// shared-memory traffic per flop.
template <int BN>
struct F8Cfg {
  static constexpr int B_BYTES = BN * F8_BK;
  static constexpr int STAGE_BYTES = F8_A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;
};

// sa: row-wise: [M]; block-wise: [ceil(K / 128)][M] (K-block major, so a warp reads consecutive rows).
// sb: row-wise: [N]; block-wise: [ceil(N / 128)][ceil(K / 128)].
template <bool BLOCK_SCALED, int F8_BN>
__global__ void __launch_bounds__(192, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cptr,
                const float* __restrict__ sa, const float* __restrict__ sb, int M, int N, int K, int ldc, int out_f32, int* err) {
  using Cfg = F8Cfg<F8_BN>;
  constexpr int F8_STAGES = Cfg::STAGES;
  constexpr int F8_STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr int F8_TMEM_COLS = Cfg::TMEM_COLS;
  static_assert(!BLOCK_SCALED || F8_BN == 128, "block-wise scales: one weight scale block per tile column");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + F8_STAGES * F8_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (F8_STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * F8_STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * F8_STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * F8_STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (M + F8_BM - 1) / F8_BM;
  const int n_blocks = (N + F8_BN - 1) / F8_BN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (K + F8_BK - 1) / F8_BK;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 128);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, F8_TMEM_COLS);
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
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mb = tile % m_blocks, nb = tile / m_blocks;   // consecutive CTAs share a B panel
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * F8_STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), F8_STAGE_BYTES);
          tma_load_2d(sA, &tmA, full_bar(stage), kb * F8_BK, mb * F8_BM);
          tma_load_2d(sA + F8_A_BYTES, &tmB, full_bar(stage), kb * F8_BK, nb * F8_BN);
          ++issued;
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const int pending = issued < F8_STAGES ? issued : F8_STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) { /* ~1 ms per stage for copies in flight */ }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(F8_BM, F8_BN, 0, 0, 0, 0);   // e4m3 x e4m3, both K-major
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t nbuf = 0;       // accumulator buffers handed out so far (block-wise: one per K block; else one per tile)
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          const bool fresh = BLOCK_SCALED || kb == 0;
          const int buf = (int)(nbuf & 1u);
          if (fresh) {
            if (!mbar_wait(tempty_bar(buf), ((nbuf >> 1) & 1u) ^ 1u, err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
            tc_fence_after();
          }
          const uint32_t d_tmem = tmem_base + buf * F8_BN;
          if (!mbar_wait(full_bar(stage), phase, err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * F8_STAGE_BYTES;
          const uint64_t adesc = make_smem_desc_sw128(sA, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sA + F8_A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < F8_BK / F8_UMMA_K; ++k)   // +32 bytes per 32 K-elements inside the swizzled row
            umma_f8(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (fresh && k == 0) ? 0u : 1u);
          umma_commit(empty_bar(stage));
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1u; }
          if (BLOCK_SCALED || kb == num_kb - 1) {
            umma_commit(tfull_bar(buf));
            ++nbuf;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    bool ok = true;
    uint32_t nbuf = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int mb = tile % m_blocks, nb = tile / m_blocks;
      const int m0 = mb * F8_BM, n0 = nb * F8_BN;
      const int row = m0 + row_in_tile;
      const bool row_ok = row < M;
      if constexpr (BLOCK_SCALED) {
        float acc[F8_BN];
#pragma unroll
        for (int j = 0; j < F8_BN; ++j) acc[j] = 0.f;
        for (int kb = 0; kb < num_kb; ++kb, ++nbuf) {
          const int buf = (int)(nbuf & 1u);
          const float s = (row_ok ? sa[(size_t)kb * M + row] : 0.f) * sb[(size_t)nb * num_kb + kb];
          if (!mbar_wait(tfull_bar(buf), (nbuf >> 1) & 1u, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * F8_BN;
#pragma unroll
          for (int c = 0; c < F8_BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(t_row + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(s, __uint_as_float(r[j]), acc[c * 32 + j]);
          }
          tc_fence_before();
          mbar_arrive(tempty_bar(buf));
        }
        if (ok && row_ok) {
#pragma unroll
          for (int c = 0; c < F8_BN / 8; ++c) {
            const int col = n0 + c * 8;
            if (col + 8 <= N) {
              if (out_f32) {
                float4* C4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(Cptr) + (size_t)row * ldc + col);
                C4[0] = make_float4(acc[c * 8], acc[c * 8 + 1], acc[c * 8 + 2], acc[c * 8 + 3]);
                C4[1] = make_float4(acc[c * 8 + 4], acc[c * 8 + 5], acc[c * 8 + 6], acc[c * 8 + 7]);
              } else {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(Cptr) + (size_t)row * ldc + col) =
                    make_uint4(pack_bf16(acc[c * 8], acc[c * 8 + 1]), pack_bf16(acc[c * 8 + 2], acc[c * 8 + 3]),
                               pack_bf16(acc[c * 8 + 4], acc[c * 8 + 5]), pack_bf16(acc[c * 8 + 6], acc[c * 8 + 7]));
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (col + j < N) {
                  if (out_f32) reinterpret_cast<float*>(Cptr)[(size_t)row * ldc + col + j] = acc[c * 8 + j];
                  else reinterpret_cast<__nv_bfloat16*>(Cptr)[(size_t)row * ldc + col + j] = __float2bfloat16(acc[c * 8 + j]);
                }
              }
            }
          }
        }
      } else {
        const int buf = (int)(nbuf & 1u);
        if (!mbar_wait(tfull_bar(buf), (nbuf >> 1) & 1u, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const float sr = row_ok ? sa[row] : 0.f;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * F8_BN;
#pragma unroll 1
        for (int c = 0; c < F8_BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              if (col + j + 1 < N) {
                const float2 sc = *reinterpret_cast<const float2*>(sb + col + j);   // N is even (checked by the host)
                const float v0 = __uint_as_float(r[j]) * sr * sc.x, v1 = __uint_as_float(r[j + 1]) * sr * sc.y;
                if (out_f32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(Cptr) + (size_t)row * ldc + col + j) = make_float2(v0, v1);
                else *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(Cptr) + (size_t)row * ldc + col + j) = pack_bf16(v0, v1);
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(tempty_bar(buf));
        ++nbuf;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, F8_TMEM_COLS);
  }
}

template <bool BLOCK_SCALED, int F8_BN>
static int launch_fp8(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N, int K, int lda, int ldb,
                      int ldc, int out_f32, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc = ab2host::encode_tmap_2d(&tmA, A, 1, (uint64_t)K, (uint64_t)M, (uint64_t)lda, F8_BK, F8_BM, true, 2);
  if (rc) return 100 + rc;
  rc = ab2host::encode_tmap_2d(&tmB, B, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, F8_BK, F8_BN, true, 2);
  if (rc) return 200 + rc;
  using Cfg = F8Cfg<F8_BN>;
  constexpr int F8_SMEM_BYTES = Cfg::SMEM_BYTES;
  auto kern = gemm_fp8_kernel<BLOCK_SCALED, F8_BN>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, F8_SMEM_BYTES, dev_state, &num_sms)) return 300;
  (void)num_sms;
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  kern<<<grid, 192, F8_SMEM_BYTES, stream>>>(tmA, tmB, C, sa, sb, M, N, K, ldc, out_f32, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

// ------------------------------------------------------------------ quantisation
__device__ __forceinline__ float fp8_scale_of(float amax, int pow2) {
  float s = fmaxf(amax, 1e-12f) / 448.f;          // 448 = largest finite e4m3 value
  if (pow2) s = exp2f(ceilf(log2f(s)));           // power-of-two scales (UE8M0-representable)
  return s;
}
__device__ __forceinline__ uint32_t pack_fp8x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// One warp per (row, 128-wide K block); BLOCK = false: one warp per row with a single scale.
// x: [M, K] bf16 (ldx elements per row); out: [M, K] fp8 (ldo bytes per row).
// scales: BLOCK: [ceil(K / 128)][M]; else [M].
template <bool BLOCK>
__global__ void __launch_bounds__(256)
quant_fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out, float* __restrict__ scales, int M, int K,
                      long long ldx, long long ldo, int pow2) {
  const int lane = threadIdx.x & 31;
  const long long w0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nw = (long long)gridDim.x * (blockDim.x >> 5);
  const int kblocks = (K + 127) / 128;
  if constexpr (BLOCK) {
    for (long long w = w0; w < (long long)M * kblocks; w += nw) {
      const int row = (int)(w / kblocks), kb = (int)(w - (long long)row * kblocks);
      const int k0 = kb * 128 + lane * 4;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (k0 + 4 <= K) {
        const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)row * ldx + k0);
        const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
      } else {
        for (int j = 0; j < 4; ++j) if (k0 + j < K) v[j] = __bfloat162float(x[(size_t)row * ldx + k0 + j]);
      }
      const float amax = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
      const float s = fp8_scale_of(amax, pow2), inv = 1.f / s;
      if (lane == 0) scales[(size_t)kb * M + row] = s;
      if (k0 + 4 <= K) {
        *reinterpret_cast<uint32_t*>(out + (size_t)row * ldo + k0) = pack_fp8x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
      } else {
        for (int j = 0; j < 4; ++j)
          if (k0 + j < K) out[(size_t)row * ldo + k0 + j] = (uint8_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3);
      }
    }
  } else {
    for (long long row = w0; row < M; row += nw) {
      const __nv_bfloat16* xr = x + (size_t)row * ldx;
      float amax = 0.f;
      for (int k = lane * 4; k < K; k += 128) {
        if (k + 4 <= K) {
          const uint2 raw = *reinterpret_cast<const uint2*>(xr + k);
          const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y);
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
        } else {
          for (int j = 0; k + j < K; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(xr[k + j])));
        }
      }
      amax = warp_max(amax);
      const float s = fp8_scale_of(amax, pow2), inv = 1.f / s;
      if (lane == 0) scales[row] = s;
      uint8_t* orow = out + (size_t)row * ldo;
      for (int k = lane * 4; k < K; k += 128) {
        if (k + 4 <= K) {
          const uint2 raw = *reinterpret_cast<const uint2*>(xr + k);
          const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y);
          *reinterpret_cast<uint32_t*>(orow + k) = pack_fp8x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
        } else {
          for (int j = 0; k + j < K; ++j) orow[k + j] = (uint8_t)__nv_cvt_float_to_fp8(__bfloat162float(xr[k + j]) * inv, __NV_SATFINITE, __NV_E4M3);
        }
      }
    }
  }
}

// One CTA (256 threads) per 128 x 128 block of w [N, K]: scales [ceil(N / 128)][ceil(K / 128)].
__global__ void __launch_bounds__(256)
quant_fp8_block128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ out, float* __restrict__ scales, int N, int K,
                          long long ldw, long long ldo, int pow2) {
  __shared__ float red[8];
  const int kblocks = (K + 127) / 128;
  const int nb = blockIdx.x / kblocks, kb = blockIdx.x % kblocks;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k0 = kb * 128 + lane * 4;
  float amax = 0.f;
  for (int r = warp; r < 128; r += 8) {
    const int row = nb * 128 + r;
    if (row >= N) break;
    for (int j = 0; j < 4; ++j)
      if (k0 + j < K) amax = fmaxf(amax, fabsf(__bfloat162float(w[(size_t)row * ldw + k0 + j])));
  }
  amax = warp_max(amax);
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = fp8_scale_of(amax, pow2), inv = 1.f / s;
  if (threadIdx.x == 0) scales[(size_t)nb * kblocks + kb] = s;
  for (int r = warp; r < 128; r += 8) {
    const int row = nb * 128 + r;
    if (row >= N) break;
    if (k0 + 4 <= K) {
      const uint2 raw = *reinterpret_cast<const uint2*>(w + (size_t)row * ldw + k0);
      const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y);
      *reinterpret_cast<uint32_t*>(out + (size_t)row * ldo + k0) = pack_fp8x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
    } else {
      for (int j = 0; j < 4; ++j)
        if (k0 + j < K) out[(size_t)row * ldo + k0 + j] = (uint8_t)__nv_cvt_float_to_fp8(__bfloat162float(w[(size_t)row * ldw + k0 + j]) * inv, __NV_SATFINITE, __NV_E4M3);
    }
  }
}

}  // namespace ab2

extern "C" {

// C[M, N] = A[M, K] * B[N, K]^T with e4m3 operands (one byte per element, K-major; lda / ldb in
// elements, multiples of 16; pointers 16-byte aligned) and fp32 accumulation.
//   block_scaled = 0: sa [M], sb [N] (row-wise scales; N must be even)
//   block_scaled = 1: sa [ceil(K/128)][M], sb [ceil(N/128)][ceil(K/128)]
//   out_f32 = 0: C is bf16 (ldc multiple of 8); 1: C is fp32 (ldc multiple of 4)
int ab2_gemm_fp8(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N, int K, int lda, int ldb,
                 int ldc, int block_scaled, int out_f32, void* stream) {
  using namespace ab2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 15) || (ldb & 15) || (ldc & (out_f32 ? 3 : 7)) || (N & 1)) return 10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return 11;
  if (!sa || !sb) return 12;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (block_scaled) return launch_fp8<true, 128>(A, B, C, sa, sb, M, N, K, lda, ldb, ldc, out_f32, s);
  // wide tiles when they still fill the machine
  const long long tiles256 = (long long)((M + F8_BM - 1) / F8_BM) * ((N + 255) / 256);
  if (N % 256 == 0 && tiles256 >= 120) return launch_fp8<false, 256>(A, B, C, sa, sb, M, N, K, lda, ldb, ldc, out_f32, s);
  return launch_fp8<false, 128>(A, B, C, sa, sb, M, N, K, lda, ldb, ldc, out_f32, s);
}

// x [rows, K] bf16 -> e4m3 + scales. mode 0: one scale per row ([rows]); mode 1: one per (row,
// 128-wide K block) ([ceil(K/128)][rows]); mode 2: one per 128 x 128 block ([ceil(rows/128)][ceil(K/128)]).
// pow2 != 0 rounds every scale up to a power of two. ldx in elements (multiple of 4), ldo in bytes (multiple of 4).
int ab2_quant_fp8(const void* x, void* out, float* scales, int rows, int K, long long ldx, long long ldo, int mode, int pow2, void* stream) {
  using namespace ab2;
  if (rows <= 0 || K <= 0) return 0;
  if ((ldx & 3) || (ldo & 3)) return 10;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int kblocks = (K + 127) / 128;
  if (mode == 2) {
    const int blocks = ((rows + 127) / 128) * kblocks;
    quant_fp8_block128_kernel<<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)out, scales, rows, K, ldx, ldo, pow2);
  } else {
    const long long work = mode == 1 ? (long long)rows * kblocks : rows;
    long long want = (work + 7) / 8;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    if (mode == 1)
      quant_fp8_rows_kernel<true><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)out, scales, rows, K, ldx, ldo, pow2);
    else
      quant_fp8_rows_kernel<false><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)out, scales, rows, K, ldx, ldo, pow2);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
}
