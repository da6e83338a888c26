// Dense bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by TMA into 128B-swizzled shared memory, persistent over output tiles.
//
//   C[M,N] (+)= A * B      A given K-major ([M,K] row-major) or MN-major ([K,M] row-major)
//                          B given K-major ([N,K] row-major, the nn.Linear weight layout)
//                            or MN-major ([K,N] row-major)
//
// which covers forward (x @ W^T), input-gradient (dy @ W) and weight-gradient (dy^T @ x,
// accumulated in fp32) of a linear layer without any explicit transpose.
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane)
// and TMEM owner, warps 2..5 = epilogue (TMEM -> registers -> global). Two TMEM accumulator
// buffers let the epilogue of tile i overlap the main loop of tile i+1.
//
// Replaces the cuBLAS calls behind every linear layer of the reference
// (areal/experimental/models/archon/qwen3/model/model.py, HF modules in
// areal/engine/fsdp_engine.py).
#include <stdio.h>

#include "common.cuh"

namespace ab2 {

static constexpr int BM = 128;
static constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
static constexpr int UMMA_K = 16;

enum Epilogue : int {
  EPI_BF16 = 0,       // C = bf16(acc)
  EPI_F32 = 1,        // C = acc
  EPI_F32_ACC = 2,    // C += acc                (fp32 gradient accumulation)
  EPI_BF16_RESID = 3, // C = bf16(acc + R)       (residual add fused)
  EPI_BF16_BCAST = 4  // bf16(acc) stored into the same place of SEVERAL buffers (this GPU's and its
                      // peers'), then a release-add on each buffer's arrival counter: the product is
                      // handed to every tensor-parallel rank from inside the epilogue
};

// Destinations of EPI_BF16_BCAST: `n` buffers with C's shape and ldc (peer-mapped symmetric memory)
// and one 64-bit arrival counter per buffer. Every epilogue warp adds, per tile, the number of
// (row, 32-column chunk) pieces it stored, so one product adds M * ceil(N / 32) to each counter
// whatever the tile shape.
static constexpr int BCAST_MAX = 8;
struct BcastArgs {
  void* dst[BCAST_MAX];
  unsigned long long* counter[BCAST_MAX];
  int n;
};

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int& mb, int& nb) {
  // Groups of 16 M-blocks sweep all N-blocks together so the CTAs that run concurrently
  // share B tiles (and a small set of A tiles) in L2.
  constexpr int GROUP = 16;
  const int per_group = GROUP * n_blocks;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(GROUP, m_blocks - first_m);
  const int in_g = tile - g * per_group;
  mb = first_m + in_g % gsize;
  nb = in_g / gsize;
}

// SPLITK: the K range is cut into `splits` pieces of `kb_per` k-blocks; a tile index also selects
// the piece, and piece ks stores its fp32 partial product at Cptr + ks * M * ldc (the caller sums
// the pieces). Used for decode-shaped products whose output alone has too few tiles to keep the
// machine's load pipes busy.
template <int BN, bool A_MN, bool B_MN, bool SPLITK = false>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 void* __restrict__ Cptr, const __nv_bfloat16* __restrict__ Rptr, int M, int N,
                 int K, int ldc, const int EPI, int* err, int splits, int kb_per, const BcastArgs bc) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  // barrier map (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem slot
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (M + BM - 1) / BM;
  const int n_blocks = (N + BN - 1) / BN;
  const int mn_tiles = m_blocks * n_blocks;
  const int num_tiles = SPLITK ? mn_tiles * splits : mn_tiles;
  const int num_kb_all = (K + BK - 1) / BK;
  // k-block range of a tile: everything, or piece ks of the split
  auto kb_begin = [&](int tile) { return SPLITK ? (tile / mn_tiles) * kb_per : 0; };
  auto kb_end = [&](int tile) { return SPLITK ? min(num_kb_all, (tile / mn_tiles + 1) * kb_per) : num_kb_all; };

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    for (int s = 0; s < STAGES; ++s) {
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
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  // barriers, tensor memory and descriptors are set up: from here on the kernel touches what the
  // previous kernel of the stream may still be producing
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(SPLITK ? tile % mn_tiles : tile, m_blocks, n_blocks, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = kb_begin(tile); kb < kb_end(tile); ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, full_bar(stage), kb * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sA + c * (BK * 128), &tmA, full_bar(stage), m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, full_bar(stage), kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * (BK * 128), &tmB, full_bar(stage), n0 + c * 64, kb * BK);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies already in flight a bounded chance to land before the CTA retires.
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) { /* ~1 ms per stage */ }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const int kb0 = kb_begin(tile);
        for (int kb = kb0; kb < kb_end(tile); ++kb) {
          if (!mbar_wait(full_bar(stage), phase, err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint64_t adesc = make_smem_desc_sw128(sA, A_MN ? BK * 128 : 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sB, B_MN ? BK * 128 : 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: +32 B per 16 K-elements inside the swizzled row.
            // MN-major: +16 K-rows of 128 B.
            const uint64_t ad = adesc + (A_MN ? (uint64_t)(k * (UMMA_K * 128 >> 4)) : (uint64_t)(k * 2));
            const uint64_t bd = bdesc + (B_MN ? (uint64_t)(k * (UMMA_K * 128 >> 4)) : (uint64_t)(k * 2));
            umma_f16(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    // ------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int row_in_tile = q * 32 + lane;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int mb, nb;
      tile_coords(SPLITK ? tile % mn_tiles : tile, m_blocks, n_blocks, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      void* Cptr_t = SPLITK ? static_cast<void*>(reinterpret_cast<float*>(Cptr) + (size_t)(tile / mn_tiles) * M * ldc) : Cptr;
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), use & 1u, err, ERR_WAIT_TMEM_FULL));   // the warp leaves together
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      int pieces = 0;   // EPI_BF16_BCAST: (row, chunk) pieces this thread handed out
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          const bool full = (col + 32 <= N);
          if (EPI == EPI_BF16_BCAST) {
            uint32_t p[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) p[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            for (int d = 0; d < bc.n; ++d) {
              __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(bc.dst[d]) + (size_t)row * ldc + col;
              if (full) {
                uint4* C4 = reinterpret_cast<uint4*>(C);
#pragma unroll
                for (int j = 0; j < 4; ++j) C4[j] = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col + j < N) C[j] = __float2bfloat16(__uint_as_float(r[j]));
              }
            }
            ++pieces;
          } else if (EPI == EPI_BF16 || EPI == EPI_BF16_RESID) {
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(Cptr_t) + (size_t)row * ldc + col;
            if (full) {
              uint32_t p[16];
              if (EPI == EPI_BF16_RESID) {
                const uint4* R4 = reinterpret_cast<const uint4*>(Rptr + (size_t)row * ldc + col);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 rv = R4[j];
                  const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16(rr[e]);
                    p[j * 4 + e] = pack_bf16(__uint_as_float(r[j * 8 + e * 2]) + f.x,
                                             __uint_as_float(r[j * 8 + e * 2 + 1]) + f.y);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  p[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
              }
              uint4* C4 = reinterpret_cast<uint4*>(C);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                C4[j] = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < N) {
                  float v = __uint_as_float(r[j]);
                  if (EPI == EPI_BF16_RESID) v += __bfloat162float(Rptr[(size_t)row * ldc + col + j]);
                  C[j] = __float2bfloat16(v);
                }
              }
            }
          } else {
            float* C = reinterpret_cast<float*>(Cptr_t) + (size_t)row * ldc + col;
            if (full) {
              float4* C4 = reinterpret_cast<float4*>(C);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (EPI == EPI_F32_ACC) {
                  const float4 o = C4[j];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                C4[j] = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < N) {
                  float v = __uint_as_float(r[j]);
                  if (EPI == EPI_F32_ACC) v += C[j];
                  C[j] = v;
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
      if (EPI == EPI_BF16_BCAST) {
        // the warp's stores of this tile become visible everywhere before its share of the count does
        int total = pieces;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);   // also orders the lanes' stores before lane 0
        if (lane == 0 && total > 0) {
          __threadfence_system();
          for (int d = 0; d < bc.n; ++d)
            asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(bc.counter[d]), "l"((unsigned long long)total) : "memory");
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

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(int epi, const void* A, const void* B, void* C, const void* R, int M, int N,
                       int K, int lda, int ldb, int ldc, cudaStream_t stream, const BcastArgs* bcast = nullptr) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = ab2host::encode_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true, 0);
  else
    rc = ab2host::encode_tmap_2d(&tmA, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, true, 0);
  if (rc) return 100 + rc;
  if (!B_MN)
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, true, 0);
  else
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true, 0);
  if (rc) return 200 + rc;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static ab2host::DevState st;
  int num_sms = 0;
  if (int e = ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, st, &num_sms)) return e;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  BcastArgs none = {};
  launch_pdl(kern, dim3(grid), dim3(192), (size_t)Cfg::SMEM_BYTES, stream, tmA, tmB, C, reinterpret_cast<const __nv_bfloat16*>(R), M, N, K,
             ldc, epi, err, 1, 0, bcast ? *bcast : none);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

// Sum of the split-K pieces: out[i] = bf16(sum_s ws[s * MN + i] (+ resid[i])). MN is a multiple of 4.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out,
                                     const __nv_bfloat16* __restrict__ resid, int splits, long long MN) {
  pdl_wait();
  pdl_trigger();
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < MN; i += (long long)gridDim.x * blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4*>(ws + i);
    for (int sp = 1; sp < splits; ++sp) {
      const float4 v = *reinterpret_cast<const float4*>(ws + (size_t)sp * MN + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (resid != nullptr) {
      const uint2 r = *reinterpret_cast<const uint2*>(resid + i);
      const float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y);
      acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
    }
    *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
  }
}

// Y[M, N] (bf16) = A[M, K] B[N, K]^T (+ R) with the K range split over `splits` CTAs per output tile:
// pieces go to ws ([splits, M, N] fp32) with plain stores, a second kernel sums them.
template <int BN>
static int launch_splitk(const void* A, const void* B, void* Y, const void* R, float* ws, int M, int N, int K, int lda, int ldb,
                         int splits, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = ab2host::encode_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true, 0);
  if (rc) return 100 + rc;
  rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, true, 0);
  if (rc) return 200 + rc;
  auto kern = gemm_bf16_kernel<BN, false, false, true>;
  static ab2host::DevState st;
  int num_sms = 0;
  if (int e = ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, st, &num_sms)) return e;
  const int num_kb = (K + BK - 1) / BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per - 1) / kb_per;             // every piece owns at least one k-block
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
  const int grid = tiles < num_sms ? tiles : num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  if (launch_pdl(kern, dim3(grid), dim3(192), (size_t)Cfg::SMEM_BYTES, stream, tmA, tmB, (void*)ws, (const __nv_bfloat16*)nullptr, M, N, K, N,
                 (int)EPI_F32, err, splits, kb_per, BcastArgs{}) != cudaSuccess)
    return 302;
  const long long MN = (long long)M * N;
  long long want = (MN / 4 + 255) / 256;
  const int rgrid = (int)(want < 148 * 8 ? want : 148 * 8);
  if (launch_pdl(splitk_reduce_kernel, dim3(rgrid), dim3(256), 0, stream, (const float*)ws, (__nv_bfloat16*)Y, (const __nv_bfloat16*)R, splits,
                 MN) != cudaSuccess)
    return 303;
  return 0;
}

template <int BN>
static int dispatch_major(int a_mn, int b_mn, int epi, const void* A, const void* B, void* C,
                          const void* R, int M, int N, int K, int lda, int ldb, int ldc,
                          cudaStream_t s) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  return launch_gemm<BN, true, true>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
}

}  // namespace ab2

extern "C" {

// C[M,N] (+)= op(A) op(B) with bf16 inputs and fp32 accumulation on tcgen05 tensor cores.
//   a_mn = 0: A is [M,K] row-major (lda >= K);  a_mn = 1: A is [K,M] row-major (lda >= M)
//   b_mn = 0: B is [N,K] row-major (ldb >= K);  b_mn = 1: B is [K,N] row-major (ldb >= N)
//   epi: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate into C, 3 bf16 store of acc + R
//        (R has C's shape and ldc).
//   bn: output tile width (256/128/64/32) or 0 to choose from the problem size.
// Requirements: leading dimensions multiples of 8 elements, pointers 16-byte aligned.
// Returns 0 on success (launch only; asynchronous on `stream`).
int ab2_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda,
                  int ldb, int ldc, int a_mn, int b_mn, int epi, int bn, void* stream) {
  using namespace ab2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epi < 0 || epi > 3) return 13;
  if ((lda & 7) || (ldb & 7) || (ldc & 3)) return 10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return 11;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0) {
    const int mblk = (M + BM - 1) / BM;
    bn = 256;
    // Shrink the tile until the grid can fill the machine (small-M decode GEMMs).
    while (bn > (b_mn ? 64 : 32) && mblk * ((N + bn - 1) / bn) < 120) bn >>= 1;
  }
  if (b_mn && bn < 64) bn = 64;
  switch (bn) {
    case 256: return dispatch_major<256>(a_mn, b_mn, epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
    case 128: return dispatch_major<128>(a_mn, b_mn, epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
    case 64: return dispatch_major<64>(a_mn, b_mn, epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
    case 32: return dispatch_major<32>(a_mn, b_mn, epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  }
  return 12;
}

// Y = A[M, K] B[N, K]^T in bf16, stored into `ndst` buffers at once (dst[i], all with leading dimension
// ldc; peers' buffers are addressed through peer-mapped symmetric memory), followed by a release-add of
// M * ceil(N / 32) on counters[i]. The row-parallel products of a tensor-parallel layer use it to hand
// their partial result to every rank of the group from inside the GEMM epilogue; the consumer
// (ab2_tp_reduce_rmsnorm) waits on its own counter and sums the partials.
int ab2_gemm_bf16_bcast(const void* A, const void* B, void* const* dst, void* const* counters, int ndst, int M, int N, int K,
                        int lda, int ldb, int ldc, int bn, void* stream) {
  using namespace ab2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (ndst < 1 || ndst > BCAST_MAX) return 13;
  if ((lda & 7) || (ldb & 7) || (ldc & 7)) return 10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return 11;
  BcastArgs bc = {};
  bc.n = ndst;
  for (int i = 0; i < ndst; ++i) {
    if (!dst[i] || !counters[i] || (reinterpret_cast<uintptr_t>(dst[i]) & 15)) return 11;
    bc.dst[i] = dst[i];
    bc.counter[i] = reinterpret_cast<unsigned long long*>(counters[i]);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0) {
    const int mblk = (M + BM - 1) / BM;
    bn = 256;
    while (bn > 32 && mblk * ((N + bn - 1) / bn) < 120) bn >>= 1;
  }
  switch (bn) {
    case 256: return launch_gemm<256, false, false>(EPI_BF16_BCAST, A, B, dst[0], nullptr, M, N, K, lda, ldb, ldc, s, &bc);
    case 128: return launch_gemm<128, false, false>(EPI_BF16_BCAST, A, B, dst[0], nullptr, M, N, K, lda, ldb, ldc, s, &bc);
    case 64: return launch_gemm<64, false, false>(EPI_BF16_BCAST, A, B, dst[0], nullptr, M, N, K, lda, ldb, ldc, s, &bc);
    case 32: return launch_gemm<32, false, false>(EPI_BF16_BCAST, A, B, dst[0], nullptr, M, N, K, lda, ldb, ldc, s, &bc);
  }
  return 12;
}

// Decode-shaped product: Y[M, N] (bf16, dense rows) = A[M, K] B[N, K]^T (+ R, Y's layout), K split over
// `splits` CTAs per 128 x bn output tile. ws: fp32 workspace of at least splits * M * N elements (no
// initialisation needed). N must be a multiple of 4; lda / ldb multiples of 8.
int ab2_gemm_splitk(const void* A, const void* B, void* Y, const void* R, void* ws, int M, int N, int K, int lda, int ldb, int splits,
                    int bn, void* stream) {
  using namespace ab2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (N & 3) || splits < 1 || !ws) return 10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(Y)) & 15) return 11;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* w = reinterpret_cast<float*>(ws);
  switch (bn) {
    case 256: return launch_splitk<256>(A, B, Y, R, w, M, N, K, lda, ldb, splits, s);
    case 128: return launch_splitk<128>(A, B, Y, R, w, M, N, K, lda, ldb, splits, s);
    case 64: return launch_splitk<64>(A, B, Y, R, w, M, N, K, lda, ldb, splits, s);
  }
  return 12;
}
}
