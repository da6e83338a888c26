// Grouped bf16 GEMM for mixture-of-experts layers: one persistent tcgen05 kernel computes
//
//   C[rows of expert e, N] = A[rows of expert e, K] * op(B[e])        for every local expert e
//
// where the token rows are sorted by expert (variable group sizes) and B is the stack of expert
// weights. The host turns the group sizes into a tile table (expert, first row, valid rows,
// n-block); the TMA producer loads A tiles by row offset and B tiles through a 3-D tensor map
// indexed by expert, the epilogue masks the rows that spill into the next group. Pipeline (TMA ->
// 128B-swizzled smem -> tcgen05.mma -> TMEM -> epilogue warps) as in gemm.cu.
//
// Takes the place of torch._grouped_mm in the reference's expert layers
// (areal/experimental/models/archon/moe/grouped_experts.py:100-207) and of the per-expert
// Python loop of GEMM launches.
#include "common.cuh"

namespace ab2 {

static constexpr int BM = 128;
static constexpr int BK = 64;
static constexpr int UMMA_K = 16;

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

// tiles: int4 per output tile = (expert, first row, valid rows, n-block). A is K-major [R, K]
// (rows grouped by expert), B is the expert stack [E, N, K] (K-major) or [E, K, N] (MN-major).
template <int BN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    __nv_bfloat16* __restrict__ Cptr, const int4* __restrict__ tiles, int num_tiles, int N,
                    int K, int ldc, int* err, const int* __restrict__ num_rt_dev, int nblk) {
  constexpr bool A_MN = false;
  // Row-tile mode (nblk > 0): `tiles` lists 128-row tiles only, written by the routing kernel together with
  // their number; output tile i covers row tile i / nblk and n-block i % nblk, and the grid was sized for
  // an upper bound of the row tiles.
  if (nblk > 0) {
    const int have = *num_rt_dev * nblk;
    num_tiles = have < num_tiles ? have : num_tiles;
  }
  auto tile_info = [&](int tile) -> int4 {
    if (nblk > 0) {
      int4 t = tiles[tile / nblk];
      t.w = tile % nblk;
      return t;
    }
    return tiles[tile];
  };
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
  const int num_kb = (K + BK - 1) / BK;

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

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int4 ti = tile_info(tile);
        const int expert = ti.x, m0 = ti.y, n0 = ti.w * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            tma_load_3d(sB, &tmB, full_bar(stage), kb * BK, n0, expert);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sB + c * (BK * 128), &tmB, full_bar(stage), n0 + c * 64, kb * BK, expert);
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
        for (int kb = 0; kb < num_kb; ++kb) {
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
            umma_f16(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
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
      const int4 ti = tile_info(tile);
      const int m0 = ti.y, rows_valid = ti.z, n0 = ti.w * BN;
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      if (!mbar_wait(tfull_bar(buf), use & 1u, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row_in_tile < rows_valid && col < N) {       // rows past the expert's group belong to the next one
          __nv_bfloat16* C = Cptr + (size_t)row * ldc + col;
          if (col + 32 <= N) {
            uint4* C4 = reinterpret_cast<uint4*>(C);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              C4[j] = make_uint4(pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                 pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                 pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                 pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
          } else {
            for (int j = 0; j < 32; ++j)
              if (col + j < N) C[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}


template <int BN, bool B_MN>
static int launch_grouped(const void* A, const void* B, void* C, const void* tiles, int num_tiles, int R, int N, int K, int E,
                          int lda, int ldc, cudaStream_t stream, const int* num_rt_dev = nullptr, int nblk = 0) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc = ab2host::encode_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)R, (uint64_t)lda * 2, BK, BM, true, 0);
  if (rc) return 100 + rc;
  if (!B_MN)  // [E, N, K]
    rc = ab2host::encode_tmap_3d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)E, (uint64_t)K * 2, (uint64_t)N * K * 2, BK, BN, 1, true, 0);
  else        // [E, K, N]
    rc = ab2host::encode_tmap_3d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)E, (uint64_t)N * 2, (uint64_t)N * K * 2, 64, BK, 1, true, 0);
  if (rc) return 200 + rc;
  auto kern = gemm_grouped_kernel<BN, B_MN>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, dev_state, &num_sms)) return 300;
  (void)num_sms;
  const int grid = num_tiles < num_sms ? num_tiles : num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), reinterpret_cast<const int4*>(tiles),
                                               num_tiles, N, K, ldc, err, num_rt_dev, nblk);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

}  // namespace ab2

extern "C" {

// A: [R, K] bf16 rows grouped by expert (lda elements per row). B: [E, N, K] (b_mn = 0) or
// [E, K, N] (b_mn = 1) bf16, contiguous. C: [R, N] bf16 (ldc). tiles: device int32[num_tiles][4] =
// (expert, first row, valid rows (<= 128), n-block of width bn). bn: 128 or 256 (b_mn needs >= 64).
int ab2_gemm_grouped(const void* A, const void* B, void* C, const void* tiles, int num_tiles, int R, int N, int K, int E, int lda,
                     int ldc, int b_mn, int bn, void* stream) {
  using namespace ab2;
  if (num_tiles <= 0 || R <= 0) return 0;
  if ((lda & 7) || (ldc & 7) || (K & 7) || (N & 7)) return 10;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 256) return b_mn ? launch_grouped<256, true>(A, B, C, tiles, num_tiles, R, N, K, E, lda, ldc, s)
                             : launch_grouped<256, false>(A, B, C, tiles, num_tiles, R, N, K, E, lda, ldc, s);
  if (bn == 128) return b_mn ? launch_grouped<128, true>(A, B, C, tiles, num_tiles, R, N, K, E, lda, ldc, s)
                             : launch_grouped<128, false>(A, B, C, tiles, num_tiles, R, N, K, E, lda, ldc, s);
  return 12;
}

// Same product with the tile list made on the device: row_tiles [max_row_tiles] int4 = (expert, first row,
// valid rows, -) and *num_row_tiles as written by ab2_moe_route; no host copy of the group sizes is needed.
int ab2_gemm_grouped_rt(const void* A, const void* B, void* C, const void* row_tiles, const void* num_row_tiles, int max_row_tiles,
                        int R, int N, int K, int E, int lda, int ldc, int b_mn, int bn, void* stream) {
  using namespace ab2;
  if (max_row_tiles <= 0 || R <= 0) return 0;
  if ((lda & 7) || (ldc & 7) || (K & 7) || (N & 7)) return 10;
  if (bn != 128 && bn != 256) return 12;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nblk = (N + bn - 1) / bn;
  const long long max_tiles = (long long)max_row_tiles * nblk;
  if (max_tiles > 0x7fffffffLL) return 13;
  const int* nrt = reinterpret_cast<const int*>(num_row_tiles);
  if (bn == 256) return b_mn ? launch_grouped<256, true>(A, B, C, row_tiles, (int)max_tiles, R, N, K, E, lda, ldc, s, nrt, nblk)
                             : launch_grouped<256, false>(A, B, C, row_tiles, (int)max_tiles, R, N, K, E, lda, ldc, s, nrt, nblk);
  return b_mn ? launch_grouped<128, true>(A, B, C, row_tiles, (int)max_tiles, R, N, K, E, lda, ldc, s, nrt, nblk)
              : launch_grouped<128, false>(A, B, C, row_tiles, (int)max_tiles, R, N, K, E, lda, ldc, s, nrt, nblk);
}
}
