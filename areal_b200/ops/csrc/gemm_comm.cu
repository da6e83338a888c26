// GEMMs fused with their tensor-parallel collective over NVLink peer memory (one kernel each):
//
//   all-gather -> GEMM : C[M, N] = gather_rows(A_0 .. A_{P-1}) * B^T (or * B)
//       A is the row-wise concatenation of P rank-local [M/P, K] blocks that live in symmetric
//       (peer-mapped) memory. The TMA producer picks, per output tile, the tensor map of the
//       rank that owns the tile's rows and loads straight from that GPU's HBM over NVLink
//       (plain TMA loads, no multicast). Tiles whose rows are local come first, so the local
//       math covers the latency of the first remote loads.
//
//   GEMM -> reduce-scatter : out_r[M/P, N] (fp32) += rows r of (A * B^T)   for every owner r
//       each rank computes its partial product and the epilogue adds every tile row directly
//       into the owning rank's fp32 buffer with vector reductions (red.global.add.v4.f32) on
//       the peer pointer; the transfer of tile i overlaps the math of tile i+1 (two TMEM
//       accumulators). Remote owners are visited first.
//
// Operand layouts: A K-major ([rows, K]); B K-major ([N, K], the weight layout) or MN-major
// ([K, N]). The pipeline (TMA -> 128B-swizzled smem -> tcgen05.mma -> TMEM -> epilogue warps)
// is the one of gemm.cu. Callers bracket the kernels with the bounded device barrier
// (ab2_signal_barrier): buffers complete before remote loads, reductions landed before use.
//
// Takes the place of the all_gather / reduce_scatter + cuBLAS pairs behind the reference's
// tensor-parallel linear layers (areal/engine/fsdp_utils/parallel.py:227-385, DTensor
// Colwise/Rowwise plans) and of SGLang's TP all-reduce on the rollout side.
#include "common.cuh"

namespace ab2 {

static constexpr int GC_BM = 128;
static constexpr int GC_BK = 64;
static constexpr int GC_UMMA_K = 16;
static constexpr int GC_MAX_PEERS = 8;

struct TmapArray {
  CUtensorMap m[GC_MAX_PEERS];
};
struct OutPtrs {
  float* p[GC_MAX_PEERS];
};

template <int BN>
struct GcCfg {
  static constexpr int A_BYTES = GC_BM * GC_BK * 2;
  static constexpr int B_BYTES = BN * GC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (196 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

// Tile order: M-blocks are rotated so that the blocks owned by `first_owner` come first.
__device__ __forceinline__ void gc_tile(int tile, int m_blocks, int n_blocks, int blocks_per_rank, int first_owner, int P,
                                        int& mb, int& nb) {
  const int m_lin = tile / n_blocks;
  nb = tile - m_lin * n_blocks;
  mb = (m_lin + first_owner * blocks_per_rank) % m_blocks;
}

// MODE 0: gathered A, local bf16 output. MODE 1: local A, fp32 reduction into the row owners.
template <int BN, bool B_MN, int MODE>
__global__ void __launch_bounds__(192, 1)
gemm_comm_kernel(const __grid_constant__ TmapArray tmA, const __grid_constant__ CUtensorMap tmB,
                 __nv_bfloat16* __restrict__ Cloc, const __grid_constant__ OutPtrs outs, int M, int N, int K, int ldc, int rows_per_rank,
                 int my_rank, int P, int* err) {
  using Cfg = GcCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (M + GC_BM - 1) / GC_BM;
  const int n_blocks = (N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (K + GC_BK - 1) / GC_BK;
  const int blocks_per_rank = rows_per_rank / GC_BM;
  // gather: start with the local rows; reduce: start with the next rank's rows (remote first)
  const int first_owner = MODE == 0 ? my_rank : (my_rank + 1) % P;

  if (threadIdx.x == 0) {
    for (int r = 0; r < (MODE == 0 ? P : 1); ++r) prefetch_tmap(&tmA.m[r]);
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
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        gc_tile(tile, m_blocks, n_blocks, blocks_per_rank, first_owner, P, mb, nb);
        const int m0 = mb * GC_BM, n0 = nb * BN;
        const int owner = MODE == 0 ? m0 / rows_per_rank : 0;
        const int a_row = MODE == 0 ? m0 - owner * rows_per_rank : m0;
        const CUtensorMap* ta = &tmA.m[owner];
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
          tma_load_2d(sA, ta, full_bar(stage), kb * GC_BK, a_row);
          if (!B_MN) {
            tma_load_2d(sB, &tmB, full_bar(stage), kb * GC_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * (GC_BK * 128), &tmB, full_bar(stage), n0 + c * 64, kb * GC_BK);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long t0 = clock64();
          while (clock64() - t0 < 4000000LL) { /* bounded grace for (possibly remote) copies in flight */ }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(GC_BM, BN, 1, 1, 0, B_MN ? 1 : 0);
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
          const uint64_t adesc = make_smem_desc_sw128(sA, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sB, B_MN ? GC_BK * 128 : 16, 1024);
#pragma unroll
          for (int k = 0; k < GC_BK / GC_UMMA_K; ++k) {
            const uint64_t ad = adesc + (uint64_t)(k * 2);
            const uint64_t bd = bdesc + (B_MN ? (uint64_t)(k * (GC_UMMA_K * 128 >> 4)) : (uint64_t)(k * 2));
            umma_f16(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int mb, nb;
      gc_tile(tile, m_blocks, n_blocks, blocks_per_rank, first_owner, P, mb, nb);
      const int m0 = mb * GC_BM, n0 = nb * BN;
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      if (!mbar_wait(tfull_bar(buf), use & 1u, err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      float* red_row = nullptr;
      if (MODE == 1 && row < M) {
        const int owner = row / rows_per_rank;
        red_row = outs.p[owner] + (size_t)(row - owner * rows_per_rank) * ldc;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          const bool full = (col + 32 <= N);
          if (MODE == 0) {
            __nv_bfloat16* C = Cloc + (size_t)row * ldc + col;
            if (full) {
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
          } else {
            float* dst = red_row + col;
            if (full) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j), "f"(__uint_as_float(r[4 * j])),
                             "f"(__uint_as_float(r[4 * j + 1])), "f"(__uint_as_float(r[4 * j + 2])),
                             "f"(__uint_as_float(r[4 * j + 3]))
                             : "memory");
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col + j < N) atomicAdd(dst + j, __uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
    }
    if (MODE == 1) __threadfence_system();  // reductions on peer memory ordered before the closing barrier
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool B_MN, int MODE>
static int launch_gc(void* const* a_ptrs, const void* B, void* C, float* const* out_ptrs, int M, int N, int K, int lda, int ldb,
                     int ldc, int rows_per_rank, int my_rank, int P, cudaStream_t stream) {
  using Cfg = GcCfg<BN>;
  TmapArray ta;
  int rc;
  const int nA = MODE == 0 ? P : 1;
  const uint64_t a_rows = MODE == 0 ? (uint64_t)rows_per_rank : (uint64_t)M;
  for (int r = 0; r < nA; ++r) {
    rc = ab2host::encode_tmap_2d(&ta.m[r], a_ptrs[r], 2, (uint64_t)K, a_rows, (uint64_t)lda * 2, GC_BK, GC_BM, true, 0);
    if (rc) return 100 + rc;
  }
  for (int r = nA; r < GC_MAX_PEERS; ++r) ta.m[r] = ta.m[0];
  CUtensorMap tmB;
  if (!B_MN)
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, GC_BK, BN, true, 0);
  else
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, GC_BK, true, 0);
  if (rc) return 200 + rc;
  OutPtrs op;
  for (int r = 0; r < GC_MAX_PEERS; ++r) op.p[r] = (MODE == 1 && r < P) ? out_ptrs[r] : nullptr;
  auto kern = gemm_comm_kernel<BN, B_MN, MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return 300;
    attr_set = true;
  }
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + GC_BM - 1) / GC_BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(ta, tmB, reinterpret_cast<__nv_bfloat16*>(C), op, M, N, K, ldc, rows_per_rank,
                                               my_rank, P, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

template <int MODE>
static int dispatch_gc(int bn, int b_mn, void* const* a_ptrs, const void* B, void* C, float* const* out_ptrs, int M, int N, int K,
                       int lda, int ldb, int ldc, int rpr, int me, int P, cudaStream_t s) {
  if (bn == 256) {
    return b_mn ? launch_gc<256, true, MODE>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, s)
                : launch_gc<256, false, MODE>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, s);
  }
  return b_mn ? launch_gc<128, true, MODE>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, s)
              : launch_gc<128, false, MODE>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, s);
}

}  // namespace ab2

extern "C" {

// C[M, N] (bf16, local) = concat_r(A_r)[M, K] * op(B). a_ptrs[r]: rank r's [M/P, K] block (lda
// elements per row) as mapped into this process; rows_per_rank = M / P must be a multiple of
// 128. b_mn = 0: B is [N, K]; 1: B is [K, N].
int ab2_allgather_gemm(void* const* a_ptrs, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int b_mn,
                       int my_rank, int world, void* stream) {
  using namespace ab2;
  if (world < 1 || world > GC_MAX_PEERS) return 10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M % world || (M / world) % GC_BM) return 11;
  if ((lda & 7) || (ldb & 7) || (ldc & 7)) return 12;
  const int bn = (N % 256 == 0 && ((M + 127) / 128) * (N / 256) >= 120) ? 256 : 128;
  return dispatch_gc<0>(bn, b_mn, a_ptrs, B, C, nullptr, M, N, K, lda, ldb, ldc, M / world, my_rank, world,
                        reinterpret_cast<cudaStream_t>(stream));
}

// out_r[M/P, N] (fp32, rank r's buffer as mapped here, ldc elements per row) += rows r of A * op(B).
// All buffers must be zero (or hold the value to add to) and visible before any rank launches;
// results are complete after a barrier that follows every rank's kernel.
int ab2_gemm_reduce_scatter(const void* A, const void* B, void* const* out_ptrs, int M, int N, int K, int lda, int ldb, int ldc,
                            int b_mn, int my_rank, int world, void* stream) {
  using namespace ab2;
  if (world < 1 || world > GC_MAX_PEERS) return 10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M % world || (M / world) % GC_BM) return 11;
  if ((lda & 7) || (ldb & 7) || (ldc & 3)) return 12;
  const int bn = (N % 256 == 0 && ((M + 127) / 128) * (N / 256) >= 120) ? 256 : 128;
  void* a1[1] = {const_cast<void*>(A)};
  return dispatch_gc<1>(bn, b_mn, a1, B, nullptr, reinterpret_cast<float* const*>(out_ptrs), M, N, K, lda, ldb, ldc, M / world,
                        my_rank, world, reinterpret_cast<cudaStream_t>(stream));
}
}
