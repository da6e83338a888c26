// Dense bf16 GEMM on CTA PAIRS: tcgen05.mma.cta_group::2 computes one 256 x 256 output tile on
// two SMs of a cluster. Each CTA stages its own 128 rows of A and only HALF of the B tile (its
// 128 of the 256 columns): the tensor cores of both SMs read both halves, so the shared-memory
// traffic per flop drops by a third against the one-CTA 128 x 256 tile of gemm.cu, which is
// bound by the shared-memory -> tensor-core path.
//
//   C[M,N] (+)= A * B      operand layouts and epilogues exactly as ab2_gemm_bf16 (gemm.cu)
//
// Cluster of 2 CTAs along M, 192 threads each: warp 0 = TMA producer (each CTA loads its own
// tiles; both CTAs' copies complete on the LEADER's "full" barrier: plain non-multicast loads
// with the cta_group::2 form), warp 1 of the leader (cluster rank 0) = MMA issuer for the pair,
// warps 2..5 of each CTA = epilogue of that CTA's 128 rows (its own TMEM). "Stage consumed"
// and "accumulator ready" are signalled to both CTAs with tcgen05.commit ... multicast::cluster;
// "accumulator drained" comes back to the leader as remote mbarrier arrives.
//
// Every wait is bounded (common.cuh); a give-up records its code and both CTAs unwind through
// the closing cluster barrier.
#include <stdio.h>

#include "common.cuh"

namespace ab2 {

static constexpr int P2_BM = 128;      // rows per CTA (256 per pair)
static constexpr int P2_BN = 256;      // columns per pair; each CTA stages 128 of them
static constexpr int P2_BK = 64;
static constexpr int P2_UMMA_K = 16;

struct P2Cfg {
  static constexpr int A_BYTES = P2_BM * P2_BK * 2;
  static constexpr int B_BYTES = (P2_BN / 2) * P2_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 32 KiB per CTA and stage
  static constexpr int STAGES = 6;
  static constexpr int TMEM_COLS = 512;                      // two 256-column accumulators
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load of the pair form: data lands in THIS CTA's shared memory, the bytes are counted on
// the barrier at `bar_cluster_addr` (the leader's). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at the same offset in BOTH CTAs of the pair once the MMAs issued so far retire
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
               : "memory");
}

enum Epi2 : int { E2_BF16 = 0, E2_F32 = 1, E2_F32_ACC = 2, E2_BF16_RESID = 3 };

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cptr,
                     const __nv_bfloat16* __restrict__ Rptr, int M, int N, int K, int ldc, const int EPI, int* err) {
  using Cfg = P2Cfg;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw2[];
  const uint32_t smem_base = (smem_u32(smem_raw2) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                         // used in the leader only
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };             // one per CTA
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };         // one per CTA
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };    // used in the leader only
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const bool leader = crank == 0;
  const int m_pairs = (M + 2 * P2_BM - 1) / (2 * P2_BM);
  const int n_blocks = (N + P2_BN - 1) / P2_BN;
  const int num_tiles = m_pairs * n_blocks;
  const int num_kb = (K + P2_BK - 1) / P2_BK;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  // tile order: groups of 8 row pairs sweep the column blocks together (L2 reuse of B and A)
  auto tile_coords2 = [&](int tile, int& mp, int& nb) {
    constexpr int GROUP = 8;
    const int per_group = GROUP * n_blocks;
    const int g = tile / per_group;
    const int first = g * GROUP;
    const int gsize = min(GROUP, m_pairs - first);
    const int in_g = tile - g * per_group;
    mp = first + in_g % gsize;
    nb = in_g / gsize;
  };

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);       // the leader's expect_tx arrive; bytes come from both CTAs
      mbar_init(empty_bar(s), 1);      // one multicast commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);      // one multicast commit
      mbar_init(tempty_bar(b), 8);     // 4 epilogue warps of each CTA
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);    // warp 1 of BOTH CTAs, collectively
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // the peer's barriers exist before anything signals them
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += n_clusters) {
        int mp, nb;
        tile_coords2(tile, mp, nb);
        const int m0 = mp * 2 * P2_BM + (int)crank * P2_BM;           // this CTA's rows
        const int n0 = nb * P2_BN + (int)crank * (P2_BN / 2);        // this CTA's half of the columns
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint32_t fb = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d_pair(sA, &tmA, fb, kb * P2_BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < P2_BM / 64; ++c) tma_load_2d_pair(sA + c * (P2_BK * 128), &tmA, fb, m0 + c * 64, kb * P2_BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, fb, kb * P2_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < (P2_BN / 2) / 64; ++c) tma_load_2d_pair(sB + c * (P2_BK * 128), &tmB, fb, n0 + c * 64, kb * P2_BK);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) { /* let copies in flight land */ }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader only, for the pair)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = make_idesc(2 * P2_BM, P2_BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += n_clusters, ++local) {
        const int buf = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * P2_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          const uint64_t adesc = make_smem_desc_sw128(sA, A_MN ? P2_BK * 128 : 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sB, B_MN ? P2_BK * 128 : 16, 1024);
#pragma unroll
          for (int k = 0; k < P2_BK / P2_UMMA_K; ++k) {
            const uint64_t ad = adesc + (A_MN ? (uint64_t)(k * (P2_UMMA_K * 128 >> 4)) : (uint64_t)(k * 2));
            const uint64_t bd = bdesc + (B_MN ? (uint64_t)(k * (P2_UMMA_K * 128 >> 4)) : (uint64_t)(k * 2));
            umma_f16_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));          // both CTAs may refill this stage
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(buf));       // both CTAs' epilogues may read their accumulators
      }
    }
  } else {
    // ------------------------------------------------ epilogue (warps 2..5 of each CTA, its own 128 rows)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t tempty_leader0 = map_to_cta(tempty_bar(0), 0), tempty_leader1 = map_to_cta(tempty_bar(1), 0);
    bool ok = true;
    int local = 0;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += n_clusters, ++local) {
      int mp, nb;
      tile_coords2(tile, mp, nb);
      const int m0 = mp * 2 * P2_BM + (int)crank * P2_BM, n0 = nb * P2_BN;
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), use & 1u, err, ERR_WAIT_TMEM_FULL));
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * P2_BN;
#pragma unroll 1
      for (int c = 0; c < P2_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          const bool full = (col + 32 <= N);
          if (EPI == E2_BF16 || EPI == E2_BF16_RESID) {
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(Cptr) + (size_t)row * ldc + col;
            if (full) {
              uint32_t p[16];
              if (EPI == E2_BF16_RESID) {
                const uint4* R4 = reinterpret_cast<const uint4*>(Rptr + (size_t)row * ldc + col);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint4 rv = R4[j];
                  const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16(rr[e]);
                    p[j * 4 + e] = pack_bf16(__uint_as_float(r[j * 8 + e * 2]) + f.x, __uint_as_float(r[j * 8 + e * 2 + 1]) + f.y);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) p[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
              }
              uint4* C4 = reinterpret_cast<uint4*>(C);
#pragma unroll
              for (int j = 0; j < 4; ++j) C4[j] = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < N) {
                  float v = __uint_as_float(r[j]);
                  if (EPI == E2_BF16_RESID) v += __bfloat162float(Rptr[(size_t)row * ldc + col + j]);
                  C[j] = __float2bfloat16(v);
                }
              }
            }
          } else {
            float* C = reinterpret_cast<float*>(Cptr) + (size_t)row * ldc + col;
            if (full) {
              float4* C4 = reinterpret_cast<float4*>(C);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                       __uint_as_float(r[4 * j + 3]));
                if (EPI == E2_F32_ACC) {
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
                  if (EPI == E2_F32_ACC) v += C[j];
                  C[j] = v;
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? tempty_leader1 : tempty_leader0);   // this warp is done with the accumulator
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // nobody leaves (or frees TMEM) while the peer may still touch this CTA
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch_gemm_2sm(int epi, const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc,
                           cudaStream_t stream) {
  using Cfg = P2Cfg;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = ab2host::encode_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, P2_BK, P2_BM, true, 0);
  else
    rc = ab2host::encode_tmap_2d(&tmA, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, P2_BK, true, 0);
  if (rc) return 100 + rc;
  if (!B_MN)
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, P2_BK, P2_BN / 2, true, 0);
  else
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, P2_BK, true, 0);
  if (rc) return 200 + rc;
  auto kern = gemm_bf16_2sm_kernel<A_MN, B_MN>;
  static ab2host::DevState st;
  int num_sms = 0;
  if (int e = ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, st, &num_sms)) return e;
  const int tiles = ((M + 2 * P2_BM - 1) / (2 * P2_BM)) * ((N + P2_BN - 1) / P2_BN);
  int clusters = num_sms / 2;
  if (tiles < clusters) clusters = tiles;
  int* err = ab2host::error_flag();
  if (!err) return 301;
  kern<<<dim3(2 * clusters), dim3(192), Cfg::SMEM_BYTES, stream>>>(tmA, tmB, C, reinterpret_cast<const __nv_bfloat16*>(R), M, N, K, ldc, epi,
                                                                    err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

}  // namespace ab2

extern "C" {

// Same contract as ab2_gemm_bf16 (gemm.cu) on 256 x 256 tiles computed by CTA pairs. Meant for large
// products (at least a few hundred 256 x 256 tiles); small or skinny ones stay on the one-CTA kernel.
int ab2_gemm_bf16_2sm(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                      int b_mn, int epi, void* stream) {
  using namespace ab2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epi < 0 || epi > 3) return 13;
  if ((lda & 7) || (ldb & 7) || (ldc & 3)) return 10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return 11;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch_gemm_2sm<false, false>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  if (!a_mn && b_mn) return launch_gemm_2sm<false, true>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  if (a_mn && !b_mn) return launch_gemm_2sm<true, false>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
  return launch_gemm_2sm<true, true>(epi, A, B, C, R, M, N, K, lda, ldb, ldc, s);
}
}
