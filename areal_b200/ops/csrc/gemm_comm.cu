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
//   all-gather -> GEMM, copy-once form (MODE 2): a few CTAs of the same kernel copy each remote
//       row block into a local gathered buffer exactly once (so A crosses NVLink once instead
//       of once per output-tile column) and publish a per-block flag; the GEMM CTAs take local
//       tiles first and wait (bounded) on the flag of a remote block before its first TMA load.
//       All CTAs are co-resident (grid <= number of SMs), so the wait cannot starve.
//
//   GEMM -> all-to-all by columns (MODE 3, Ulysses seq->heads after the QKV projection): the
//       epilogue stores every tile straight into the buffer of the rank that owns those output
//       columns (heads), at this rank's row offset: [T_local, N] -> [P * T_local, N / P] on
//       every owner, plain 16-byte peer stores, no separate all-to-all.
//
//   all-to-all by columns -> GEMM (MODE 4, Ulysses heads->seq before the output projection):
//       the K dimension of A is spread over the ranks ([P * T_local, K / P] each); copy CTAs
//       pull this rank's rows of every remote panel once (TMA load/store pipeline) into a
//       local [T_local, K] buffer, the GEMM starts with the local panel's k-blocks and waits
//       (bounded) per (row block, owner) flag.
//
//   GEMM -> reduce-scatter with bf16 payload (RED_BF16): the epilogue packs to bf16x2 and uses
//       red.global.add.noftz.v4.bf16x2, halving the NVLink bytes (for small groups).
//
// Operand layouts: A K-major ([rows, K]); B K-major ([N, K], the weight layout) or MN-major
// ([K, N]). The pipeline (TMA -> 128B-swizzled smem -> tcgen05.mma -> TMEM -> epilogue warps)
// is the one of gemm.cu. Callers bracket the kernels with the bounded device barrier
// (ab2_signal_barrier): buffers complete before remote loads, reductions landed before use.
//
// Takes the place of the all_gather / reduce_scatter + cuBLAS pairs behind the reference's
// tensor-parallel linear layers (areal/engine/fsdp_utils/parallel.py:227-385, DTensor
// Colwise/Rowwise plans) and of SGLang's TP all-reduce on the rollout side.
#define AB2_WAIT_LIMIT_CYCLES 3000000000LL   // stages here are filled after a peer's flag arrived: allow the ranks' skew
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
  void* p[GC_MAX_PEERS];
};
struct GatherArgs {
  const __nv_bfloat16* peer_a[GC_MAX_PEERS];  // every rank's [rows_per_rank, K] block as mapped here
  __nv_bfloat16* gathered;                    // local [M, K] buffer (remote blocks land here)
  int* flags;                                 // one per 128-row block: == epoch when the block is complete
  int epoch;
  int n_copy;                                 // CTAs [0, n_copy) copy, the rest compute
  int lda;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

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

// MODE 0: A gathered by remote TMA loads, local bf16 output. MODE 1: local A, reduction into the
// row owners (fp32, or bf16x2 with RED_BF16). MODE 2: A gathered by copy CTAs (each remote block
// crosses NVLink once), local bf16 output.
template <int BN, bool B_MN, int MODE, bool RED_BF16>
__global__ void __launch_bounds__(192, 1)
gemm_comm_kernel(const __grid_constant__ TmapArray tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmG, __nv_bfloat16* __restrict__ Cloc, const __grid_constant__ OutPtrs outs, const __grid_constant__ GatherArgs ga,
                 int M, int N, int K, int ldc, int rows_per_rank, int my_rank, int P, int* err) {
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
  const int blocks_per_rank = (MODE == 3 || MODE == 4) ? 0 : rows_per_rank / GC_BM;
  // gather: start with the local rows; reduce: start with the next rank's rows (remote first)
  const int first_owner = MODE == 1 ? (my_rank + 1) % P : ((MODE == 3 || MODE == 4) ? 0 : my_rank);
  const int n_copy = (MODE == 2 || MODE == 4) ? ga.n_copy : 0;
  const int kb_per_rank = MODE == 4 ? (rows_per_rank / GC_BK) : 0;  // MODE 4: rows_per_rank carries K / P
  const int n_compute = gridDim.x - n_copy;

  if (MODE == 4 && (int)blockIdx.x < n_copy) {
    // ------------------------------------------------ copy CTA (column panels): this rank's rows of
    // every remote rank's [T_full, K / P] panel -> local [T_local, K] buffer, once.
    constexpr int GROUP = 6;
    constexpr int BOX_BYTES = GC_BM * GC_BK * 2;
    if (threadIdx.x == 0) {
      const uint32_t gbar0 = smem_base + 2 * GROUP * BOX_BYTES;
      mbar_init(gbar0, 1);
      mbar_init(gbar0 + 8, 1);
      fence_mbar_init();
      for (int r = 0; r < P; ++r) prefetch_tmap(&tmA.m[r]);
      prefetch_tmap(&tmG);
      const int pairs = m_blocks * (P - 1);
      bool ok = true;
      uint32_t ph[2] = {0u, 0u};
      for (int i = blockIdx.x; i < pairs && ok; i += n_copy) {
        const int mb = i / (P - 1);
        const int owner = (my_rank + 1 + (i - mb * (P - 1))) % P;
        const int m0 = mb * GC_BM;
        const int src_row = my_rank * M + m0;             // my rows inside the owner's [P * M, K / P] panel
        const CUtensorMap* ts = &tmA.m[owner];
        const int n_batches = (kb_per_rank + GROUP - 1) / GROUP;
        auto issue_loads = [&](int batch) {
          const int g = batch & 1;
          const int kb_lo = batch * GROUP;
          const int n = min(GROUP, kb_per_rank - kb_lo);
          mbar_expect_tx(gbar0 + 8 * g, n * BOX_BYTES);
          for (int j = 0; j < n; ++j)
            tma_load_2d(smem_base + (g * GROUP + j) * BOX_BYTES, ts, gbar0 + 8 * g, (kb_lo + j) * GC_BK, src_row);
        };
        issue_loads(0);
        if (n_batches > 1) issue_loads(1);
        for (int batch = 0; batch < n_batches; ++batch) {
          const int g = batch & 1;
          if (!mbar_wait(gbar0 + 8 * g, ph[g], err, ERR_WAIT_FULL)) { ok = false; break; }
          ph[g] ^= 1u;
          const int kb_lo = batch * GROUP;
          const int n = min(GROUP, kb_per_rank - kb_lo);
          for (int j = 0; j < n; ++j)
            tma_store_2d(&tmG, smem_base + (g * GROUP + j) * BOX_BYTES, (owner * kb_per_rank + kb_lo + j) * GC_BK, m0);
          tma_store_commit();
          if (batch + 2 < n_batches) {
            tma_store_wait_read<0>();
            issue_loads(batch + 2);
          }
        }
        tma_store_wait<0>();
        fence_proxy_async_global();
        __threadfence();
        if (ok) st_release_gpu(ga.flags + mb * P + owner, ga.epoch);
      }
    }
    return;
  }

  if (MODE == 2 && (int)blockIdx.x < n_copy) {
    // ------------------------------------------------ copy CTA: remote row blocks -> local buffer, once.
    // One elected thread drives a TMA pipeline: 128x64 boxes are loaded from the owner's
    // memory into shared memory (two groups of GROUP stages, so one group's loads are in
    // flight while the other group's stores drain) and stored to the local gathered buffer.
    constexpr int GROUP = 6;
    constexpr int BOX_BYTES = GC_BM * GC_BK * 2;
    if (threadIdx.x == 0) {
      const uint32_t gbar0 = smem_base + 2 * GROUP * BOX_BYTES;  // two 8-byte barriers after the boxes
      mbar_init(gbar0, 1);
      mbar_init(gbar0 + 8, 1);
      fence_mbar_init();
      for (int r = 0; r < P; ++r) prefetch_tmap(&tmA.m[r]);
      prefetch_tmap(&tmG);
      const int remote_blocks = m_blocks - blocks_per_rank;
      bool ok = true;
      uint32_t ph[2] = {0u, 0u};
      for (int i = blockIdx.x; i < remote_blocks && ok; i += n_copy) {
        // i-th remote block in the order the compute CTAs will want them
        const int mb = ((my_rank + 1) * blocks_per_rank + i) % m_blocks;
        const int m0 = mb * GC_BM;
        const int owner = m0 / rows_per_rank;
        const int src_row = m0 - owner * rows_per_rank;
        const CUtensorMap* ts = &tmA.m[owner];
        const int n_batches = (num_kb + GROUP - 1) / GROUP;
        auto issue_loads = [&](int batch) {
          const int g = batch & 1;
          const int kb_lo = batch * GROUP;
          const int n = min(GROUP, num_kb - kb_lo);
          mbar_expect_tx(gbar0 + 8 * g, n * BOX_BYTES);
          for (int j = 0; j < n; ++j)
            tma_load_2d(smem_base + (g * GROUP + j) * BOX_BYTES, ts, gbar0 + 8 * g, (kb_lo + j) * GC_BK, src_row);
        };
        issue_loads(0);
        if (n_batches > 1) issue_loads(1);
        for (int batch = 0; batch < n_batches; ++batch) {
          const int g = batch & 1;
          if (!mbar_wait(gbar0 + 8 * g, ph[g], err, ERR_WAIT_FULL)) { ok = false; break; }
          ph[g] ^= 1u;
          const int kb_lo = batch * GROUP;
          const int n = min(GROUP, num_kb - kb_lo);
          for (int j = 0; j < n; ++j) tma_store_2d(&tmG, smem_base + (g * GROUP + j) * BOX_BYTES, (kb_lo + j) * GC_BK, m0);
          tma_store_commit();
          if (batch + 2 < n_batches) {
            tma_store_wait_read<0>();  // this group's boxes have been read out: refill them
            issue_loads(batch + 2);
          }
        }
        tma_store_wait<0>();           // the whole block is in local memory
        fence_proxy_async_global();
        __threadfence();
        if (ok) st_release_gpu(ga.flags + mb, ga.epoch);
      }
    }
    return;  // copy CTAs own no TMEM
  }

  if (threadIdx.x == 0) {
    for (int r = 0; r < (MODE == 1 ? 1 : P); ++r) prefetch_tmap(&tmA.m[r]);
    if (MODE == 2 || MODE == 4) prefetch_tmap(&tmG);
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
      for (int tile = blockIdx.x - n_copy; tile < num_tiles && ok; tile += n_compute) {
        int mb, nb;
        gc_tile(tile, m_blocks, n_blocks, blocks_per_rank, first_owner, P, mb, nb);
        const int m0 = mb * GC_BM, n0 = nb * BN;
        int owner = 0, a_row = m0;
        if (MODE == 0) {
          owner = m0 / rows_per_rank;
          a_row = m0 - owner * rows_per_rank;
        } else if (MODE == 2) {
          if (m0 / rows_per_rank == my_rank) {
            owner = my_rank;                 // this rank's own block
            a_row = m0 - my_rank * rows_per_rank;
          } else {
            owner = -1;                      // the gathered buffer, filled by the copy CTAs
            const long long t0 = clock64();
            while (ld_acquire_gpu(ga.flags + mb) != ga.epoch) {
              if (clock64() - t0 > WAIT_LIMIT_CYCLES) { set_error(err, ERR_WAIT_PEER_FLAG); ok = false; break; }
              __nanosleep(64);
            }
            if (!ok) break;
            fence_proxy_async_global();
          }
        }
        const CUtensorMap* ta = owner < 0 ? &tmG : &tmA.m[owner];
        for (int it = 0; it < num_kb; ++it) {
          int kb = it;                     // k-block this iteration loads (MODE 4 starts with the local panel)
          int a_col = it * GC_BK;
          if constexpr (MODE == 4) {
            kb = (it + my_rank * kb_per_rank) % num_kb;
            const int k_owner = kb / kb_per_rank;
            if (k_owner == my_rank) {
              ta = &tmA.m[my_rank];
              a_col = (kb - my_rank * kb_per_rank) * GC_BK;
              a_row = my_rank * M + m0;
            } else {
              if (kb == k_owner * kb_per_rank || it == 0) {   // first block of a remote panel: wait for its copy
                const long long t0 = clock64();
                while (ld_acquire_gpu(ga.flags + mb * P + k_owner) != ga.epoch) {
                  if (clock64() - t0 > WAIT_LIMIT_CYCLES) { set_error(err, ERR_WAIT_PEER_FLAG); ok = false; break; }
                  __nanosleep(64);
                }
                if (!ok) break;
                fence_proxy_async_global();
              }
              ta = &tmG;
              a_col = kb * GC_BK;
              a_row = m0;
            }
          }
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
          tma_load_2d(sA, ta, full_bar(stage), a_col, a_row);
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
      for (int tile = blockIdx.x - n_copy; tile < num_tiles && ok; tile += n_compute, ++local) {
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
    for (int tile = blockIdx.x - n_copy; tile < num_tiles && ok; tile += n_compute, ++local) {
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
      __nv_bfloat16* red_row_h = nullptr;
      if (MODE == 1 && row < M) {
        const int owner = row / rows_per_rank;
        const size_t off = (size_t)(row - owner * rows_per_rank) * ldc;
        if (RED_BF16) red_row_h = reinterpret_cast<__nv_bfloat16*>(outs.p[owner]) + off;
        else red_row = reinterpret_cast<float*>(outs.p[owner]) + off;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          const bool full = (col + 32 <= N);
          if (MODE == 3) {
            // columns -> owner (rows_per_rank carries N / P); rows land at this rank's offset
            const int c_owner = col / rows_per_rank;
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(outs.p[c_owner]) + (size_t)(my_rank * M + row) * ldc +
                               (col - c_owner * rows_per_rank);
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
          } else if (MODE != 1) {
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
          } else if (RED_BF16) {
            __nv_bfloat16* dst = red_row_h + col;
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst + 8 * j),
                             "r"(pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]))),
                             "r"(pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]))),
                             "r"(pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]))),
                             "r"(pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])))
                             : "memory");
              }
            } else {
              for (int j = 0; j + 1 < 32; j += 2) {
                if (col + j + 1 < N) {
                  asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(dst + j),
                               "r"(pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1])))
                               : "memory");
                } else if (col + j < N) {
                  asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(dst + j), "r"(pack_bf16(__uint_as_float(r[j]), 0.f))
                               : "memory");
                }
              }
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
    if (MODE == 1 || MODE == 3) __threadfence_system();  // peer writes ordered before the closing barrier
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool B_MN, int MODE, bool RED_BF16>
static int launch_gc(void* const* a_ptrs, const void* B, void* C, void* const* out_ptrs, int M, int N, int K, int lda, int ldb,
                     int ldc, int rows_per_rank, int my_rank, int P, void* gathered, int* flags, int epoch, cudaStream_t stream) {
  using Cfg = GcCfg<BN>;
  TmapArray ta;
  CUtensorMap tmG;
  GatherArgs ga = {};
  int rc;
  int nA = 1;
  if (MODE == 0) {
    nA = P;
    for (int r = 0; r < P; ++r) {
      rc = ab2host::encode_tmap_2d(&ta.m[r], a_ptrs[r], 2, (uint64_t)K, (uint64_t)rows_per_rank, (uint64_t)lda * 2, GC_BK, GC_BM, true, 0);
      if (rc) return 100 + rc;
    }
  } else if (MODE == 1 || MODE == 3) {
    rc = ab2host::encode_tmap_2d(&ta.m[0], a_ptrs[0], 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, GC_BK, GC_BM, true, 0);
    if (rc) return 100 + rc;
  } else if (MODE == 4) {
    // rows_per_rank carries K / P: every rank holds a [P * M, K / P] column panel
    nA = P;
    for (int r = 0; r < P; ++r) {
      rc = ab2host::encode_tmap_2d(&ta.m[r], a_ptrs[r], 2, (uint64_t)rows_per_rank, (uint64_t)P * M, (uint64_t)lda * 2, GC_BK, GC_BM, true, 0);
      if (rc) return 100 + rc;
    }
    rc = ab2host::encode_tmap_2d(&tmG, gathered, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, GC_BK, GC_BM, true, 0);
    if (rc) return 110 + rc;
    ga.gathered = reinterpret_cast<__nv_bfloat16*>(gathered);
    ga.flags = flags;
    ga.epoch = epoch;
    ga.lda = lda;
  } else {
    nA = P;
    for (int r = 0; r < P; ++r) {
      rc = ab2host::encode_tmap_2d(&ta.m[r], a_ptrs[r], 2, (uint64_t)K, (uint64_t)rows_per_rank, (uint64_t)lda * 2, GC_BK, GC_BM, true, 0);
      if (rc) return 100 + rc;
    }
    rc = ab2host::encode_tmap_2d(&tmG, gathered, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, GC_BK, GC_BM, true, 0);
    if (rc) return 110 + rc;
    for (int r = 0; r < GC_MAX_PEERS; ++r) ga.peer_a[r] = r < P ? reinterpret_cast<const __nv_bfloat16*>(a_ptrs[r]) : nullptr;
    ga.gathered = reinterpret_cast<__nv_bfloat16*>(gathered);
    ga.flags = flags;
    ga.epoch = epoch;
    ga.lda = lda;
  }
  for (int r = nA; r < GC_MAX_PEERS; ++r) ta.m[r] = ta.m[0];
  if (MODE != 2 && MODE != 4) tmG = ta.m[0];
  CUtensorMap tmB;
  if (!B_MN)
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, GC_BK, BN, true, 0);
  else
    rc = ab2host::encode_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, GC_BK, true, 0);
  if (rc) return 200 + rc;
  OutPtrs op;
  for (int r = 0; r < GC_MAX_PEERS; ++r) op.p[r] = ((MODE == 1 || MODE == 3) && r < P) ? out_ptrs[r] : nullptr;
  auto kern = gemm_comm_kernel<BN, B_MN, MODE, RED_BF16>;
  static ab2host::DevState dev_state;
  int num_sms = 0;
  if (ab2host::prepare_launch(kern, Cfg::SMEM_BYTES, dev_state, &num_sms)) return 300;
  (void)num_sms;
  const int tiles = ((M + GC_BM - 1) / GC_BM) * ((N + BN - 1) / BN);
  int grid = tiles < num_sms ? tiles : num_sms;
  if (MODE == 2 || MODE == 4) {
    // copy CTAs and compute CTAs must all be resident at once: the compute side waits on flags
    // that the copy side sets
    ga.n_copy = P > 1 ? (num_sms >= 64 ? 8 : 2) : 0;
    grid = num_sms;
    if (tiles + ga.n_copy < grid) grid = tiles + ga.n_copy;
  }
  int* err = ab2host::error_flag();
  if (!err) return 301;
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(ta, tmB, tmG, reinterpret_cast<__nv_bfloat16*>(C), op, ga, M, N, K, ldc, rows_per_rank,
                                               my_rank, P, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 302;
}

template <int MODE, bool RED_BF16>
static int dispatch_gc(int bn, int b_mn, void* const* a_ptrs, const void* B, void* C, void* const* out_ptrs, int M, int N, int K,
                       int lda, int ldb, int ldc, int rpr, int me, int P, void* gathered, int* flags, int epoch, cudaStream_t s) {
  if (bn == 256) {
    return b_mn ? launch_gc<256, true, MODE, RED_BF16>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, gathered, flags, epoch, s)
                : launch_gc<256, false, MODE, RED_BF16>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, gathered, flags, epoch, s);
  }
  return b_mn ? launch_gc<128, true, MODE, RED_BF16>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, gathered, flags, epoch, s)
              : launch_gc<128, false, MODE, RED_BF16>(a_ptrs, B, C, out_ptrs, M, N, K, lda, ldb, ldc, rpr, me, P, gathered, flags, epoch, s);
}

}  // namespace ab2

extern "C" {

// C[M, N] (bf16, local) = concat_r(A_r)[M, K] * op(B). a_ptrs[r]: rank r's [M/P, K] block (lda
// elements per row) as mapped into this process; rows_per_rank = M / P must be a multiple of
// 128. b_mn = 0: B is [N, K]; 1: B is [K, N].
// gathered == null: remote tiles are loaded by TMA straight from the owner's memory (every
// output-tile column re-reads them over NVLink). gathered != null (local [M, K] bf16) with
// flags (int32 per 128-row block) and a per-call epoch that differs from every earlier one:
// copy CTAs bring each remote block over once and the tiles read the local copy.
int ab2_allgather_gemm(void* const* a_ptrs, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int b_mn,
                       int my_rank, int world, void* gathered, void* flags, int epoch, void* stream) {
  using namespace ab2;
  if (world < 1 || world > GC_MAX_PEERS) return 10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M % world || (M / world) % GC_BM) return 11;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (K & 7)) return 12;
  const int bn = (N % 256 == 0 && ((M + 127) / 128) * (N / 256) >= 120) ? 256 : 128;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gathered != nullptr) {
    if (!flags) return 13;
    return dispatch_gc<2, false>(bn, b_mn, a_ptrs, B, C, nullptr, M, N, K, lda, ldb, ldc, M / world, my_rank, world, gathered,
                                 reinterpret_cast<int*>(flags), epoch, s);
  }
  return dispatch_gc<0, false>(bn, b_mn, a_ptrs, B, C, nullptr, M, N, K, lda, ldb, ldc, M / world, my_rank, world, nullptr, nullptr, 0, s);
}

// out_r[M/P, N] (rank r's buffer as mapped here, ldc elements per row) += rows r of A * op(B).
// out_bf16 = 0: fp32 buffers and fp32 reductions; 1: bf16 buffers, bf16x2 reductions (half the
// NVLink bytes; every add rounds to bf16, meant for small groups). All buffers must be zero (or
// hold the value to add to) and visible before any rank launches; results are complete after
// a barrier that follows every rank's kernel.
// Ulysses seq->heads fused into the projection: Y = A[M, K] * op(B) (N columns) is never stored
// locally; columns [r * N/P, (r+1) * N/P) go to rank r's buffer out_ptrs[r] ([P * M, N / P] bf16,
// ld_out elements per row) at rows [my_rank * M, (my_rank + 1) * M). N / P must be a multiple of 32.
int ab2_gemm_scatter_cols(const void* A, const void* B, void* const* out_ptrs, int M, int N, int K, int lda, int ldb, int ld_out,
                          int b_mn, int my_rank, int world, void* stream) {
  using namespace ab2;
  if (world < 1 || world > GC_MAX_PEERS) return 10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % world || (N / world) % 32) return 11;
  if ((lda & 7) || (ldb & 7) || (ld_out & 7)) return 12;
  const int bn = (N % 256 == 0 && ((M + 127) / 128) * (N / 256) >= 120) ? 256 : 128;
  void* a1[1] = {const_cast<void*>(A)};
  return dispatch_gc<3, false>(bn, b_mn, a1, B, nullptr, out_ptrs, M, N, K, lda, ldb, ld_out, N / world, my_rank, world, nullptr, nullptr,
                               0, reinterpret_cast<cudaStream_t>(stream));
}

// Ulysses heads->seq fused into the output projection: C[M, N] (bf16, local) = A * op(B) where
// A[M, K] is this rank's M rows of every rank's column panel: a_ptrs[r] is rank r's
// [P * M, K / P] buffer (lda elements per row) as mapped here; this rank's rows start at
// my_rank * M. K / P must be a multiple of 64, M of 128. gathered: local [M, K] bf16 scratch;
// flags: int32[(M / 128) * P]; epoch: differs from every earlier call on these flags.
int ab2_gather_cols_gemm(void* const* a_ptrs, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int b_mn,
                         int my_rank, int world, void* gathered, void* flags, int epoch, void* stream) {
  using namespace ab2;
  if (world < 1 || world > GC_MAX_PEERS) return 10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % world || (K / world) % GC_BK || M % GC_BM) return 11;
  if ((lda & 7) || (ldb & 7) || (ldc & 7)) return 12;
  if (!gathered || !flags) return 13;
  const int bn = (N % 256 == 0 && ((M + 127) / 128) * (N / 256) >= 120) ? 256 : 128;
  return dispatch_gc<4, false>(bn, b_mn, a_ptrs, B, C, nullptr, M, N, K, lda, ldb, ldc, K / world, my_rank, world, gathered,
                               reinterpret_cast<int*>(flags), epoch, reinterpret_cast<cudaStream_t>(stream));
}

int ab2_gemm_reduce_scatter(const void* A, const void* B, void* const* out_ptrs, int M, int N, int K, int lda, int ldb, int ldc,
                            int b_mn, int my_rank, int world, int out_bf16, void* stream) {
  using namespace ab2;
  if (world < 1 || world > GC_MAX_PEERS) return 10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M % world || (M / world) % GC_BM) return 11;
  if ((lda & 7) || (ldb & 7) || (ldc & (out_bf16 ? 7 : 3))) return 12;
  const int bn = (N % 256 == 0 && ((M + 127) / 128) * (N / 256) >= 120) ? 256 : 128;
  void* a1[1] = {const_cast<void*>(A)};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (out_bf16)
    return dispatch_gc<1, true>(bn, b_mn, a1, B, nullptr, out_ptrs, M, N, K, lda, ldb, ldc, M / world, my_rank, world, nullptr, nullptr, 0, s);
  return dispatch_gc<1, false>(bn, b_mn, a1, B, nullptr, out_ptrs, M, N, K, lda, ldb, ldc, M / world, my_rank, world, nullptr, nullptr, 0, s);
}
}
