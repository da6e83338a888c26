// Mixture-of-experts routing on the device: from the router logits to everything the expert
// GEMMs need, without a host read.
//
//   moe_topk      one warp per token: softmax / sigmoid scores in fp32, optional selection bias,
//                 top-k by k rounds of a warp arg-max (ties go to the lower expert id), optional
//                 renormalisation and scaling of the chosen weights.
//   moe_count     per-chunk histogram of the chosen experts (a chunk is CHUNK consecutive
//                 (token, slot) entries).
//   moe_scan      one block: expert totals, expert offsets, the chunk offsets that make the
//                 placement stable, and the table of 128-row tiles (expert, first row, valid rows)
//                 with its length for the grouped GEMM.
//   moe_place     one warp per chunk: every entry gets its row in the expert-sorted order; equal
//                 experts keep token order (a stable counting sort: same result run after run).
//
// Takes the place of softmax + torch.topk + argsort + bincount + the host copy of the counts in the
// reference's router and token re-orderer (areal/experimental/models/archon/moe/router.py:234-297,
// areal/experimental/models/archon/moe/utils.py permutation helpers).
#include "common.cuh"

namespace ab2 {

static constexpr int ROUTE_CHUNK = 2048;
static constexpr int ROUTE_MAX_E = 256;
static constexpr int ROUTE_MAX_K = 16;

__global__ void __launch_bounds__(256)
moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ probs,
                float* __restrict__ topw, int* __restrict__ tope, int T, int E, int k, int use_sigmoid, int norm,
                float scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  constexpr int PER = ROUTE_MAX_E / 32;
  float p[PER], c[PER];
  const float* row = logits + (size_t)t * E;
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = j * 32 + lane;
    p[j] = e < E ? row[e] : -INFINITY;
    m = fmaxf(m, p[j]);
  }
  if (use_sigmoid) {
#pragma unroll
    for (int j = 0; j < PER; ++j) p[j] = (j * 32 + lane) < E ? 1.f / (1.f + expf(-p[j])) : 0.f;
  } else {
    m = warp_max(m);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      p[j] = (j * 32 + lane) < E ? expf(p[j] - m) : 0.f;
      s += p[j];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < PER; ++j) p[j] *= inv;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = j * 32 + lane;
    if (e < E) {
      if (probs) probs[(size_t)t * E + e] = p[j];
      c[j] = bias ? p[j] + bias[e] : p[j];
    } else {
      c[j] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;      // lane i keeps the weight of the i-th choice
  int my_e = 0;
  for (int i = 0; i < k; ++i) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (c[j] > bv) { bv = c[j]; be = j * 32 + lane; }        // ascending j: the lowest id wins a tie inside the lane
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    if (be == 0x7fffffff) be = i;                              // every score was NaN / -inf: still name k distinct experts
    const int owner = be & 31, slot = be >> 5;
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j == slot && lane == owner) { w = p[j]; c[j] = -INFINITY; }
    w = __shfl_sync(0xffffffffu, w, owner);
    wsum += w;
    if (lane == i) { my_w = w; my_e = be; }
  }
  if (lane < k) {
    float w = my_w;
    if (norm) w = w / fmaxf(wsum, 1e-20f);
    topw[(size_t)t * k + lane] = w * scale;
    tope[(size_t)t * k + lane] = my_e;
  }
}

// chunkcnt[chunk][e]: entries of the chunk that chose expert e.
__global__ void __launch_bounds__(256)
moe_count_kernel(const int* __restrict__ tope, int n_entries, int E, int* __restrict__ chunkcnt) {
  __shared__ int hist[ROUTE_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int lo = blockIdx.x * ROUTE_CHUNK;
  const int hi = min(n_entries, lo + ROUTE_CHUNK);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const int e = tope[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) chunkcnt[(size_t)blockIdx.x * E + e] = hist[e];
}

// One block of ROUTE_MAX_E threads; thread e owns expert e. On return chunkcnt[chunk][e] holds the row at
// which the chunk's first entry for expert e lands; counts / offs (E + 1 entries) / row tiles are filled.
__global__ void __launch_bounds__(ROUTE_MAX_E)
moe_scan_kernel(int* __restrict__ chunkcnt, int n_chunks, int E, int* __restrict__ counts, int* __restrict__ offs,
                int4* __restrict__ row_tiles, int* __restrict__ num_row_tiles, int max_row_tiles) {
  __shared__ int s_cnt[ROUTE_MAX_E];
  __shared__ int s_off[ROUTE_MAX_E + 1];
  __shared__ int s_tile[ROUTE_MAX_E + 1];
  const int e = threadIdx.x;
  int total = 0;
  if (e < E) {
    for (int b = 0; b < n_chunks; ++b) {
      const int c = chunkcnt[(size_t)b * E + e];
      chunkcnt[(size_t)b * E + e] = total;       // rank of the chunk's first entry inside the expert's group
      total += c;
    }
    s_cnt[e] = total;
    counts[e] = total;
  }
  __syncthreads();
  if (e == 0) {
    int o = 0, tl = 0;
    for (int i = 0; i < E; ++i) {
      s_off[i] = o;
      s_tile[i] = tl;
      o += s_cnt[i];
      tl += (s_cnt[i] + 127) >> 7;
    }
    s_off[E] = o;
    s_tile[E] = tl;
    *num_row_tiles = tl < max_row_tiles ? tl : max_row_tiles;
  }
  __syncthreads();
  if (e < E) {
    const int o = s_off[e];
    offs[e] = o;
    if (e == 0) offs[E] = s_off[E];
    for (int b = 0; b < n_chunks; ++b) chunkcnt[(size_t)b * E + e] += o;
    const int n = s_cnt[e];
    int tl = s_tile[e];
    for (int r0 = 0; r0 < n && tl < max_row_tiles; r0 += 128, ++tl)
      row_tiles[tl] = make_int4(e, o + r0, min(128, n - r0), 0);
  }
}

// order[row] = entry (token * k + slot) that lands on that row; token_of[row] = its token; inv[entry] = row.
__global__ void __launch_bounds__(32)
moe_place_kernel(const int* __restrict__ tope, int n_entries, int E, int k, const int* __restrict__ chunkoff,
                 int* __restrict__ order, int* __restrict__ token_of, int* __restrict__ inv) {
  __shared__ int base[ROUTE_MAX_E];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) base[e] = chunkoff[(size_t)blockIdx.x * E + e];
  __syncwarp();
  const int lo = blockIdx.x * ROUTE_CHUNK;
  const int hi = min(n_entries, lo + ROUTE_CHUNK);
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    int e = i < hi ? tope[i] : -1;
    if (e >= E) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    int pos = -1;
    if (e >= 0) pos = base[e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) base[e] += __popc(same);
    __syncwarp();
    if (pos >= 0) {
      order[pos] = i;
      token_of[pos] = i / k;
      inv[i] = pos;
    }
  }
}

}  // namespace ab2

extern "C" {

// Number of ints the caller must provide as `workspace` for n_entries = T * k entries over E experts.
long long ab2_moe_route_workspace(long long n_entries, int E) {
  const long long chunks = (n_entries + ab2::ROUTE_CHUNK - 1) / ab2::ROUTE_CHUNK;
  return (chunks > 0 ? chunks : 1) * E;
}

// logits [T, E] fp32; bias [E] fp32 or null (added for the choice only). flags: bit 0 sigmoid scores,
// bit 1 renormalise the chosen weights, bit 2 tope is given (skip the selection; topw / probs untouched).
// Outputs: probs [T, E] (nullable), topw [T, k] fp32, tope [T, k] int32, counts [E], offs [E + 1],
// order / token_of [T * k], inv [T * k], row_tiles [max_row_tiles] int4, num_row_tiles [1].
int ab2_moe_route(const void* logits, const void* bias, int T, int E, int k, int flags, float scale, void* probs, void* topw,
                  void* tope, void* counts, void* offs, void* order, void* token_of, void* inv, void* row_tiles,
                  void* num_row_tiles, int max_row_tiles, void* workspace, void* stream) {
  using namespace ab2;
  if (T <= 0) return 0;
  if (E <= 0 || E > ROUTE_MAX_E || k <= 0 || k > ROUTE_MAX_K || k > E) return 10;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long n_entries_ll = (long long)T * k;
  if (n_entries_ll > 0x7fffffffLL) return 11;
  const int n_entries = (int)n_entries_ll;
  const int chunks = (n_entries + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  if (!(flags & 4)) {
    const int warps = 8;
    moe_topk_kernel<<<(T + warps - 1) / warps, warps * 32, 0, s>>>(
        reinterpret_cast<const float*>(logits), reinterpret_cast<const float*>(bias), reinterpret_cast<float*>(probs),
        reinterpret_cast<float*>(topw), reinterpret_cast<int*>(tope), T, E, k, flags & 1, (flags >> 1) & 1, scale);
  }
  moe_count_kernel<<<chunks, 256, 0, s>>>(reinterpret_cast<const int*>(tope), n_entries, E, reinterpret_cast<int*>(workspace));
  moe_scan_kernel<<<1, ROUTE_MAX_E, 0, s>>>(reinterpret_cast<int*>(workspace), chunks, E, reinterpret_cast<int*>(counts),
                                            reinterpret_cast<int*>(offs), reinterpret_cast<int4*>(row_tiles),
                                            reinterpret_cast<int*>(num_row_tiles), max_row_tiles);
  moe_place_kernel<<<chunks, 32, 0, s>>>(reinterpret_cast<const int*>(tope), n_entries, E, k,
                                         reinterpret_cast<const int*>(workspace), reinterpret_cast<int*>(order),
                                         reinterpret_cast<int*>(token_of), reinterpret_cast<int*>(inv));
  return cudaGetLastError() == cudaSuccess ? 0 : 20;
}
}
