// Allocation-free entry point of the kernel library.
//
// This function has no counterpart in the reference project; it exists for callers of this
// library that are not allowed to allocate device memory at call time: code running inside a
// CUDA-graph capture or a latency-critical serving loop where cudaMalloc would serialise the
// device, plug-ins hosted by a runtime that owns the allocator (so a foreign cudaMalloc /
// torch allocation is forbidden), and embedders that link the .so without PyTorch at all.
//
// Paged decode attention normally needs a split-KV workspace (partial outputs and partial
// max/sum per (sequence, head, split)) that the caller allocates. Here the workspace is a
// fixed array that lives inside the library image on every GPU that loads it (about 8.1 MiB
// per device, held until the process exits), so the caller passes inputs and outputs only.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in workspace covers: B * Hq * num_splits rows of (D + 2) floats,
// with D <= 128.
#define AB2_NOALLOC_MAX_ROWS 16384

// Same computation and argument meaning as ab2_paged_decode(), minus the two workspace
// pointers:
//   q [B, Hq, D] bf16, kc/vc paged caches [slots, Hkv, D] bf16, page_table [B, max_pages]
//   int32, seq_lens [B] int32, out [B, Hq, D] bf16, D in {64, 128}.
// Returns 0 on success; 20 when B * Hq * num_splits exceeds AB2_NOALLOC_MAX_ROWS or D > 128
// (nothing is launched); 21 when the address of the built-in workspace cannot be resolved on
// the current device; other codes as ab2_paged_decode().
//
// Contract:
//  * No cudaMalloc / cudaFree / allocating library call is made, on any call.
//  * The first call on each device resolves the workspace address for that device (the device
//    must be current, as for every call). Make that first call before any stream capture.
//  * All calls on a device share the one workspace and it keeps the previous call's contents.
//    Every slot that a call reads is written earlier in the same call, so nothing has to be
//    cleared in between; but two calls whose kernels overlap in time on the same GPU (different
//    streams, or concurrent graph launches) race on it. Serialise them on one stream.
int ab2_paged_decode_noalloc(const void* q, const void* kc, const void* vc, const int* page_table,
                             const int* seq_lens, void* out, int B, int Hq, int Hkv, int D, int page_size,
                             int max_pages, int num_splits, float scale, void* stream);

#ifdef __cplusplus
}
#endif
