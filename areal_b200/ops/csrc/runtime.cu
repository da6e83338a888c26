// Host-side runtime shared by all kernels of the library: per-device error word,
// TMA tensor-map encoding through the driver entry point (no link-time libcuda
// dependency), and a few exported C helpers.
#include <cstdlib>
#include <cudaTypedefs.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace ab2host {

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e == cudaSuccess && q == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

// Driver entry points need a context bound to the calling thread; threads that have only
// seen the runtime API lazily (e.g. autograd worker threads) may not have one yet.
static void bind_context_once() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(0);
    bound = true;
  }
}

static CUtensorMapDataType dtype_of(int code) {
  switch (code) {
    case 0: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case 1: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case 2: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case 3: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                   uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                   uint32_t box_outer, bool swizzle128, int dtype_code) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  bind_context_once();
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, dtype_of(dtype_code), 2, const_cast<void*>(base), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_bytes;
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int encode_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1,
                   uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0,
                   uint32_t b1, uint32_t b2, bool swizzle128, int dtype_code) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  bind_context_once();
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, dtype_of(dtype_code), 3, const_cast<void*>(base), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_bytes;
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int* g_err[64] = {nullptr};
static std::mutex g_err_mu;

int* error_flag() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_err_mu);
  if (!g_err[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    g_err[dev] = p;
  }
  return g_err[dev];
}

bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("AB2_PDL"); return e && e[0] == '1'; }();
  return on;
}

}  // namespace ab2host

extern "C" {

// Reads (and clears) the current device's kernel error word. Synchronises the device.
// 0 = no error; otherwise an ab2::KernelError code recorded by a bounded wait that gave up.
int ab2_kernel_error() {
  int* p = ab2host::error_flag();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// Enqueues on `stream` a copy of the current device's error word into `host_word` (pinned host
// memory owned by the caller). The caller reads host_word after its next synchronisation of that
// stream: a step loop that already synchronises once per step learns of a wait that gave up
// without paying for a second synchronisation.
int ab2_kernel_error_peek(int* host_word, void* stream) {
  int* p = ab2host::error_flag();
  if (!p || !host_word) return -1;
  return cudaMemcpyAsync(host_word, p, sizeof(int), cudaMemcpyDeviceToHost, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : -2;
}

// Allocates the error word of the current device ahead of time (call once per device
// before capturing CUDA graphs).
int ab2_runtime_init() { return ab2host::error_flag() ? 0 : -1; }

int ab2_num_sms() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

const char* ab2_build_info() { return "areal_b200 kernels, sm_100a, tcgen05+TMA"; }
}
