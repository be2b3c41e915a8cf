// Host-side TMA tensor-map encoding.  cuTensorMapEncodeTiled is fetched through the runtime's
// driver entry point query, so the library does not link against libcuda directly.  Maps are
// encoded per call (about a microsecond) and passed to kernels as __grid_constant__ parameters;
// nothing is cached on input pointers.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

namespace dsa {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows][inner] of `elem_bytes`-wide elements, box = [box_rows][box_inner],
// 128-byte swizzle (box_inner * elem_bytes must be <= 128), out-of-range elements read as zero.
inline bool make_tmap_2d_sw128(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes,
                               const void* base, uint64_t inner, uint64_t rows, uint32_t box_inner,
                               uint32_t box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {inner * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, type, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Programmatic dependent launch between the kernels of one operator chain is on by default;
// DSA_PDL=0 launches them strictly serialised (use it when timing kernels one by one: with PDL a
// dependent kernel's duration includes the time it waits for its predecessor).
inline int pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("DSA_PDL");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on;
}

constexpr int kMaxDevices = 64;

inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return dev;
}

// SM count of the CURRENT device (one process may drive several GPUs; cached per device).
inline int sm_count() {
  static std::atomic<int> cached[kMaxDevices];
  const int dev = current_device();
  if (dev < 0) return 148;  // no device visible (host-only tooling): plan for a B200
  if (dev < kMaxDevices) {
    const int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 148;
  }
  if (dev < kMaxDevices) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// Opt a kernel in to more than 48 KB of dynamic shared memory.  Function attributes belong to the
// current device's context, so this is remembered per device (`done` is one word per call site:
// bit d = set on device d); devices beyond the mask get the attribute on every launch.
inline cudaError_t opt_in_dynamic_smem(const void* kernel, size_t bytes, std::atomic<uint64_t>& done) {
  const int dev = current_device();
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && ((done.load(std::memory_order_acquire) >> dev) & 1ull)) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && tracked) done.fetch_or(1ull << dev, std::memory_order_release);
  return e;
}

}  // namespace dsa
