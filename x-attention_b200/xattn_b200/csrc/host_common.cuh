// Host-side helpers shared by the launchers: status codes, TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), device checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <utility>

#include "../../../include/xattn_b200.h"

namespace xb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 16-bit tensor seen as up to 5 dimensions, innermost first.  `strides_bytes` has rank-1 entries
// (the innermost stride is one element).  128-byte swizzle, zero fill outside the tensor.
inline int make_tmap_16bit(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return XATTN_B200_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return XATTN_B200_ERR_ARG;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      if (strides_bytes[i - 1] % 16 != 0 || strides_bytes[i - 1] == 0) return XATTN_B200_ERR_ARG;
      gstr[i - 1] = strides_bytes[i - 1];
    }
  }
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                   gdim, gstr, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? XATTN_B200_OK : XATTN_B200_ERR_CUDA;
}

inline int check_sm100() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return XATTN_B200_ERR_CUDA;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return XATTN_B200_ERR_CUDA;
  return major == 10 ? XATTN_B200_OK : XATTN_B200_ERR_ARCH;
}

inline int sm_count() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

// Kernel launches issued by this library in this process (every launcher calls launch_status() right after its
// <<<>>>): a diagnostic the benchmark reads through xattn_b200_launch_count().
inline std::atomic<unsigned long long>& launch_counter() {
  static std::atomic<unsigned long long> n{0};
  return n;
}

inline int launch_status() {
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? XATTN_B200_OK : XATTN_B200_ERR_CUDA;
}

// Launches `kernel` so that it may start while the kernel before it in the stream is still running (programmatic
// stream serialization): the kernel must execute pdl_wait() before it touches anything that kernel writes.
template <typename... KArgs, typename... Args>
inline int launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream,
                            Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? XATTN_B200_OK : XATTN_B200_ERR_CUDA;
}

}  // namespace xb
