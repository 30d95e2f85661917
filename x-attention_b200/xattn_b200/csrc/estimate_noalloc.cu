// xattn_b200_estimate_static: the block-importance estimate for callers that cannot hand over
// scratch memory of their own.
//
// Some hosts of this library may not allocate device memory at the point where they call it: a serving
// process whose memory pool was carved up at start-up and is owned by another component, a plugin
// loaded into a runtime that forbids cudaMalloc after initialisation, a caller inside a latency-critical
// section where an allocation (which may synchronise the device) is unacceptable.  The regular estimate
// needs a workspace from the caller; this variant brings its own, a fixed array that is part of the
// library image, so the only memory the caller supplies is the inputs and the output.
//
// The array costs XATTN_B200_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library,
// from load until the process exits, whether or not this entry point is ever called.  It is therefore
// kept modest: enough for, e.g., 8 query heads at 32K tokens with stride 8, or 32 heads at 8K.
// Larger problems are refused with XATTN_B200_ERR_LIMIT; use xattn_b200_estimate with a workspace.
#include "host_common.cuh"

namespace xb {
size_t estimate_workspace_bytes(int batch, int hq, int q_len, int k_len, int stride, int block_size, int chunk_size,
                                int causal, int semantics);
int estimate_launch(const void* q, const void* k, int dtype, int batch, int hq, int hkv, int q_len, int k_len,
                    int head_dim, int64_t qsb, int64_t qsh, int64_t qsl, int64_t ksb, int64_t ksh, int64_t ksl,
                    int stride, int block_size, int chunk_size, float scale, int causal, int semantics,
                    float* attn_sums, void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream);
}  // namespace xb

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table, not an
// address a kernel could use; the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[XATTN_B200_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

// Look up (first call on this device) or return the device address of the scratch array.  The device whose
// address is wanted must be current.  Two threads making the first call at once both store the same value.
// The address belongs to the device's primary context: an application that resets the device
// (cudaDeviceReset) must not use this entry point again in the same process.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return XATTN_B200_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return XATTN_B200_ERR_LIMIT;
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return XATTN_B200_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return XATTN_B200_OK;
}
}  // namespace

extern "C" int xattn_b200_estimate_static(const void* q, const void* k, int dtype, int batch, int hq, int hkv,
                                          int q_len, int k_len, int head_dim, int64_t q_stride_b,
                                          int64_t q_stride_h, int64_t q_stride_l, int64_t k_stride_b,
                                          int64_t k_stride_h, int64_t k_stride_l, int stride, int block_size,
                                          int chunk_size, float scale, int causal, int semantics, float* attn_sums,
                                          int* status, void* cuda_stream) {
  const size_t need = xb::estimate_workspace_bytes(batch, hq, q_len, k_len, stride, block_size, chunk_size,
                                                   causal ? 1 : 0, semantics);
  if (need == 0) return XATTN_B200_ERR_ARG;
  if (need > static_cast<size_t>(XATTN_B200_STATIC_SCRATCH_BYTES)) return XATTN_B200_ERR_LIMIT;
  int rc = xb::check_sm100();                       // a foreign device is an architecture error, not a CUDA error
  if (rc != XATTN_B200_OK) return rc;
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc != XATTN_B200_OK) return rc;
  // Nothing in the scratch has to start at zero: the tile tables, the per-tile maxima and the partial
  // sums are all written by this call's kernels before this call's kernels read them.
  return xb::estimate_launch(q, k, dtype, batch, hq, hkv, q_len, k_len, head_dim, q_stride_b, q_stride_h,
                             q_stride_l, k_stride_b, k_stride_h, k_stride_l, stride, block_size, chunk_size, scale,
                             causal, semantics, attn_sums, scratch, static_cast<size_t>(XATTN_B200_STATIC_SCRATCH_BYTES),
                             status, static_cast<cudaStream_t>(cuda_stream));
}
