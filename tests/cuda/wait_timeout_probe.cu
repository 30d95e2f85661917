// Test-only kernel: makes a bounded device-side wait run out and checks that the abort protocol of the library's
// kernels does what it promises -- every role gives up, the CTA reaches its teardown, the caller's status word
// receives 101 and the context stays usable.  Built by tests/test_device_wait_timeout.py with a wait limit of
// about a millisecond (-DXB_WAIT_CYCLE_LIMIT=...); nothing here faults, traps or spins without a bound.
#include "sm100_primitives.cuh"

namespace {
__global__ void wait_timeout_probe_kernel(int* status, int* roles_seen) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    xb::mbar_init(xb::smem_u32(&bar), 1);      // one arrival expected, and no thread ever arrives
    abort_word = 0;
    xb::fence_mbar_init();
  }
  __syncthreads();
  // two "roles" (warps) wait for a phase that never completes: the first one to run out of time raises the CTA's
  // abort flag, the other one sees the flag at its next poll
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = xb::mbar_wait(xb::smem_u32(&bar), 0, abort_flag);
  if (!ok) atomicAdd(roles_seen, 1);
  __syncthreads();                              // the common teardown every role falls through to
  if (*abort_flag && threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(xb::kDevWaitTimeout));
}
}  // namespace

extern "C" int wait_timeout_probe(int* status, int* roles_seen, void* stream) {
  wait_timeout_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, roles_seen);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
