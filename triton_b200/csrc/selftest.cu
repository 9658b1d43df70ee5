// Self-test of the device-side failure handling every kernel of this library shares: a wait that runs out.
// One thread waits, through the same bounded mbar_wait the kernels use, on an mbarrier that nothing ever arrives
// at.  After `limit_us` the wait gives up: it records KST_TIMEOUT_CONSUMER in the device status word, raises the
// CTA's abort flag, and the kernel falls through the common teardown (which still frees its tensor memory) and
// returns normally — no trap, no endless loop, the context stays usable.  The host then sees TRN_E_KERNEL from
// trinity_last_kernel_status() until trinity_clear_kernel_status() resets the word.
#include "common.cuh"
#include "host.h"

namespace trn {
namespace {

__global__ void __launch_bounds__(64, 1) wait_timeout_selftest_kernel(unsigned long long limit_ns, int* status) {
  __shared__ uint64_t bar_mem;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_mem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  Ctl ctl{status, &abort_flag};
  if (warp == 1) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait(bar, 0, ctl, KST_TIMEOUT_CONSUMER, limit_ns);   // nobody arrives: runs out
    ok = __all_sync(0xffffffffu, ok);
    (void)ok;
  }
  // ---- the teardown every kernel ends with
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 32);
  }
}

}  // namespace
}  // namespace trn

using namespace trn;

extern "C" int trinity_selftest_wait_timeout(int limit_us, void* cuda_stream) {
  if (limit_us < 1 || limit_us > 100000) return TRN_E_SHAPE;     // at most 0.1 s
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<unsigned long long>(limit_us) * 1000ull, ds->status);
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}
