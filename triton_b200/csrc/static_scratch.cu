// trinity_attn_block_static: the whole attention block for callers that can hand over inputs and outputs
// but no scratch buffer and must not allocate one — a plugin whose host runtime gives it only the tensors of
// the operator, or a serving loop that forbids device allocation after start-up because cudaMalloc
// synchronises the device and stalls every other stream.
//
// The scratch the block needs (per-row RMS scales and the two log-sum-exp arrays, all fp32) lives in a
// file-scope device array of fixed size instead of a caller workspace.  Every GPU that loads this library
// holds that array (kStaticScratchBytes) until the process exits.
#include <mutex>

#include "host.h"

namespace trn {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB: B*M*(1 + 2*Hq) fp32 values up to ~2 M

// Device storage.  In host code this name is only a handle for the runtime: it is NOT a device address and
// must never be passed to a kernel; the address is looked up per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDev = 64;
void* g_scratch_ptr[kMaxDev] = {};
std::mutex g_scratch_mu;

// once per device, with that device current
int static_scratch_address(void** out) {
  int dev = -1;
  TRN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) return TRN_E_DEVICE;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return record_cuda_error(e, "cudaGetSymbolAddress(static scratch)");
    if (p == nullptr) return TRN_E_CUDA;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return TRN_OK;
}

}  // namespace
}  // namespace trn

using namespace trn;

extern "C" size_t trinity_static_scratch_capacity(void) { return kStaticScratchBytes; }

extern "C" int trinity_attn_block_static(const TrnBlockArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  if (trinity_attn_block_workspace(a) == 0) return TRN_E_SHAPE;
  // the optional split-KV area is used as far as the array reaches; only the required part must fit
  const size_t need = block_workspace_required(*a);
  if (need > kStaticScratchBytes) return TRN_E_STATIC_SCRATCH;   // too large for the built-in scratch
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != TRN_OK) return rc;
  // Same block, same kernels; only the workspace pointer differs.  Nothing in the scratch has to start at
  // zero: row scales and log-sum-exp values are written for every valid row before they are read.
  TrnBlockArgs b = *a;
  b.workspace = scratch;
  b.workspace_bytes = kStaticScratchBytes;
  return trinity_attn_block(&b, cuda_stream);
}
