// Host-side plumbing shared by the .cu files: error recording, the per-device status word,
// device checks and TMA descriptor (CUtensorMap) construction through the driver entry point.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/trinity_b200.h"

namespace trn {

// records the CUDA error text for trinity_last_cuda_error(); returns TRN_E_CUDA
int record_cuda_error(cudaError_t e, const char* where);
int record_driver_error(CUresult r, const char* where);

#define TRN_CUDA_TRY(expr)                                          \
  do {                                                              \
    cudaError_t _e = (expr);                                        \
    if (_e != cudaSuccess) return ::trn::record_cuda_error(_e, #expr); \
  } while (0)

// Per-device state created on first use (make that first call outside stream capture: it looks up the
// address of the status word, a __device__ variable of the library, with cudaGetSymbolAddress).
struct DeviceState {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int* status = nullptr;   // device int, zero-initialised
};
// returns TRN_OK and fills *out, or an error code (TRN_E_DEVICE when not sm_100)
int get_device_state(DeviceState** out);

// Tiled tensor map over a tensor of 16-bit elements with up to 4 dims (dim 0 contiguous),
// 128-byte swizzle, zero fill outside the tensor.
//   dims[i]    extent of dim i (elements)
//   strides[i] stride of dim i in ELEMENTS for i >= 1 (dim 0 has stride 1)
//   box[i]     tile extent of dim i
int make_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                    const uint32_t* box);

// opts a kernel in to `bytes` of dynamic shared memory, once per (kernel, device)
int ensure_dyn_smem(const void* kernel, int bytes, int device);

// Launch with the programmatic-stream-serialization attribute (see griddep_wait in common.cuh): the kernel may begin
// its prologue before the previous kernel of the stream has finished; capturable in CUDA graphs.  TRINITY_NO_PDL=1
// in the environment makes these plain launches.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// launchers implemented per kernel family
int launch_rmsnorm(const TrnRmsArgs& a, cudaStream_t st, const DeviceState& ds);
int launch_qkv_project(const TrnProjArgs& a, cudaStream_t st, const DeviceState& ds);
int launch_lora(const TrnLoraArgs& a, cudaStream_t st, const DeviceState& ds);
int launch_gmlp(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds);
// at most 16 tokens: one latency-oriented launch (gmlp_small.cu); callers validate the arguments first
bool gmlp_small_applies(const TrnGmlpArgs& a);
int launch_gmlp_small(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds);
// at most 16 tokens: one latency-oriented launch (lora_small.cu); callers validate the arguments first
bool lora_small_applies(const TrnLoraArgs& a);
int launch_lora_small(const TrnLoraArgs& a, cudaStream_t st, const DeviceState& ds);
// Per-key statistics a caller would take from the attention pass's scores right afterwards (trinity_attn_colstats on
// the perturbed scores when the launch carries noise, else on the plain ones).  With `fused` given, launch_attention
// computes them in the same launch when the shape allows and sets done = 1; otherwise it leaves done = 0 and the caller
// runs the statistics kernel.
struct AttnFusedStats {
  void* sum_p;
  void* sum_p2;    // or nullptr
  int stats_fp32;
  int done;
};
int launch_attention(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds, AttnFusedStats* fused = nullptr);
// attention with at most 16 queries per head: one latency-oriented launch (attn_small.cu); launch_attention validates
// the arguments and routes here
bool attn_small_applies(const TrnAttnArgs& a);
bool attn_small_stats_applies(const TrnAttnArgs& a, int sm_count);
int launch_attn_small(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds, const AttnFusedStats* fs = nullptr);
// split-KV policy of the attention kernel: how many CTAs share one tile pair's key range (1: no split),
// and the scratch a launch of that shape wants for the partial results (0: it would not split)
constexpr int kAttnMaxSplits = 8;
constexpr int kAttnNominalSMs = 148;     // sizing only: the launch itself uses the device's SM count
int attn_split_count(int ctas, int L, int sm_count);
size_t attn_split_workspace(int B, int M, int P, int Hq, int Hkv, int D, int sm_count);
// the split count a launch of this shape picks when its workspace is large enough
int attn_planned_splits(int B, int M, int P, int Hq, int Hkv, int D, int causal, int sm_count);
// > 0: attention launches made by this thread use exactly this many splits (workspace permitting) instead
// of their own choice; set by callers that cut one problem into several launches and want each output
// element computed as the uncut launch would
extern thread_local int tls_attn_split_override;
// smallest workspace trinity_attn_block accepts (its optional split-KV area excluded)
size_t block_workspace_required(const TrnBlockArgs& a);
int launch_colstats(const TrnColStatsArgs& a, cudaStream_t st, const DeviceState& ds);
int launch_topk(const TrnTopkArgs& a, cudaStream_t st, const DeviceState& ds);
int launch_convert(const void* src, void* dst, long long n, int dtype16, int to_fp32, cudaStream_t st,
                   const DeviceState& ds);

}  // namespace trn
