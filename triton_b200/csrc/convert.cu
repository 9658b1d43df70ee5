// Element-type conversion between fp32 and the 16-bit io types, for callers whose tensors are fp32 (the
// fp32 Vanilla configuration): inputs are rounded to bf16 / fp16 once, the block runs on the 16-bit
// kernels with fp32 accumulation, and its outputs are widened back.  HBM-bound, 128-bit accesses.
#include "common.cuh"
#include "host.h"

namespace trn {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) narrow_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n8) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i);
    const float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    uint4 o;
    o.x = Io<T>::pack2(a.x, a.y); o.y = Io<T>::pack2(a.z, a.w);
    o.z = Io<T>::pack2(b.x, b.y); o.w = Io<T>::pack2(b.z, b.w);
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) widen_kernel(const T* __restrict__ src, float* __restrict__ dst, long long n8) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    const float2 a = Io<T>::unpack2(v.x), b = Io<T>::unpack2(v.y), c = Io<T>::unpack2(v.z), d = Io<T>::unpack2(v.w);
    reinterpret_cast<float4*>(dst)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
    reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
  }
}

}  // namespace

int launch_convert(const void* src, void* dst, long long n, int dtype16, int to_fp32, cudaStream_t st,
                   const DeviceState& ds) {
  if (n < 0 || (n & 7) != 0) return TRN_E_SHAPE;
  if (n == 0) return TRN_OK;
  if (src == nullptr || dst == nullptr) return TRN_E_NULL;
  if (!aligned16(src) || !aligned16(dst)) return TRN_E_ALIGN;
  const long long n8 = n >> 3;
  long long blocks = (n8 + 255) / 256;
  const long long cap = static_cast<long long>(ds.sm_count) * 8;
  const int grid = static_cast<int>(blocks < cap ? blocks : cap);
  if (dtype16 == TRN_BF16) {
    if (to_fp32) widen_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n8);
    else narrow_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n8);
  } else if (dtype16 == TRN_FP16) {
    if (to_fp32) widen_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(src), static_cast<float*>(dst), n8);
    else narrow_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const float*>(src), static_cast<__half*>(dst), n8);
  } else {
    return TRN_E_DTYPE;
  }
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}

}  // namespace trn
