// Standalone RMSNorm, HBM-bound:  y = x * rsqrt(mean(x^2) + eps) * gamma.
// Math follows ref_rms.py:102-103 (eps = 0, no gamma) and ref_attn.py:348-350 (eps, weight).
//
// A row is kept in registers between the reduction and the scaled write (one warp per short row, one
// 256-thread CTA per long row), so each element crosses HBM exactly once in each direction: algorithmic
// bytes per row = 2 * cols * sizeof(elem) (+ gamma once per launch, L2/L1 resident afterwards).
// All global accesses are 128-bit; the row sum of squares is reduced in fp32 with warp shuffles.
#include "common.cuh"
#include "host.h"

namespace trn {

namespace {

constexpr int kWarpsPerCta = 4;

template <typename T, int VPL>   // VPL: 16-byte vectors per lane held in registers
__global__ void __launch_bounds__(kWarpsPerCta * 32)
rmsnorm_rows_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ gamma,
                    float* __restrict__ rstd_out, long long rows, int cols, long long x_stride,
                    long long y_stride, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
  const int nvec = cols >> 3;
  const float inv_cols = 1.0f / static_cast<float>(cols);

  for (long long row = warp0; row < rows; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
    uint4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) v[i] = __ldcs(xr + c);
      else v[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float2 a = Io<T>::unpack2(v[i].x), b = Io<T>::unpack2(v[i].y);
      float2 c = Io<T>::unpack2(v[i].z), d = Io<T>::unpack2(v[i].w);
      ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss);
      ss = fmaf(b.x, b.x, ss); ss = fmaf(b.y, b.y, ss);
      ss = fmaf(c.x, c.x, ss); ss = fmaf(c.y, c.y, ss);
      ss = fmaf(d.x, d.x, ss); ss = fmaf(d.y, d.y, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss * inv_cols + eps);
    if (rstd_out != nullptr && lane == 0) rstd_out[row] = rstd;
    if (y == nullptr) continue;

    uint4* yr = reinterpret_cast<uint4*>(y + row * y_stride);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float2 a = Io<T>::unpack2(v[i].x), b = Io<T>::unpack2(v[i].y);
        float2 cc = Io<T>::unpack2(v[i].z), d = Io<T>::unpack2(v[i].w);
        a.x *= rstd; a.y *= rstd; b.x *= rstd; b.y *= rstd;
        cc.x *= rstd; cc.y *= rstd; d.x *= rstd; d.y *= rstd;
        if (gamma != nullptr) {
          const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
          float2 ga = Io<T>::unpack2(g.x), gb = Io<T>::unpack2(g.y);
          float2 gc = Io<T>::unpack2(g.z), gd = Io<T>::unpack2(g.w);
          a.x *= ga.x; a.y *= ga.y; b.x *= gb.x; b.y *= gb.y;
          cc.x *= gc.x; cc.y *= gc.y; d.x *= gd.x; d.y *= gd.y;
        }
        uint4 o;
        o.x = Io<T>::pack2(a.x, a.y); o.y = Io<T>::pack2(b.x, b.y);
        o.z = Io<T>::pack2(cc.x, cc.y); o.w = Io<T>::pack2(d.x, d.y);
        __stcs(yr + c, o);
      }
    }
  }
}

// Long rows: one CTA of at most 256 threads per row (grid-stride over rows), each thread keeps its 2-4 vectors
// in registers.  Few registers per thread -> full occupancy -> enough 128-bit loads in flight per SM
// to cover HBM latency; one __syncthreads per row (the per-warp partial sums are double-buffered).
// The CTA has just enough warps for the row's vectors at VPT per thread (4 544 columns = 568 vectors: 192 threads x 3
// instead of 256 x 3 with the third pass three-quarters empty).
constexpr int kRowCtaThreads = 256;

template <typename T, int VPT>   // VPT: 16-byte vectors per thread
__global__ void __launch_bounds__(kRowCtaThreads)
rmsnorm_cta_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ gamma,
                   float* __restrict__ rstd_out, long long rows, int cols, long long x_stride,
                   long long y_stride, float eps) {
  griddep_launch();        // the projection that follows may set itself up while the rows stream
  __shared__ float partial[2][kRowCtaThreads / 32];
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int nvec = cols >> 3;
  const float inv_cols = 1.0f / static_cast<float>(cols);
  int buf = 0;
  // software pipeline over rows: the loads of the CTA's next row are issued before the current row is
  // reduced and written, which doubles the bytes each SM keeps in flight
  uint4 nxt[VPT];
  {
    const long long row0 = blockIdx.x;
    const uint4* xr0 = reinterpret_cast<const uint4*>(x + row0 * x_stride);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = tid + i * nthreads;
      nxt[i] = (row0 < rows && c < nvec) ? __ldcs(xr0 + c) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x, buf ^= 1) {
    uint4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) v[i] = nxt[i];
    {
      const long long rown = row + gridDim.x;
      const uint4* xn = reinterpret_cast<const uint4*>(x + rown * x_stride);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = tid + i * nthreads;
        if (rown < rows && c < nvec) nxt[i] = __ldcs(xn + c);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Io<T>::unpack2(w[j]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) partial[buf][warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < nwarps; ++w) tot += partial[buf][w];
    const float rstd = rsqrtf(tot * inv_cols + eps);
    if (rstd_out != nullptr && tid == 0) rstd_out[row] = rstd;
    if (y == nullptr) continue;
    uint4* yr = reinterpret_cast<uint4*>(y + row * y_stride);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = tid + i * nthreads;
      if (c < nvec) {
        uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        uint32_t g[4] = {0u, 0u, 0u, 0u};
        if (gamma != nullptr) {
          const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
          g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = Io<T>::unpack2(w[j]);
          f.x *= rstd; f.y *= rstd;
          if (gamma != nullptr) {
            const float2 gg = Io<T>::unpack2(g[j]);
            f.x *= gg.x; f.y *= gg.y;
          }
          w[j] = Io<T>::pack2(f.x, f.y);
        }
        __stcs(yr + c, make_uint4(w[0], w[1], w[2], w[3]));
      }
    }
  }
}

// Any row length: first pass reduces, second pass re-reads the row (it is L2-resident by then).
template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
rmsnorm_rows_2pass_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ gamma,
                          float* __restrict__ rstd_out, long long rows, int cols, long long x_stride,
                          long long y_stride, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * kWarpsPerCta;
  const int nvec = cols >> 3;
  const float inv_cols = 1.0f / static_cast<float>(cols);
  for (long long row = warp0; row < rows; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
    float ss = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      const uint4 v = __ldg(xr + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = Io<T>::unpack2(w[j]);
        ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss * inv_cols + eps);
    if (rstd_out != nullptr && lane == 0) rstd_out[row] = rstd;
    if (y == nullptr) continue;
    uint4* yr = reinterpret_cast<uint4*>(y + row * y_stride);
    for (int c = lane; c < nvec; c += 32) {
      const uint4 v = __ldg(xr + c);
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t g[4] = {0, 0, 0, 0};
      if (gamma != nullptr) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
        g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = Io<T>::unpack2(w[j]);
        f.x *= rstd; f.y *= rstd;
        if (gamma != nullptr) {
          float2 gg = Io<T>::unpack2(g[j]);
          f.x *= gg.x; f.y *= gg.y;
        }
        w[j] = Io<T>::pack2(f.x, f.y);
      }
      __stcs(yr + c, make_uint4(w[0], w[1], w[2], w[3]));
    }
  }
}

template <typename T>
int launch_typed(const TrnRmsArgs& a, cudaStream_t st, const DeviceState& ds) {
  const int nvec = static_cast<int>(a.cols >> 3);
  const T* x = static_cast<const T*>(a.x);
  T* y = static_cast<T*>(a.y);
  const T* g = static_cast<const T*>(a.gamma);
  const int cols = static_cast<int>(a.cols);
  if (nvec > 128 && nvec <= 4 * kRowCtaThreads) {
    // rows of 1 K .. 8 K elements (the models' hidden sizes): CTA per row
    const int vpt = (nvec + kRowCtaThreads - 1) / kRowCtaThreads;
    const int threads = ((nvec + vpt - 1) / vpt + 31) & ~31;       // warps that the row's vectors fill at vpt each
    // one resident wave: grid = SMs x CTAs that fit per SM (asked once per instantiation)
#define TRN_RMS_CTA(V)                                                                                     \
  do {                                                                                                     \
    static int per_sm_of[kRowCtaThreads / 32 + 1] = {};                                                    \
    int& per_sm = per_sm_of[threads / 32];                                                                 \
    if (per_sm == 0) {                                                                                     \
      int n = 0;                                                                                           \
      TRN_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, rmsnorm_cta_kernel<T, V>, threads, 0)); \
      per_sm = n > 0 ? n : 1;                                                                              \
    }                                                                                                      \
    const long long cap = static_cast<long long>(ds.sm_count) * per_sm;                                    \
    const int grid = static_cast<int>(a.rows < cap ? a.rows : cap);                                        \
    rmsnorm_cta_kernel<T, V><<<grid, threads, 0, st>>>(x, y, g, a.rstd_out, a.rows, cols, a.x_row_stride, \
                                                              a.y_row_stride, a.eps);                      \
  } while (0)
    if (vpt == 1) TRN_RMS_CTA(1);
    else if (vpt == 2) TRN_RMS_CTA(2);
    else if (vpt == 3) TRN_RMS_CTA(3);
    else TRN_RMS_CTA(4);
#undef TRN_RMS_CTA
    TRN_CUDA_TRY(cudaGetLastError());
    return TRN_OK;
  }
  const int vpl = (nvec + 31) / 32;
  long long want = (a.rows + kWarpsPerCta - 1) / kWarpsPerCta;
  const long long cap = static_cast<long long>(ds.sm_count) * 16;   // 16 CTAs of 4 warps per SM
  const int grid = static_cast<int>(want < cap ? want : cap);
#define TRN_RMS_LAUNCH(V)                                                                              \
  rmsnorm_rows_kernel<T, V><<<grid, kWarpsPerCta * 32, 0, st>>>(x, y, g, a.rstd_out, a.rows, cols,      \
                                                                a.x_row_stride, a.y_row_stride, a.eps)
  if (vpl <= 2) TRN_RMS_LAUNCH(2);
  else if (vpl <= 4) TRN_RMS_LAUNCH(4);
  else
    rmsnorm_rows_2pass_kernel<T><<<grid, kWarpsPerCta * 32, 0, st>>>(x, y, g, a.rstd_out, a.rows, cols,
                                                                     a.x_row_stride, a.y_row_stride, a.eps);
#undef TRN_RMS_LAUNCH
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}

}  // namespace

int launch_rmsnorm(const TrnRmsArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.rows < 0 || a.cols <= 0 || (a.cols & 7) != 0 || a.cols > (1 << 24)) return TRN_E_SHAPE;
  if (a.rows == 0) return TRN_OK;      // nothing to do (an empty tensor may carry a null pointer)
  if (a.x == nullptr || (a.y == nullptr && a.rstd_out == nullptr)) return TRN_E_NULL;
  if (a.x_row_stride < a.cols || (a.y != nullptr && a.y_row_stride < a.cols)) return TRN_E_SHAPE;
  if ((a.x_row_stride & 7) != 0 || (a.y != nullptr && (a.y_row_stride & 7) != 0)) return TRN_E_ALIGN;
  if (!aligned16(a.x) || !aligned16(a.y) || !aligned16(a.gamma)) return TRN_E_ALIGN;
  if (a.dtype == TRN_BF16) return launch_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
