// Pieces shared by the attention forward kernel and the per-key statistics kernel:
// the 4-D TMA view of a head-split tensor, KeyFormer's noise (tensor or counter-based Gumbel) and
// a few math helpers.
#pragma once

#include "common.cuh"
#include "host.h"

namespace trn {

// A (b, s, h, d) tensor as a rank-4 TMA descriptor whose dims are ordered by ascending stride
// (d first).  pos_* give the position (1..3) of s, h and b among the descriptor's dims, so that a
// kernel can place its coordinates.
struct HeadMapInfo {
  int pos_s, pos_h, pos_b;
};

// Tile = `box_rows` positions x 64 head_dim elements of one (b, h).
inline int make_head_tmap(CUtensorMap* out, HeadMapInfo* info, const TrnHeadTensor& t, int S, int H, int B, int D,
                          uint32_t box_rows) {
  if (t.ptr == nullptr) return TRN_E_NULL;
  // dims of extent 1 may carry any stride: give them one that keeps the descriptor valid
  uint64_t ss = static_cast<uint64_t>(t.stride_s), sh = static_cast<uint64_t>(t.stride_h),
           sb = static_cast<uint64_t>(t.stride_b);
  if (t.stride_s < 0 || t.stride_h < 0 || t.stride_b < 0) return TRN_E_SHAPE;
  uint64_t span = static_cast<uint64_t>(D);
  if (S > 1 && ss * S > span) span = ss * S;
  if (H > 1 && sh * H > span) span = sh * H;
  if (B > 1 && sb * B > span) span = sb * B;
  span = (span + 7) & ~7ull;
  if (S == 1) ss = span;
  if (H == 1) sh = span;
  if (B == 1) sb = span;
  struct Dim { uint64_t extent, stride; uint32_t box; int which; };   // which: 0 = s, 1 = h, 2 = b
  Dim dm[3] = {{static_cast<uint64_t>(S), ss, box_rows, 0},
               {static_cast<uint64_t>(H), sh, 1u, 1},
               {static_cast<uint64_t>(B), sb, 1u, 2}};
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (dm[j].stride < dm[i].stride) { Dim tmp = dm[i]; dm[i] = dm[j]; dm[j] = tmp; }
  uint64_t dims[4] = {static_cast<uint64_t>(D), dm[0].extent, dm[1].extent, dm[2].extent};
  uint64_t strides[4] = {1, dm[0].stride, dm[1].stride, dm[2].stride};
  uint32_t box[4] = {64u, dm[0].box, dm[1].box, dm[2].box};
  for (int i = 0; i < 3; ++i) {
    if (dm[i].which == 0) info->pos_s = i + 1;
    if (dm[i].which == 1) info->pos_h = i + 1;
    if (dm[i].which == 2) info->pos_b = i + 1;
  }
  return make_tmap_16bit(out, t.ptr, 4, dims, strides, box);
}

// load one [rows x 64] tile: head_dim offset d0, position s0 of (b, h)
__device__ __forceinline__ void tma_load_head_tile(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                                   const HeadMapInfo& inf, int d0, int s0, int h, int b) {
  int c[4];
  c[0] = d0;
  c[inf.pos_s] = s0;
  c[inf.pos_h] = h;
  c[inf.pos_b] = b;
  tma_load_4d(dst, m, bar, c[0], c[1], c[2], c[3]);
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------------------------------
// KeyFormer noise.  Counter-based: element (b, h, query i, key j) of a [B, Hq, M, L] noise field gets
// 32 hashed bits in three steps so that most of the work is shared along a row or a column:
//   headkey = mix32(seed_lo ^ mix32(b * Hq + h + seed_hi * 0x9e3779b9))      once per (b, h)
//   rowhash = mix32(headkey + i * 0x9e3779b9)                                once per query
//   bits    = fmix(rowhash ^ (j * 0x85ebca6b))                               per element
// 23 of the bits make u in (0,1) and g = -log(-log(u)) ~ Gumbel(0,1).  The host restatement of this
// function (same integer steps, float64 logs) lives with the parity oracle.
// ------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du;
  x ^= x >> 15; x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__host__ __device__ __forceinline__ uint32_t noise_headkey(uint64_t seed, uint32_t bh) {
  return mix32(static_cast<uint32_t>(seed) ^ mix32(bh + static_cast<uint32_t>(seed >> 32) * 0x9e3779b9u));
}
__host__ __device__ __forceinline__ uint32_t noise_rowhash(uint32_t headkey, uint32_t i) {
  return mix32(headkey + i * 0x9e3779b9u);
}
__host__ __device__ __forceinline__ uint32_t noise_elem_bits(uint32_t rowhash, uint32_t j) {
  uint32_t x = rowhash ^ (j * 0x85ebca6bu);
  x ^= x >> 16; x *= 0x7feb352du;
  x ^= x >> 15;
  return x;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// g = -ln(-ln u), u = (k + 0.5) / 2^23 with k the top 23 bits.  Two MUFU log2; when u is within 2^-10 of 1
// (where log2's absolute error, ~2^-22, would dominate) -ln u comes from the series v + v^2/2 of v = 1 - u
// instead (truncation < 3e-7 relative).  Relative error of the inner logarithm <= ~2e-4, absolute error of
// g of the same order.
constexpr float kGumbelSeriesBelow = 0.0009765625f;   // 2^-10
// u and 1 - u are built from the bits without an integer-to-float conversion (those share the MUFU pipe with
// the logarithms): 0x3f800000 | k is the float 1 + k 2^-23, and subtracting 1 - 2^-24 leaves (k + 0.5) 2^-23
// exactly; 0x7fffff - k = k ^ 0x7fffff gives 1 - u the same way.
__device__ __forceinline__ float unit_from_23bits(uint32_t k) {
  return __uint_as_float(0x3f800000u | k) - 0.999999940395355224609375f;
}
__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  const uint32_t k = bits >> 9;
  const float u = unit_from_23bits(k);
  const float v = unit_from_23bits(k ^ 0x7fffffu);                                             // 1 - u, exact
  const float w_log = -0.6931471805599453f * lg2_approx(u);
  const float w_ser = fmaf(0.5f * v, v, v);                                                     // v + v^2/2
  const float w = (v < kGumbelSeriesBelow) ? w_ser : w_log;
  return -0.6931471805599453f * lg2_approx(w);
}

// log2 of E = -ln u for the same u: the Gumbel value is g = -ln2 * log2(E), so callers that work in the
// log2 domain fold the constant into their own scale
__device__ __forceinline__ float gumbel_log2e_from_bits(uint32_t bits) {
  const uint32_t k = bits >> 9;
  const float u = unit_from_23bits(k);
  const float v = unit_from_23bits(k ^ 0x7fffffu);
  const float w_log = -0.6931471805599453f * lg2_approx(u);
  const float w_ser = fmaf(0.5f * v, v, v);
  return lg2_approx((v < kGumbelSeriesBelow) ? w_ser : w_log);
}

struct NoiseSrc {
  int mode;                  // TRN_NOISE_*
  const void* ptr;           // tensor mode
  long long sb, sh, si;      // element strides of (b, h, i); j contiguous
  unsigned long long seed;   // gumbel mode
  long long M, L, Hq;        // field extents (Hq: query heads of the WHOLE field, of which a launch may hold a slice)
  long long bh0;             // b * Hq + h of the launch's first (batch item, head) inside the whole field
};

// noise of element (b, h, i, j); `rowhash` is noise_rowhash(noise_headkey(seed, b*Hq+h), i)
template <typename T>
__device__ __forceinline__ float noise_at(const NoiseSrc& n, uint32_t rowhash, int b, int h, int i, int j) {
  if (n.mode == TRN_NOISE_TENSOR) {
    const T* p = static_cast<const T*>(n.ptr) + b * n.sb + h * n.sh + i * n.si + j;
    return Io<T>::to_f(*p);
  }
  return gumbel_from_bits(noise_elem_bits(rowhash, static_cast<uint32_t>(j)));
}

}  // namespace trn
