// C ABI of the library (declared in include/trinity_b200.h): argument validation, per-device
// state, TMA descriptor construction and the composition of the kernels into the whole attention
// block the reference's generated forward() computes (TritonGen.py:590-708).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "host.h"

namespace trn {

namespace {

thread_local char g_cuda_err[512] = "";

// Device-side status word: kernels write a non-zero code when a bounded wait ran out.
// One copy per device that loads this library; addressed through cudaGetSymbolAddress.
__device__ int g_kernel_status = 0;

constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];
bool g_dev_ready[kMaxDevices] = {};
std::mutex g_dev_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int load_encode_fn() {
  if (g_encode != nullptr) return TRN_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return record_cuda_error(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled not available from this driver");
    return TRN_E_CUDA;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return TRN_OK;
}

}  // namespace

bool pdl_enabled() {
  const char* v = getenv("TRINITY_NO_PDL");        // read per launch: a process may switch it between calls
  return !(v != nullptr && v[0] != '\0' && v[0] != '0');
}

int record_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
  return TRN_E_CUDA;
}

int record_driver_error(CUresult r, const char* where) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: CUresult %d", where, static_cast<int>(r));
  return TRN_E_CUDA;
}

int get_device_state(DeviceState** out) {
  int dev = -1;
  TRN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TRN_E_DEVICE;
  std::lock_guard<std::mutex> lock(g_dev_mu);
  if (!g_dev_ready[dev]) {
    DeviceState ds;
    ds.device = dev;
    TRN_CUDA_TRY(cudaDeviceGetAttribute(&ds.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    TRN_CUDA_TRY(cudaDeviceGetAttribute(&ds.sm_count, cudaDevAttrMultiProcessorCount, dev));
    if (ds.cc_major != 10) return TRN_E_DEVICE;
    void* p = nullptr;
    TRN_CUDA_TRY(cudaGetSymbolAddress(&p, g_kernel_status));
    ds.status = static_cast<int*>(p);
    int rc = load_encode_fn();
    if (rc != TRN_OK) return rc;
    g_dev[dev] = ds;
    g_dev_ready[dev] = true;
  }
  *out = &g_dev[dev];
  return TRN_OK;
}

int make_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                    const uint32_t* box) {
  if (g_encode == nullptr) {
    int rc = load_encode_fn();
    if (rc != TRN_OK) return rc;
  }
  if (rank < 2 || rank > 4) return TRN_E_SHAPE;
  if (!aligned16(base)) return TRN_E_ALIGN;
  cuuint64_t gdim[4];
  cuuint64_t gstride[3];
  cuuint32_t gbox[4];
  cuuint32_t estride[4];
  for (int i = 0; i < rank; ++i) {
    if (dims[i] == 0) return TRN_E_SHAPE;
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estride[i] = 1;
    if (i >= 1) {
      const uint64_t bytes = strides[i] * 2ull;
      if ((bytes & 15ull) != 0) return TRN_E_ALIGN;
      gstride[i - 1] = bytes;
    }
  }
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                        gdim, gstride, gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return record_driver_error(r, "cuTensorMapEncodeTiled");
  return TRN_OK;
}

int ensure_dyn_smem(const void* kernel, int bytes, int device) {
  struct Entry { const void* k; int dev; };
  static Entry done[256];
  static int n_done = 0;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_done; ++i)
    if (done[i].k == kernel && done[i].dev == device) return TRN_OK;
  TRN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (n_done < 256) done[n_done++] = Entry{kernel, device};
  return TRN_OK;
}

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct BlockWorkspace {
  size_t row_scale_off, lse_off, lse2_off, split_off;
  size_t split_bytes;   // optional: split-KV partials of the attention launch
  size_t score_off, score_bytes, score_pitch;   // optional: scores kept for the per-key statistics (small problems)
  size_t required;      // the block cannot run with less
  size_t total;         // required + the optional areas
};

// KeyFormer / RoCo problems whose [B, Hq, M, P+M] fp32 scores fit in this many bytes keep them in memory and sum
// the per-key statistics from there (one q k^T pass instead of two)
constexpr size_t kKeepScoresMaxBytes = 32u << 20;
// ... and up to this size when the caller asks for the kept-scores schedule (TrnBlockArgs.keep_scores = 1)
constexpr size_t kKeepScoresHardMaxBytes = 1u << 30;

BlockWorkspace block_workspace_layout(const TrnBlockArgs& a) {
  BlockWorkspace w{};
  size_t off = 0;
  const size_t rows = static_cast<size_t>(a.B) * a.M;
  const size_t lse = static_cast<size_t>(a.B) * a.Hq * a.M;
  w.row_scale_off = off;
  off += align_up(rows * sizeof(float), 256);
  w.lse_off = off;
  off += align_up(lse * sizeof(float), 256);
  w.lse2_off = off;
  off += align_up(lse * sizeof(float), 256);
  w.split_off = off;
  w.required = off;
  w.split_bytes = attn_split_workspace(a.B, a.M, a.P, a.Hq, a.Hkv, a.D, kAttnNominalSMs);
  off += w.split_bytes;
  w.score_off = off;
  w.score_pitch = (static_cast<size_t>(a.P) + a.M + 31) / 32 * 32;
  const size_t sb = lse * w.score_pitch * sizeof(float);
  const bool stats = (a.variant == TRN_KEYFORMER || a.variant == TRN_ROCO);
  // the from-scores statistics kernel puts batch * heads on grid.y: larger problems take the two-pass kernel
  const bool grid_ok = static_cast<size_t>(a.B) * a.Hq <= 65535;
  const bool fits = a.keep_scores > 0 ? sb <= kKeepScoresHardMaxBytes : (a.keep_scores == 0 && sb <= kKeepScoresMaxBytes);
  w.score_bytes = (stats && grid_ok && fits) ? align_up(sb, 256) : 0;
  w.total = off + w.score_bytes;
  return w;
}

}  // namespace

// ---- host-activation pipeline (trinity_attn_block_host): two copy streams and a few events per device,
// created on the first call that pipelines
constexpr int kHostMaxChunks = 8;
struct HostPipe {
  bool ready = false;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t ev[2 + 2 * kHostMaxChunks] = {};
};
HostPipe g_host_pipe[kMaxDevices];
std::mutex g_host_pipe_mu;

int get_host_pipe(HostPipe** out) {
  int dev = -1;
  TRN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TRN_E_DEVICE;
  std::lock_guard<std::mutex> lock(g_host_pipe_mu);
  HostPipe& hp = g_host_pipe[dev];
  if (!hp.ready) {
    TRN_CUDA_TRY(cudaStreamCreateWithFlags(&hp.in, cudaStreamNonBlocking));
    TRN_CUDA_TRY(cudaStreamCreateWithFlags(&hp.out, cudaStreamNonBlocking));
    for (auto& e : hp.ev) TRN_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    hp.ready = true;
  }
  *out = &hp;
  return TRN_OK;
}

// How many batch groups the host path pipelines (1: one pass).  It pipelines when the batch items are
// separate contiguous slabs on both sides and the copies are large enough to be worth overlapping.
int host_chunk_count(const TrnBlockHostArgs& a) {
  const TrnBlockArgs& d = a.dev;
  if (d.B < 2 || d.M <= 0 || d.N <= 0) return 1;
  if (a.x_bytes + a.o_bytes < (4u << 20)) return 1;
  if (a.x_bytes != static_cast<size_t>(d.B) * d.M * d.N * 2) return 1;
  // o: batch-major slabs that tile o_bytes exactly
  if (d.o.stride_b <= 0 || static_cast<size_t>(d.o.stride_b) * 2 * d.B != a.o_bytes) return 1;
  if (d.o.stride_b < d.o.stride_s * d.M || d.o.stride_b < d.o.stride_h * d.Hq) return 1;
  if (a.stats_bytes % d.B != 0) return 1;
  if ((d.sum_p != nullptr || d.sum_p2 != nullptr) &&
      a.stats_bytes != 0 && a.stats_bytes != static_cast<size_t>(d.B) * d.Hq * (d.P + d.M) * (d.stats_fp32 ? 4 : 2))
    return 1;
  return d.B < kHostMaxChunks ? d.B : kHostMaxChunks;
}

size_t block_workspace_required(const TrnBlockArgs& a) { return block_workspace_layout(a).required; }

}  // namespace trn

using namespace trn;

extern "C" {

int trinity_abi_version(void) { return TRINITY_ABI_VERSION; }

const char* trinity_strerror(int code) {
  switch (code) {
    case TRN_OK: return "ok";
    case TRN_E_NULL: return "a required pointer is NULL";
    case TRN_E_SHAPE: return "unsupported or inconsistent shape";
    case TRN_E_ALIGN: return "pointer or stride is not 16-byte aligned";
    case TRN_E_DTYPE: return "unknown element type";
    case TRN_E_VARIANT: return "unknown variant or flag combination";
    case TRN_E_WORKSPACE: return "workspace missing, misaligned or too small";
    case TRN_E_CUDA: return "a CUDA call failed (see trinity_last_cuda_error)";
    case TRN_E_DEVICE: return "current device is not an sm_100 GPU";
    case TRN_E_KERNEL: return "a kernel reported a device-side status (a bounded wait ran out)";
    case TRN_E_STATIC_SCRATCH:
      return "problem needs more scratch than the library's built-in array holds (use trinity_attn_block with a workspace)";
    default: return "unknown error code";
  }
}

const char* trinity_last_cuda_error(void) { return g_cuda_err; }

int trinity_last_kernel_status(int* status_out) {
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  int v = 0;
  TRN_CUDA_TRY(cudaDeviceSynchronize());
  TRN_CUDA_TRY(cudaMemcpy(&v, ds->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status_out != nullptr) *status_out = v;
  return v == 0 ? TRN_OK : TRN_E_KERNEL;
}

int trinity_clear_kernel_status(void) {
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  TRN_CUDA_TRY(cudaDeviceSynchronize());
  TRN_CUDA_TRY(cudaMemset(ds->status, 0, sizeof(int)));
  TRN_CUDA_TRY(cudaDeviceSynchronize());
  return TRN_OK;
}

int trinity_rmsnorm(const TrnRmsArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_rmsnorm(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

int trinity_qkv_project(const TrnProjArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_qkv_project(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

int trinity_lora(const TrnLoraArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_lora(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

int trinity_gmlp(const TrnGmlpArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_gmlp(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

int trinity_attention(const TrnAttnArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_attention(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

size_t trinity_attention_workspace(const TrnAttnArgs* a) {
  if (a == nullptr) return 0;
  return attn_split_workspace(a->B, a->M, a->P, a->Hq, a->Hkv, a->D, kAttnNominalSMs);
}

int trinity_attn_colstats(const TrnColStatsArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_colstats(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

int trinity_topk(const TrnTopkArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_topk(*a, static_cast<cudaStream_t>(cuda_stream), *ds);
}

int trinity_convert(const void* src, void* dst, int64_t n, int dtype16, int to_fp32, void* cuda_stream) {
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  return launch_convert(src, dst, n, dtype16, to_fp32, static_cast<cudaStream_t>(cuda_stream), *ds);
}

size_t trinity_attn_block_workspace(const TrnBlockArgs* a) {
  if (a == nullptr || a->B <= 0 || a->M <= 0 || a->Hq <= 0) return 0;
  return block_workspace_layout(*a).total;
}

int trinity_attn_block(const TrnBlockArgs* a, void* cuda_stream) {
  if (a == nullptr) return TRN_E_NULL;
  if (a->variant < TRN_VANILLA || a->variant > TRN_ROCO) return TRN_E_VARIANT;
  if (a->B <= 0 || a->M <= 0 || a->P < 0 || a->Hq <= 0 || a->Hkv <= 0) return TRN_E_SHAPE;
  if (a->Hq % a->Hkv != 0) return TRN_E_SHAPE;
  DeviceState* ds = nullptr;
  int rc = get_device_state(&ds);
  if (rc != TRN_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);

  const BlockWorkspace wl = block_workspace_layout(*a);
  if (a->workspace == nullptr || a->workspace_bytes < wl.required) return TRN_E_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0) return TRN_E_WORKSPACE;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  float* row_scale = reinterpret_cast<float*>(ws + wl.row_scale_off);
  float* lse = reinterpret_cast<float*>(ws + wl.lse_off);
  float* lse_pert = reinterpret_cast<float*>(ws + wl.lse2_off);

  const bool stats = (a->variant == TRN_KEYFORMER || a->variant == TRN_ROCO);
  if (stats && a->sum_p == nullptr) return TRN_E_NULL;
  if (a->variant == TRN_ROCO && a->sum_p2 == nullptr) return TRN_E_NULL;
  if (a->variant == TRN_KEYFORMER && a->noise_mode == TRN_NOISE_TENSOR && a->noise == nullptr) return TRN_E_NULL;
  // Everything the later steps would refuse is refused here, before the first launch: a negative return code
  // means that nothing ran.
  {
    if (a->dtype != TRN_BF16 && a->dtype != TRN_FP16) return TRN_E_DTYPE;
    if (a->D != 64 && a->D != 128) return TRN_E_SHAPE;
    if (!(a->scale > 0.f)) return TRN_E_SHAPE;
    if (a->variant == TRN_KEYFORMER) {
      if (a->noise_mode <= TRN_NOISE_NONE || a->noise_mode > TRN_NOISE_GUMBEL) return TRN_E_VARIANT;
      if (!(a->tau > 0.f)) return TRN_E_SHAPE;
    }
    auto head_ok = [](const TrnHeadTensor& t) {
      return aligned16(t.ptr) && (t.stride_b & 7) == 0 && (t.stride_s & 7) == 0 && (t.stride_h & 7) == 0;
    };
    if (a->q.ptr == nullptr || a->k_cache.ptr == nullptr || a->v_cache.ptr == nullptr || a->o.ptr == nullptr)
      return TRN_E_NULL;
    if (!head_ok(a->q) || !head_ok(a->k_cache) || !head_ok(a->v_cache) || !head_ok(a->o)) return TRN_E_ALIGN;
    if (!a->skip_projection) {
      if (a->N <= 0 || (a->N & 7) != 0) return TRN_E_SHAPE;
      if (static_cast<long long>(a->B) * a->M > 0x7fffffffLL) return TRN_E_SHAPE;
      if (a->x == nullptr || a->wq == nullptr || a->wk == nullptr || a->wv == nullptr) return TRN_E_NULL;
      if (!aligned16(a->x) || !aligned16(a->wq) || !aligned16(a->wk) || !aligned16(a->wv)) return TRN_E_ALIGN;
      if (!aligned16(a->gamma_q) || !aligned16(a->gamma_k) || !aligned16(a->pre_gamma) || !aligned16(a->x_norm))
        return TRN_E_ALIGN;
      if (a->variant == TRN_PRENORM && a->pre_gamma != nullptr && a->x_norm == nullptr) return TRN_E_NULL;
    }
  }

  if (!a->skip_projection) {
    if (a->N <= 0) return TRN_E_SHAPE;
    const void* x_in = a->x;
    const float* rs = nullptr;
    if (a->variant == TRN_PRENORM) {
      TrnRmsArgs r{};
      r.x = a->x;
      r.rows = static_cast<int64_t>(a->B) * a->M;
      r.cols = a->N;
      r.x_row_stride = a->N;
      r.y_row_stride = a->N;
      r.eps = a->pre_eps;
      r.dtype = a->dtype;
      if (a->pre_gamma != nullptr || a->x_norm != nullptr) {
        // gamma scales the hidden (contraction) axis, so it cannot move to the GEMM epilogue:
        // materialise x_norm once, then project it.  A caller that passes x_norm without gamma asks for
        // the same two-step schedule (its program stores X_norm as a tensor of its own).
        if (a->x_norm == nullptr) return TRN_E_NULL;
        r.y = a->x_norm;
        r.gamma = a->pre_gamma;
        x_in = a->x_norm;
      } else {
        // (x * r_i) @ w == r_i * (x @ w): only the row statistics are computed here
        r.rstd_out = row_scale;
        rs = row_scale;
      }
      rc = launch_rmsnorm(r, st, *ds);
      if (rc != TRN_OK) return rc;
    }
    TrnProjArgs pj{};
    pj.x = x_in;
    pj.wq = a->wq;
    pj.wk = a->wk;
    pj.wv = a->wv;
    pj.row_scale = rs;
    pj.B = a->B; pj.M = a->M; pj.P = a->P; pj.N = a->N;
    pj.Hq = a->Hq; pj.Hkv = a->Hkv; pj.D = a->D;
    pj.dtype = a->dtype;
    pj.qk_norm = (a->variant == TRN_QKNORM) ? 1 : 0;
    pj.qk_eps = a->qk_eps;
    pj.gamma_q = a->gamma_q;
    pj.gamma_k = a->gamma_k;
    pj.q = a->q;
    pj.k_cache = a->k_cache;
    pj.v_cache = a->v_cache;
    rc = launch_qkv_project(pj, st, *ds);
    if (rc != TRN_OK) return rc;
  }

  TrnAttnArgs at{};
  at.q = a->q;
  at.k_cache = a->k_cache;
  at.v_cache = a->v_cache;
  at.o = a->o;
  at.lse = stats ? lse : nullptr;
  at.B = a->B; at.M = a->M; at.P = a->P; at.Hq = a->Hq; at.Hkv = a->Hkv; at.D = a->D;
  at.dtype = a->dtype;
  at.causal = a->causal;
  at.scale = a->scale;
  at.noise_mode = TRN_NOISE_NONE;
  at.tau = 1.0f;
  at.single_p = a->single_p;
  // What the caller lent beyond the required part: first the split-KV partials of the attention launch, then,
  // for small KeyFormer / RoCo problems, the scores the statistics are summed from.
  const bool keep_scores = stats && wl.score_bytes > 0 && a->workspace_bytes >= wl.score_off + wl.score_bytes;
  at.workspace = ws + wl.split_off;
  at.workspace_bytes = keep_scores ? wl.split_bytes : a->workspace_bytes - wl.split_off;
  if (keep_scores) {
    at.scores = reinterpret_cast<float*>(ws + wl.score_off);
    at.score_pitch = static_cast<int64_t>(wl.score_pitch);
  }
  if (a->variant == TRN_KEYFORMER) {
    // the same pass also gives the log-sum-exp of the perturbed scores (ref_rms.py:172,174)
    if (a->noise_mode == TRN_NOISE_NONE) return TRN_E_VARIANT;
    at.noise_mode = a->noise_mode;
    at.tau = a->tau;
    at.noise = a->noise;
    at.noise_stride_b = a->noise_stride_b;
    at.noise_stride_h = a->noise_stride_h;
    at.noise_stride_i = a->noise_stride_i;
    at.seed = a->seed;
    at.noise_heads = a->noise_heads;
    at.noise_bh0 = a->noise_bh0;
    at.lse_pert = lse_pert;
  }
  // At most 16 queries per head: the statistics ride in the attention launch (every score of a head is on chip when
  // its rows' log-sum-exp is known), whatever keep_scores says; nothing is kept and no second launch follows.
  AttnFusedStats fstats{};
  if (stats) {
    fstats.sum_p = a->sum_p;
    fstats.sum_p2 = (a->variant == TRN_ROCO) ? a->sum_p2 : nullptr;
    fstats.stats_fp32 = a->stats_fp32;
    if (attn_small_stats_applies(at, ds->sm_count)) {
      at.scores = nullptr;
      at.score_pitch = 0;
    }
  }
  rc = launch_attention(at, st, *ds, stats ? &fstats : nullptr);
  if (rc != TRN_OK) return rc;

  if (stats && !fstats.done) {
    const float* lse_for_stats = lse;
    int noise_mode = TRN_NOISE_NONE;
    if (a->variant == TRN_KEYFORMER) {
      lse_for_stats = lse_pert;
      noise_mode = a->noise_mode;
    }
    TrnColStatsArgs cs{};
    cs.q = a->q;
    cs.k_cache = a->k_cache;
    cs.lse = lse_for_stats;
    cs.sum_p = a->sum_p;
    cs.sum_p2 = (a->variant == TRN_ROCO) ? a->sum_p2 : nullptr;
    cs.B = a->B; cs.M = a->M; cs.P = a->P; cs.Hq = a->Hq; cs.Hkv = a->Hkv; cs.D = a->D;
    cs.dtype = a->dtype;
    cs.stats_fp32 = a->stats_fp32;
    cs.causal = a->causal;
    cs.scale = a->scale;
    cs.noise_mode = noise_mode;
    cs.tau = (a->variant == TRN_KEYFORMER) ? a->tau : 1.0f;
    cs.noise = a->noise;
    cs.noise_stride_b = a->noise_stride_b;
    cs.noise_stride_h = a->noise_stride_h;
    cs.noise_stride_i = a->noise_stride_i;
    cs.seed = a->seed;
    cs.noise_heads = a->noise_heads;
    cs.noise_bh0 = a->noise_bh0;
    if (keep_scores) {
      cs.scores = at.scores;
      cs.score_pitch = at.score_pitch;
    }
    rc = launch_colstats(cs, st, *ds);
    if (rc != TRN_OK) return rc;
    }
  return TRN_OK;
}

int trinity_attn_block_host(const TrnBlockHostArgs* a, void* cuda_stream) {
  if (a == nullptr || a->x_host == nullptr || a->o_host == nullptr) return TRN_E_NULL;
  if (a->dev.x == nullptr || a->dev.o.ptr == nullptr) return TRN_E_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const TrnBlockArgs& d = a->dev;
  HostPipe* hp = nullptr;
  const int chunks = host_chunk_count(*a);
  if (chunks > 1 && get_host_pipe(&hp) == TRN_OK) {
    // Batch items are independent: copy item group c+1 in while group c computes and group c-1 copies out
    // (PCIe is full duplex; the copies run on two streams of the library, ordered against the caller's
    // stream by events).  Per-element results are the same as in one pass: each output element is computed
    // by the same instructions in the same order whichever rows share its launch.
    const int per = (d.B + chunks - 1) / chunks;
    DeviceState* ds = nullptr;
    int rcd = get_device_state(&ds);
    if (rcd != TRN_OK) return rcd;
    // every group uses the split-KV count of the uncut problem
    struct SplitGuard {
      explicit SplitGuard(int n) { tls_attn_split_override = n; }
      ~SplitGuard() { tls_attn_split_override = 0; }
    } guard(attn_planned_splits(d.B, d.M, d.P, d.Hq, d.Hkv, d.D, d.causal, ds->sm_count));
    const size_t esz = 2;
    const size_t stat_esz = d.stats_fp32 ? 4 : 2;
    const size_t x_item = a->x_bytes / d.B, o_item = a->o_bytes / d.B;
    const size_t stats_item = (a->stats_bytes != 0) ? a->stats_bytes / d.B : 0;
    TRN_CUDA_TRY(cudaEventRecord(hp->ev[0], st));
    TRN_CUDA_TRY(cudaStreamWaitEvent(hp->in, hp->ev[0], 0));
    TRN_CUDA_TRY(cudaStreamWaitEvent(hp->out, hp->ev[0], 0));
    int n = 0;
    for (int b0 = 0; b0 < d.B; b0 += per, ++n) {
      const int nb = (d.B - b0 < per) ? d.B - b0 : per;
      TRN_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(const_cast<void*>(d.x)) + b0 * x_item,
                                   static_cast<const uint8_t*>(a->x_host) + b0 * x_item, nb * x_item,
                                   cudaMemcpyHostToDevice, hp->in));
      TRN_CUDA_TRY(cudaEventRecord(hp->ev[1 + 2 * n], hp->in));
    }
    n = 0;
    for (int b0 = 0; b0 < d.B; b0 += per, ++n) {
      const int nb = (d.B - b0 < per) ? d.B - b0 : per;
      TrnBlockArgs c = d;
      c.B = nb;
      auto adv = [&](const void* ptr, size_t bytes_per_item) -> void* {
        return ptr == nullptr ? nullptr : static_cast<uint8_t*>(const_cast<void*>(ptr)) + b0 * bytes_per_item;
      };
      c.x = adv(d.x, x_item);
      c.x_norm = adv(d.x_norm, x_item);
      c.q.ptr = adv(d.q.ptr, d.q.stride_b * esz);
      c.k_cache.ptr = adv(d.k_cache.ptr, d.k_cache.stride_b * esz);
      c.v_cache.ptr = adv(d.v_cache.ptr, d.v_cache.stride_b * esz);
      c.o.ptr = adv(d.o.ptr, d.o.stride_b * esz);
      c.noise = adv(d.noise, d.noise_stride_b * esz);
      const size_t stats_dev_item = static_cast<size_t>(d.Hq) * (d.P + d.M) * stat_esz;
      c.sum_p = adv(d.sum_p, stats_dev_item);
      c.sum_p2 = adv(d.sum_p2, stats_dev_item);
      // generated KeyFormer noise is indexed by the batch item of the uncut problem
      c.noise_heads = d.noise_heads > 0 ? d.noise_heads : d.Hq;
      c.noise_bh0 = d.noise_bh0 + b0 * c.noise_heads;
      TRN_CUDA_TRY(cudaStreamWaitEvent(st, hp->ev[1 + 2 * n], 0));
      int rc = trinity_attn_block(&c, cuda_stream);
      if (rc != TRN_OK) {
        cudaStreamSynchronize(hp->in);      // leave no copy of this call in flight
        cudaStreamSynchronize(st);
        return rc;
      }
      TRN_CUDA_TRY(cudaEventRecord(hp->ev[2 + 2 * n], st));
      TRN_CUDA_TRY(cudaStreamWaitEvent(hp->out, hp->ev[2 + 2 * n], 0));
      TRN_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(a->o_host) + b0 * o_item,
                                   static_cast<const uint8_t*>(d.o.ptr) + b0 * o_item, nb * o_item,
                                   cudaMemcpyDeviceToHost, hp->out));
      if (a->sum_p_host != nullptr && d.sum_p != nullptr)
        TRN_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(a->sum_p_host) + b0 * stats_item, c.sum_p, nb * stats_item,
                                     cudaMemcpyDeviceToHost, hp->out));
      if (a->sum_p2_host != nullptr && d.sum_p2 != nullptr)
        TRN_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(a->sum_p2_host) + b0 * stats_item, c.sum_p2, nb * stats_item,
                                     cudaMemcpyDeviceToHost, hp->out));
    }
    TRN_CUDA_TRY(cudaEventRecord(hp->ev[1 + 2 * kHostMaxChunks], hp->out));
    TRN_CUDA_TRY(cudaStreamWaitEvent(st, hp->ev[1 + 2 * kHostMaxChunks], 0));
    TRN_CUDA_TRY(cudaStreamSynchronize(st));
    return TRN_OK;
  }
  TRN_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(a->dev.x), a->x_host, a->x_bytes, cudaMemcpyHostToDevice, st));
  int rc = trinity_attn_block(&a->dev, cuda_stream);
  if (rc != TRN_OK) return rc;
  TRN_CUDA_TRY(cudaMemcpyAsync(a->o_host, a->dev.o.ptr, a->o_bytes, cudaMemcpyDeviceToHost, st));
  if (a->sum_p_host != nullptr && a->dev.sum_p != nullptr)
    TRN_CUDA_TRY(cudaMemcpyAsync(a->sum_p_host, a->dev.sum_p, a->stats_bytes, cudaMemcpyDeviceToHost, st));
  if (a->sum_p2_host != nullptr && a->dev.sum_p2 != nullptr)
    TRN_CUDA_TRY(cudaMemcpyAsync(a->sum_p2_host, a->dev.sum_p2, a->stats_bytes, cudaMemcpyDeviceToHost, st));
  TRN_CUDA_TRY(cudaStreamSynchronize(st));
  return TRN_OK;
}

}  // extern "C"
