"""ctypes binding of libtrinity_b200.so — mirrors include/trinity_b200.h field for field.

There is no fallback: if the shared library is missing or fails to load, importing a symbol from
here raises, and so does every operator built on it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

LIB_NAME = "libtrinity_b200.so"
# TRINITY_B200_LIB points at another build of the same library (e.g. one compiled with extra -D flags)
LIB_PATH = Path(os.environ.get("TRINITY_B200_LIB") or (Path(__file__).resolve().parent / LIB_NAME))

ABI_VERSION = 3

TRN_BF16, TRN_FP16 = 0, 1
TRN_VANILLA, TRN_PRENORM, TRN_QKNORM, TRN_KEYFORMER, TRN_ROCO = range(5)
TRN_NOISE_NONE, TRN_NOISE_TENSOR, TRN_NOISE_GUMBEL = range(3)
TRN_GATE_SILU, TRN_GATE_SIGMOID = range(2)
VARIANTS = {"vanilla": TRN_VANILLA, "prenorm": TRN_PRENORM, "qknorm": TRN_QKNORM,
            "keyformer": TRN_KEYFORMER, "roco": TRN_ROCO}

# every symbol include/trinity_b200.h declares
EXPORTS = (
    "trinity_abi_version", "trinity_strerror", "trinity_last_cuda_error", "trinity_last_kernel_status",
    "trinity_clear_kernel_status", "trinity_selftest_wait_timeout",
    "trinity_rmsnorm", "trinity_qkv_project", "trinity_lora", "trinity_gmlp", "trinity_attention", "trinity_attention_workspace",
    "trinity_attn_colstats", "trinity_topk",
    "trinity_attn_block_workspace", "trinity_attn_block", "trinity_attn_block_host",
    "trinity_static_scratch_capacity", "trinity_attn_block_static", "trinity_convert",
)


class TrnRmsArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("y", C.c_void_p), ("gamma", C.c_void_p), ("rstd_out", C.c_void_p),
        ("rows", C.c_int64), ("cols", C.c_int64), ("x_row_stride", C.c_int64), ("y_row_stride", C.c_int64),
        ("eps", C.c_float), ("dtype", C.c_int),
    ]


class TrnHeadTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_s", C.c_int64), ("stride_h", C.c_int64)]


class TrnProjArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p), ("row_scale", C.c_void_p),
        ("B", C.c_int), ("M", C.c_int), ("P", C.c_int), ("N", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int),
        ("D", C.c_int), ("dtype", C.c_int), ("qk_norm", C.c_int), ("qk_eps", C.c_float),
        ("gamma_q", C.c_void_p), ("gamma_k", C.c_void_p),
        ("q", TrnHeadTensor), ("k_cache", TrnHeadTensor), ("v_cache", TrnHeadTensor),
    ]


class TrnLoraArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("a", C.c_void_p), ("b", C.c_void_p), ("o", C.c_void_p),
        ("d", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("P", C.c_int), ("R", C.c_int), ("dtype", C.c_int),
    ]


class TrnGmlpArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w1", C.c_void_p), ("w2", C.c_void_p), ("o", C.c_void_p),
        ("M", C.c_int), ("K", C.c_int), ("N", C.c_int), ("dtype", C.c_int), ("gate", C.c_int),
    ]


class TrnAttnArgs(C.Structure):
    _fields_ = [
        ("q", TrnHeadTensor), ("k_cache", TrnHeadTensor), ("v_cache", TrnHeadTensor), ("o", TrnHeadTensor),
        ("lse", C.c_void_p),
        ("B", C.c_int), ("M", C.c_int), ("P", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("D", C.c_int),
        ("dtype", C.c_int), ("causal", C.c_int), ("scale", C.c_float), ("noise_mode", C.c_int), ("tau", C.c_float),
        ("noise", C.c_void_p), ("noise_stride_b", C.c_int64), ("noise_stride_h", C.c_int64),
        ("noise_stride_i", C.c_int64), ("seed", C.c_uint64), ("single_p", C.c_int),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("lse_pert", C.c_void_p), ("scores", C.c_void_p), ("score_pitch", C.c_int64),
        ("noise_heads", C.c_int), ("noise_bh0", C.c_int),
    ]


class TrnColStatsArgs(C.Structure):
    _fields_ = [
        ("q", TrnHeadTensor), ("k_cache", TrnHeadTensor), ("lse", C.c_void_p), ("sum_p", C.c_void_p),
        ("sum_p2", C.c_void_p),
        ("B", C.c_int), ("M", C.c_int), ("P", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("D", C.c_int),
        ("dtype", C.c_int), ("stats_fp32", C.c_int), ("causal", C.c_int), ("scale", C.c_float),
        ("noise_mode", C.c_int), ("tau", C.c_float),
        ("noise", C.c_void_p), ("noise_stride_b", C.c_int64), ("noise_stride_h", C.c_int64),
        ("noise_stride_i", C.c_int64), ("seed", C.c_uint64),
        ("scores", C.c_void_p), ("score_pitch", C.c_int64), ("noise_heads", C.c_int), ("noise_bh0", C.c_int),
    ]


class TrnTopkArgs(C.Structure):
    _fields_ = [
        ("scores", C.c_void_p), ("idx_out", C.c_void_p), ("rows", C.c_int64), ("n", C.c_int), ("k", C.c_int),
        ("score_row_stride", C.c_int64),
    ]


class TrnBlockArgs(C.Structure):
    _fields_ = [
        ("variant", C.c_int), ("dtype", C.c_int),
        ("B", C.c_int), ("M", C.c_int), ("P", C.c_int), ("N", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int),
        ("D", C.c_int), ("skip_projection", C.c_int),
        ("x", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
        ("pre_eps", C.c_float), ("pre_gamma", C.c_void_p), ("x_norm", C.c_void_p),
        ("qk_eps", C.c_float), ("gamma_q", C.c_void_p), ("gamma_k", C.c_void_p),
        ("q", TrnHeadTensor), ("k_cache", TrnHeadTensor), ("v_cache", TrnHeadTensor), ("o", TrnHeadTensor),
        ("causal", C.c_int), ("scale", C.c_float),
        ("noise_mode", C.c_int), ("tau", C.c_float), ("noise", C.c_void_p),
        ("noise_stride_b", C.c_int64), ("noise_stride_h", C.c_int64), ("noise_stride_i", C.c_int64),
        ("seed", C.c_uint64),
        ("sum_p", C.c_void_p), ("sum_p2", C.c_void_p), ("stats_fp32", C.c_int), ("single_p", C.c_int),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("keep_scores", C.c_int),
        ("noise_heads", C.c_int), ("noise_bh0", C.c_int),
    ]


class TrnBlockHostArgs(C.Structure):
    _fields_ = [
        ("dev", TrnBlockArgs), ("x_host", C.c_void_p), ("o_host", C.c_void_p),
        ("x_bytes", C.c_size_t), ("o_bytes", C.c_size_t),
        ("sum_p_host", C.c_void_p), ("sum_p2_host", C.c_void_p), ("stats_bytes", C.c_size_t),
    ]


class TrinityError(RuntimeError):
    """Raised when an entry point returns a non-zero status; carries the C-side message."""

    def __init__(self, code: int, message: str):
        super().__init__(f"trinity_b200 error {code}: {message}")
        self.code = code


_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once).  Raises if it is absent: there is no CPU or library fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m triton_b200.build` "
            "(nvcc, sm_100a).  triton_b200 has no fallback path.")
    lib = C.CDLL(str(LIB_PATH))
    lib.trinity_abi_version.restype = C.c_int
    lib.trinity_strerror.restype = C.c_char_p
    lib.trinity_strerror.argtypes = [C.c_int]
    lib.trinity_last_cuda_error.restype = C.c_char_p
    lib.trinity_last_kernel_status.restype = C.c_int
    lib.trinity_last_kernel_status.argtypes = [C.POINTER(C.c_int)]
    for name, typ in (("trinity_rmsnorm", TrnRmsArgs), ("trinity_qkv_project", TrnProjArgs), ("trinity_lora", TrnLoraArgs), ("trinity_gmlp", TrnGmlpArgs),
                      ("trinity_attention", TrnAttnArgs), ("trinity_attn_colstats", TrnColStatsArgs),
                      ("trinity_topk", TrnTopkArgs), ("trinity_attn_block", TrnBlockArgs),
                      ("trinity_attn_block_host", TrnBlockHostArgs), ("trinity_attn_block_static", TrnBlockArgs)):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(typ), C.c_void_p]
    lib.trinity_attn_block_workspace.restype = C.c_size_t
    lib.trinity_attn_block_workspace.argtypes = [C.POINTER(TrnBlockArgs)]
    lib.trinity_attention_workspace.restype = C.c_size_t
    lib.trinity_attention_workspace.argtypes = [C.POINTER(TrnAttnArgs)]
    lib.trinity_clear_kernel_status.restype = C.c_int
    lib.trinity_clear_kernel_status.argtypes = []
    lib.trinity_selftest_wait_timeout.restype = C.c_int
    lib.trinity_selftest_wait_timeout.argtypes = [C.c_int, C.c_void_p]
    lib.trinity_convert.restype = C.c_int
    lib.trinity_convert.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]
    lib.trinity_static_scratch_capacity.restype = C.c_size_t
    lib.trinity_static_scratch_capacity.argtypes = []
    if lib.trinity_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{LIB_NAME} has ABI {lib.trinity_abi_version()}, binding expects {ABI_VERSION}")
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc == 0:
        return
    lib = load()
    msg = lib.trinity_strerror(rc).decode()
    if rc == -7:
        msg += ": " + lib.trinity_last_cuda_error().decode()
    raise TrinityError(rc, msg)


def kernel_status() -> int:
    """Synchronises the device and returns the device-side status word (0 = every wait finished)."""
    st = C.c_int(0)
    load().trinity_last_kernel_status(C.byref(st))
    return st.value
