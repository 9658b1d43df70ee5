"""`from convert_module import convert_ir_to_triton` — the import the reference's harnesses make
(vanilla_llama_benchmark.py:17, convert_eval_rms.py:1).  The implementation lives in the package."""
from triton_b200.convert_module import convert_ir_to_triton  # noqa: F401

__all__ = ["convert_ir_to_triton"]
