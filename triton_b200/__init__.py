"""triton_b200 — B200-native (sm_100a) kernel backend for Trinity's fused attention-block operators.

Public pieces:
  convert_module.convert_ir_to_triton  drop-in for the reference's IR -> module-source entry point
  ops                                  operators on torch CUDA tensors (thin C-ABI calls)
  _lib                                 ctypes binding of libtrinity_b200.so (include/trinity_b200.h)
"""
__all__ = ["ops", "_lib"]
