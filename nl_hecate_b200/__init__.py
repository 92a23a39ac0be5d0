"""NL_Hecate hot path for B200 (sm_100a): memory-rule kernel pairs (Titans LMM,
Delta / DGD, Hebbian; exact and frozen-M0 chunkwise), sliding-window attention
forward/backward and the AdamW outer-parameter step, behind the reference's C
ABI (include/nlh_ffi.h). CUDA only: importing is cheap, every op raises if
libnlh_b200.so is not built.
"""
from . import ffi  # noqa: F401

__all__ = ["ffi"]
