"""Stage-B kernels: real sub-byte packing and the fused three-tier decode attention.

Module paths mirror the reference's ``src/phasekv/kernels`` package (``packing``,
``attention_triton``, ``launch_config``, ``reference``) so its callers can import from here
unchanged.  Importing this package needs no GPU; calling a kernel does.
"""
from . import launch_config, packing, tiers  # noqa: F401

__all__ = ["packing", "launch_config", "tiers", "attention_cuda", "attention_triton", "reference"]
