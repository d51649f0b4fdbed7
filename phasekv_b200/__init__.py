"""phasekv_b200: PhaseKV's stage-B hot path (sub-byte quantise+pack and the three-tier split-K
decode attention) as hand-written sm_100a CUDA behind a C ABI, with the reference's Python
entry points on top.  There is no Triton, no multi-backend dispatch and no CPU fallback."""

__version__ = "0.1.0"
