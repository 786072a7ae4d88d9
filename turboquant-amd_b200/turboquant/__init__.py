"""TurboQuant hot paths for NVIDIA B200 (sm_100a).

Drop-in for the `turboquant.core` / `turboquant.kernels` / `turboquant.integration`
entry points of andyluo7/turboquant-amd that sit on the KV-compression and
packed decode-attention paths.  All GPU work runs in hand-written CUDA kernels
reached through the C-ABI library `libtq_b200.so`; there is no CPU fallback.
"""

__version__ = "0.1.0"
