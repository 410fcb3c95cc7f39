"""mircuda_b200 — sm_100a (B200) kernels for mircuda's quantized-matmul hot path.

The product is ``libmircuda_b200.so`` (C ABI in ``include/mircuda_b200.h``); this package
builds it (``mircuda_b200.build``), loads it (``mircuda_b200._lib``) and mirrors the
reference's host-side Spec/Plan interface (``mircuda_b200.plans``). There is no CPU path:
importing ``plans`` and calling anything without the built library raises.
"""

__all__ = ["build", "plans"]
