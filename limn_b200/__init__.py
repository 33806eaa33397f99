"""limn_b200: B200-native (sm_100a) kernels for limn's fused-attention CUSTOM ops.

    import limn, limn_b200
    limn.set_device("cuda")
    limn_b200.install(limn.device.active())   # "sdpa", "sdpa_bwd_q", "sdpa_bwd_kv" now run here

The kernels live in a prebuilt shared library (python -m limn_b200.build) behind the C ABI
in include/limn_b200.h; this package is the ctypes binding and the registry builders.
"""

from limn_b200.registry import BUILDERS, NAMES, install

__all__ = ["BUILDERS", "NAMES", "install"]
