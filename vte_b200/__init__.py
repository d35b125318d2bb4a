"""B200-native replacement for VTE's split-KV decode-attention path.

The package is numpy + ctypes only.  Device work goes through `libvteb200.so`
(a C-ABI shim over the CUDA runtime/driver) and hand-written sm_100a kernels;
there is no CPU fallback: without the library and a CUDA device the runtime
raises.
"""
__version__ = "0.1.0"
