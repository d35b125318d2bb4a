"""Limits and environment switches of the bridge.

Mirrors the constants the reference keeps in vte/config.py (allocation cap,
VRAM usage limit, grid limit, cache-line size) with B200 values where the
reference's were sized for an 8 GB desktop card.
"""
import os

MAX_ALLOCATION_SIZE = 160 * 1024 ** 3      # one cudaMalloc; a B200 holds 180 GB
VRAM_USAGE_LIMIT = 0.95                    # refuse to go past 95 % of device memory
MAX_GRID_DIMENSIONS = (2 ** 31) - 1        # total CTAs of one launch
CACHE_LINE_SIZE = 128                      # slab sub-allocation alignment (bytes)
DEFAULT_SYNC_TIMEOUT_S = 30.0              # host watchdog around synchronize()

ENV_DISABLE_SPLITKV = "VTE_DISABLE_ATTN_SPLITKV"
ENV_DEVICE_INDEX = "VTE_DEVICE_INDEX"
ENV_COMPAT_KERNELS = "VTE_B200_COMPAT_KERNELS"   # launch the reference-geometry kernels
ENV_NO_PDL = "VTE_B200_NO_PDL"                   # disable programmatic dependent launch


def env_flag(name: str) -> bool:
    return bool(os.environ.get(name))
