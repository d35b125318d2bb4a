"""Exception types of the bridge.

Same hierarchy as vte/bridge/errors.py and vte/bridge/hip_runtime.py:13-15:
rejected arguments raise a *safety* error before the driver is touched, a
non-zero driver status raises a *runtime* error, and the 95 % memory cap raises
the OOM subclass of the safety error.  The HIP-named aliases let code written
against the reference's names catch the same conditions.
"""


class VTEError(Exception):
    pass


class CudaSafetyError(VTEError):
    """A host-side check refused the call; nothing reached the device."""


class CudaRuntimeError(VTEError):
    """The CUDA runtime/driver (or a kernel's status word) reported a failure."""

    def __init__(self, message: str, code: int = 0):
        super().__init__(message)
        self.code = code


class MemoryGuardianOOMError(CudaSafetyError):
    """The allocation would pass the device-memory usage limit, or cudaMalloc ran out."""


HIPSafetyError = CudaSafetyError
HIPRuntimeError = CudaRuntimeError
