from .errors import VTEError, CudaSafetyError, CudaRuntimeError, MemoryGuardianOOMError, HIPSafetyError, HIPRuntimeError
from .cuda_runtime import CudaRuntime
from .memory import SlabAllocator, MemoryRegion, MemoryBlock

__all__ = ["VTEError", "CudaSafetyError", "CudaRuntimeError", "MemoryGuardianOOMError",
           "HIPSafetyError", "HIPRuntimeError", "CudaRuntime", "SlabAllocator", "MemoryRegion",
           "MemoryBlock"]
