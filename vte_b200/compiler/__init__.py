from .codegen import CodegenEngine

__all__ = ["CodegenEngine"]
