from .split_kv_attention import SplitKVAttentionDispatcher

__all__ = ["SplitKVAttentionDispatcher"]
