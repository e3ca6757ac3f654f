"""B200 (sm_100a) MonarchAttention forward library behind the reference's module API."""
from .host_pipeline import monarch_attention_b200_host
from .monarch_attention import MonarchAttention, PadType, monarch_attention_b200, register_impl

__all__ = ["MonarchAttention", "PadType", "monarch_attention_b200", "monarch_attention_b200_host", "register_impl"]
