"""ramnet_ops for B200: the reference package's operator API
(``random_access_memory_attention``, ``topk_addr``) over hand-written sm_100a kernels."""
from .decode_graph import DecodeGraph
from .ram_attn import random_access_memory_attention, topk_addr

__all__ = [
    'DecodeGraph',
    'random_access_memory_attention',
    'topk_addr',
]
