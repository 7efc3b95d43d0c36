"""ramnet_ops for B200: the reference package's operator API
(``random_access_memory_attention``, ``topk_addr``) over hand-written sm_100a kernels."""
from .ram_attn import random_access_memory_attention, topk_addr

__all__ = [
    'random_access_memory_attention',
    'topk_addr',
]
