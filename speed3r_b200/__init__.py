"""B200 (sm_100a) implementation of Speed3R's dual-branch sparse global attention.

``SparseFlashAttentionRope`` is the drop-in module; ``ops`` holds the reference-named operator
functions; ``_lib`` binds the C-ABI library declared in include/speed3r_b200.h.
"""
from .sparse_attention import RoPE2D, SparseFlashAttentionRope  # noqa: F401
from .ops import (flash_attn_topk_func, pool_tokens, sel_attn_merge,  # noqa: F401
                  topk_blocksparse_attention)
from .host_pipeline import HostPipeline  # noqa: F401

__all__ = ["SparseFlashAttentionRope", "RoPE2D", "flash_attn_topk_func", "topk_blocksparse_attention",
           "pool_tokens", "sel_attn_merge", "HostPipeline"]
