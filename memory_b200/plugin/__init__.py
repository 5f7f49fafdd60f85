"""Kernel plugin in the shape the reference loads by file path (memory_transformer/token_routing_kernel.py:58-142)."""
from .kernel_b200 import (FSA_WEIGHTED_SEMANTICS, FSA_topk_sparse_attention_bthd,
                          FSA_topk_sparse_attention_weighted_bthd, install_plugin_files)

__all__ = ["FSA_topk_sparse_attention_bthd", "FSA_topk_sparse_attention_weighted_bthd", "FSA_WEIGHTED_SEMANTICS",
           "install_plugin_files"]
