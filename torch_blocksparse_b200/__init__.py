"""B200-native block-sparse MatMul / Softmax / sparse self-attention.

Same public names as the reference package (torch_blocksparse/__init__.py:1-5
for the ops on this path, plus the attention wrapper of
deepspeedsparseselfattention.py, also exported as SparseSelfAttention).
"""
from .softmax import Softmax
from .matmul import MatMul, Linear
from .attention import DeepSpeedSparseSelfAttention, SparseSelfAttention, SparsityConfig
from .mha import MultiheadAttention, replace_mha, make_layout
from .host import HostAttention
from . import layouts

__all__ = ['Softmax', 'MatMul', 'Linear', 'DeepSpeedSparseSelfAttention', 'SparseSelfAttention',
           'SparsityConfig', 'MultiheadAttention', 'replace_mha', 'make_layout', 'HostAttention', 'layouts']
