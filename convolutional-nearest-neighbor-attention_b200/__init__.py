"""convnn_b200 — B200 (sm_100a) implementation of the ConvNN-Attention forward path.

Import as ``convnn_b200`` (a shim at the repository root aliases this package, whose
directory name is not a Python identifier).
"""
from . import build, _capi, ops, layers, vit, dropin, sharded, lanes  # noqa: F401
from .lanes import ForwardLanes  # noqa: F401
from .layers import (MultiHeadAttention, MultiHeadBranchingAttention, MultiHeadBranchingConv,  # noqa: F401
                     MultiHeadConv1dAttention, MultiHeadConvNNAttention)
from .ops import LayerSpec  # noqa: F401
from .vit import ViT, make_args  # noqa: F401
from .dropin import install, uninstall  # noqa: F401

__all__ = ["MultiHeadConvNNAttention", "MultiHeadBranchingAttention", "MultiHeadBranchingConv",
           "MultiHeadAttention", "MultiHeadConv1dAttention", "ViT", "make_args", "LayerSpec",
           "install", "uninstall", "ops", "build"]
