"""The other halves of the branching wrappers on the GPU, through the C ABI, against the CPU
oracle: softmax attention (reference layers.py:105-130) and Conv1d attention (layers.py:477-500).

Tolerances: float32 1e-4 relative; bfloat16 2e-2 relative against the float32 oracle on the
same bfloat16-rounded inputs and weights.
"""
import math

import pytest
import torch

import convnn_b200
from convnn_b200 import _capi
from oracle.convnn_oracle import bf16_round, conv1d_attention, softmax_attention
from gpu_util import DEV, rel_err

pytestmark = pytest.mark.gpu


def _uni(shape, fan_in, g):
    return (torch.rand(shape, generator=g) * 2 - 1) / math.sqrt(fan_in)


ATTN_CASES = [
    # B, T, D, H, dtype          (bfloat16 with T <= 256 and d_k % 16 == 0: the tensor-core kernel)
    (2, 197, 384, 12, torch.bfloat16),      # the ViT-Base BranchAttention half: d_k = 32
    (3, 197, 96, 3, torch.bfloat16),
    (2, 65, 48, 3, torch.bfloat16),         # d_k = 16, one row tile
    (1, 256, 128, 1, torch.bfloat16),       # d_k = 128, full 256-token tile
    (2, 130, 192, 2, torch.bfloat16),       # d_k = 96: three 32-channel chunks
    (2, 300, 64, 2, torch.bfloat16),        # more than 256 tokens: SIMT kernel
    (2, 197, 96, 3, torch.float32),
    (2, 40, 40, 2, torch.float32),          # d_k = 20
]


@pytest.mark.parametrize("B,T,D,H,dtype", ATTN_CASES)
def test_softmax_attention_matches_oracle(B, T, D, H, dtype):
    g = torch.Generator().manual_seed(B * 100 + T + D)
    w = {f"W_{n}.weight": _uni((D, D), D, g) * (3.0 if n in "qk" else 1.0) for n in "qkvo"}
    x = torch.randn(B, T, D, generator=g)
    if dtype == torch.bfloat16:
        w = {k: bf16_round(v) for k, v in w.items()}
        x = bf16_round(x)
    m = convnn_b200.MultiHeadAttention(D, H, 0.0)
    m.load_state_dict(w, strict=True)
    m = m.eval().to(DEV, dtype)
    with torch.no_grad():
        y = m(x.to(DEV, dtype))
        # channel-slice input and output, as MultiHeadBranchingAttention uses it
        wide = torch.zeros(B, T, D + 16, device=DEV, dtype=dtype)
        wide[:, :, 16:] = x.to(DEV, dtype)
        dst = torch.full((B, T, D + 24), 5.0, device=DEV, dtype=dtype)
        m(wide[:, :, 16:], out=dst[:, :, 8:8 + D])
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    want = softmax_attention(x, w, H)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert rel_err(y, want) < tol
    assert torch.equal(dst[:, :, 8:8 + D], y)
    assert bool((dst[:, :, :8] == 5.0).all()) and bool((dst[:, :, 8 + D:] == 5.0).all())


CONV_CASES = [
    # B, T, D, H, kernel_size, dtype
    (2, 197, 96, 3, 9, torch.bfloat16),     # d_k = 32: unfold + tensor-core GEMM
    (2, 197, 48, 3, 5, torch.bfloat16),     # d_k = 16
    (2, 197, 384, 12, 9, torch.bfloat16),
    (2, 65, 40, 1, 4, torch.bfloat16),      # d_k = 40 (SIMT kernel), even kernel size
    (2, 197, 96, 3, 9, torch.float32),
    (3, 65, 24, 1, 4, torch.float32),
    (2, 33, 32, 2, 1, torch.float32),
]


@pytest.mark.parametrize("B,T,D,H,ks,dtype", CONV_CASES)
def test_conv1d_attention_matches_oracle(B, T, D, H, ks, dtype):
    g = torch.Generator().manual_seed(B * 100 + T + D + ks)
    dk = D // H
    w = {"W_x.weight": _uni((D, D), D, g), "W_x.bias": _uni((D,), D, g),
         "conv.weight": _uni((dk, dk, ks), dk * ks, g), "conv.bias": _uni((dk,), dk * ks, g),
         "W_o.weight": _uni((D, D), D, g), "W_o.bias": _uni((D,), D, g)}
    x = torch.randn(B, T, D, generator=g)
    if dtype == torch.bfloat16:
        w = {k: bf16_round(v) for k, v in w.items()}
        x = bf16_round(x)
    m = convnn_b200.MultiHeadConv1dAttention(D, H, ks)
    m.load_state_dict(w, strict=True)
    m = m.eval().to(DEV, dtype)
    with torch.no_grad():
        y = m(x.to(DEV, dtype))
        y2 = m(x.to(DEV, dtype))
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    assert torch.equal(y, y2)
    want = conv1d_attention(x, w, H, ks)
    assert rel_err(y, want) < (1e-4 if dtype == torch.float32 else 2e-2)


def test_branching_modules_fold_the_skip_connection():
    """residual + layer(x) from one call equals the two-step result bit for bit."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 197, 96, generator=g).to(DEV, torch.bfloat16)
    for m in (convnn_b200.MultiHeadBranchingAttention(96, 3, 0.0, 9, "all", -1, 0, "cosine", 197, False, "standard"),
              convnn_b200.MultiHeadBranchingConv(96, 3, 0.0, 5, 9, "all", -1, 0, "cosine")):
        m = m.eval().to(DEV, torch.bfloat16)
        with torch.no_grad():
            y = m(x)
            z = m(x, residual=x)
        assert torch.equal(z, x + y)
