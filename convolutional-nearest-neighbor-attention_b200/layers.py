"""Drop-in ``nn.Module``s for the reference's ConvNN-Attention layers.

Same constructor arguments, ``state_dict`` keys and ``forward(x)`` signature as
``MultiHeadConvNNAttention`` (reference layers.py:132-321), ``MultiHeadBranchingAttention``
(layers.py:580-652) and ``MultiHeadBranchingConv`` (layers.py:502-578), so a reference
checkpoint loads with ``strict=True`` and the reference's ``vit.py`` can construct them
in place of its own.  The ConvNN path runs in libconvnn_b200 (CUDA, sm_100a); it is
forward-only (inference) and has no CPU implementation.  The other halves of the branching
wrappers (softmax attention, Conv1d attention) and ``pointwise_linear`` run in the same
library; their modules only hold the parameters under the reference's names.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import ops
from .ops import LayerSpec


class MultiHeadConvNNAttention(nn.Module):
    def __init__(self, d_hidden, num_heads, attention_dropout, K, sampling_type, num_samples, sample_padding,
                 magnitude_type, seq_length=197, coordinate_encoding=False, convolution_type='depthwise',
                 softmax_topk_val=True):
        super().__init__()
        assert d_hidden % num_heads == 0, "d_hidden must be divisible by num_heads"
        self.d_hidden = d_hidden
        self.num_heads = num_heads
        self.attention_dropout = attention_dropout
        self.d_k = d_hidden // num_heads
        self.K = K
        self.seq_length = seq_length
        self.sampling_type = sampling_type
        self.num_samples = int(num_samples)
        self.sample_padding = int(sample_padding) if sampling_type == 'spatial' else 0
        self.magnitude_type = magnitude_type
        self.maximum = magnitude_type in ('cosine', 'matmul')
        self.coordinate_encoding = coordinate_encoding
        self.convolution_type = convolution_type
        self.softmax_topk_val = softmax_topk_val
        self.INF = 1.1
        self.NEG_INF = -0.1

        self.W_q = nn.Linear(d_hidden, d_hidden, bias=False)
        self.W_k = nn.Linear(d_hidden, d_hidden, bias=False)
        self.W_v = nn.Linear(d_hidden, d_hidden, bias=False)
        self.W_o = nn.Linear(d_hidden, d_hidden, bias=False)
        self.dropout = nn.Dropout(attention_dropout)

        self.in_channels = self.d_k + 1 if coordinate_encoding else self.d_k
        self.out_channels = self.d_k
        C, dk = self.in_channels, self.d_k
        # Parameter containers only (never called): they give the reference's state_dict
        # keys and its construction-time errors, e.g. depthwise + coordinate_encoding.
        if convolution_type == 'standard':
            self.conv = nn.Conv1d(C, dk, kernel_size=K, stride=K, padding=0, bias=False)
        elif convolution_type == 'depthwise':
            self.conv = nn.Conv1d(C, dk, kernel_size=K, stride=K, padding=0, groups=C, bias=False)
            self.conv.weight.data.fill_(1.0)
        elif convolution_type == 'depthwise-separable':
            self.conv = nn.Sequential(
                nn.Conv1d(C, C, kernel_size=K, stride=K, padding=0, groups=C, bias=False),
                nn.Conv1d(C, dk, kernel_size=1, stride=1, padding=0, bias=False))
        # (any other string leaves the module without a conv, as in the reference)

        self._candidate_override: Optional[torch.Tensor] = None
        self.stage_timer = None   # callable(label): records a CUDA event between the stage calls
        self._packed = None
        self._packed_key = None
        self._spatial_cache = {}

    # -- host-side helpers --------------------------------------------------------------
    @property
    def candidate_override(self) -> Optional[torch.Tensor]:
        """Fixes the candidate set of the sampled modes (instead of a fresh draw per call)."""
        return self._candidate_override

    @candidate_override.setter
    def candidate_override(self, cand: Optional[torch.Tensor]) -> None:
        if cand is not None:
            ops.check_candidates(cand)      # negatives here; the upper bound once T is known
        self._candidate_override = cand
        self._override_checked_T = None

    def _spec(self) -> LayerSpec:
        return LayerSpec(self.d_hidden, self.num_heads, self.K, self.sampling_type, self.magnitude_type,
                         self.convolution_type, self.softmax_topk_val, self.coordinate_encoding,
                         self.seq_length)

    def _conv_params(self):
        if self.convolution_type == 'depthwise-separable':
            return (self.conv[0].weight, self.conv[1].weight)
        return (self.conv.weight,)

    def packed_weights(self, dtype, device):
        params = (self.W_q.weight, self.W_k.weight, self.W_v.weight, self.W_o.weight) + self._conv_params()
        key = (dtype, device) + tuple((p.data_ptr(), p._version) for p in params)
        if self._packed_key != key:
            self._packed = ops.pack_weights(self._spec(), self.W_q.weight, self.W_k.weight, self.W_v.weight,
                                            self.W_o.weight, self._conv_params(), dtype, device)
            self._packed_key = key
        return self._packed

    def candidates(self, T: int, device) -> Optional[torch.Tensor]:
        """Candidate token indices for this call, drawn as the reference draws them
        (layers.py:284, 297) unless ``candidate_override`` is set."""
        if self.sampling_type == 'all':
            return None
        if self._candidate_override is not None:
            if getattr(self, "_override_checked_T", None) != T:
                ops.check_candidates(self._candidate_override, T)    # once per sequence length
                self._override_checked_T = T
            return self._candidate_override.to(device)
        if self.sampling_type == 'random':
            return torch.randperm(T, device=device)[:self.num_samples]
        if self.sampling_type == 'spatial':
            key = (T, str(device))
            if key not in self._spatial_cache:
                self._spatial_cache[key] = torch.linspace(
                    0 + self.sample_padding, T - self.sample_padding - 1, self.num_samples, device=device).long()
            return self._spatial_cache[key]
        raise ValueError("Invalid sampling_type. Must be one of ['all', 'random', 'spatial']")

    def _check_mode(self, x):
        if not x.is_cuda:
            raise RuntimeError("convnn_b200.MultiHeadConvNNAttention runs on CUDA (sm_100a) only; "
                               "there is no CPU path")
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            raise RuntimeError("convnn_b200 is forward-only: call it under torch.no_grad() "
                               "(training / backward is outside this library)")
        if self.training and self.attention_dropout > 0:
            raise RuntimeError("convnn_b200 is forward-only: dropout > 0 needs module.eval()")
        if self.magnitude_type not in ('cosine', 'matmul', 'euclidean'):
            raise ValueError(f"unknown magnitude_type {self.magnitude_type!r}")

    def forward(self, x, out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None):
        """``layer(x)``; with ``residual`` the caller's skip connection is folded into the last
        store (``residual + layer(x)``), with ``out`` the result is written in place."""
        self._check_mode(x)
        B, T, D = x.shape
        cand = self.candidates(T, x.device)
        packed = self.packed_weights(x.dtype, x.device)
        if self.stage_timer is not None:
            return self._forward_staged(x, packed, cand, out, residual)
        return ops.forward(self._spec(), x, packed, cand, out=out, residual=residual)

    def prenorm_supported(self, x) -> bool:
        """Whether ``forward_prenorm`` takes this input (bfloat16, sampling 'all', a K/V/Q weight tile
        that stays resident in shared memory); otherwise the caller normalises and calls ``forward``."""
        return x.is_cuda and self.prenorm_supported_shape(x.shape[0], x.shape[1], x.dtype)

    def prenorm_supported_shape(self, B: int, T: int, dtype) -> bool:
        """``prenorm_supported`` for a CUDA input (B, T, d_hidden) of ``dtype`` that does not exist yet."""
        return (dtype == torch.bfloat16 and self.stage_timer is None and
                ops.prenorm_forward_supported(self._spec(), B, T, dtype))

    def forward_prenorm(self, x, moments, norm: nn.LayerNorm, residual: Optional[torch.Tensor] = None,
                        want_moments: bool = False, skip_out_proj: bool = False):
        """``layer(norm(x))`` (``+ residual``) from the rows ``x`` BEFORE ``norm`` and their moments,
        the LayerNorm folded into the K/V/Q projection.  Returns (out, moments of out or None).  With
        ``skip_out_proj`` (num_heads = 1) the result is the layer's output BEFORE ``W_o``, for a caller
        that fuses the projection into what follows (``ops.outproj_mlp`` with ``self.packed_w_o``)."""
        self._check_mode(x)
        w_qkv, w_conv, w_pw, w_o = self.packed_weights(x.dtype, x.device)
        if getattr(self, "_folded", None) is None:
            self._folded = _PackedParams()
        wf, wx = self._folded.get((w_qkv, norm.weight, norm.bias), x.dtype, x.device, lambda: ops.fold_layernorm(
            w_qkv.view(-1, w_qkv.shape[-1]), None, norm.weight.detach().to(x.device, x.dtype),
            norm.bias.detach().to(x.device, x.dtype)))
        self.packed_w_o = w_o
        return ops.prenorm_forward(self._spec(), x, moments, norm.eps, (wf, wx, w_conv, w_pw, None if skip_out_proj else w_o),
                                   residual=residual, want_moments=want_moments)

    def _forward_staged(self, x, packed, cand, out, residual=None):
        """The same kernels in the same order as ``convnn_b200_forward``, issued through the
        four stage entry points so a profiler hook can bracket each with CUDA events."""
        spec, mark = self._spec(), self.stage_timer
        w_qkv, w_conv, w_pw, w_o = packed
        mark("begin")
        q, k, v, qs, ks = ops.qkv_proj(spec, x, w_qkv, cand)
        mark("qkv_proj")
        idx, val = ops.sim_topk(spec, q, k, qs, ks, cand)
        mark("sim_topk")
        o = ops.gather_conv(spec, v, idx, val, w_conv, w_pw, S=q.shape[1])
        mark("gather_conv")
        y = ops.out_proj(spec, o, w_o, out=out, S=q.shape[1], residual=residual)
        mark("out_proj")
        return y


def _library_call(x: torch.Tensor, what: str) -> None:
    if not x.is_cuda:
        raise RuntimeError(f"convnn_b200.{what} runs on CUDA (sm_100a) only; there is no CPU path")
    if torch.is_grad_enabled() and x.requires_grad:
        raise RuntimeError("convnn_b200 is forward-only: call it under torch.no_grad() "
                           "(training / backward is outside this library)")


class _PackedParams:
    """Kernel-side copies of a module's parameters, rebuilt when a parameter changes."""

    def __init__(self):
        self._key, self._val = None, None

    def get(self, params, dtype, device, build):
        key = (dtype, device) + tuple((p.data_ptr(), p._version) for p in params)
        if key != self._key:
            self._val, self._key = build(), key
        return self._val


class MultiHeadAttention(nn.Module):
    """Softmax attention half of MultiHeadBranchingAttention (reference layers.py:90-130):
    bias-free W_q/W_k/W_v/W_o, softmax(QK^T / sqrt(d_k)) V.  The modules hold the parameters (same
    ``state_dict`` keys as the reference); the forward runs in libconvnn_b200: one packed
    three-output projection, the softmax-attention kernel, the output projection."""

    def __init__(self, d_hidden, num_heads, attention_dropout):
        super().__init__()
        assert d_hidden % num_heads == 0, "d_hidden must be divisible by num_heads"
        self.d_hidden, self.num_heads, self.d_k = d_hidden, num_heads, d_hidden // num_heads
        self.dropout = nn.Dropout(attention_dropout)
        self.W_q = nn.Linear(d_hidden, d_hidden, bias=False)
        self.W_k = nn.Linear(d_hidden, d_hidden, bias=False)
        self.W_v = nn.Linear(d_hidden, d_hidden, bias=False)
        self.W_o = nn.Linear(d_hidden, d_hidden, bias=False)
        self._packed = _PackedParams()

    def forward(self, x, mask=None, out: Optional[torch.Tensor] = None):
        _library_call(x, "MultiHeadAttention")
        if mask is not None:
            raise RuntimeError("convnn_b200.MultiHeadAttention takes no mask (the reference's ViT never passes one)")
        if self.training and self.dropout.p > 0:
            raise RuntimeError("convnn_b200 is forward-only: dropout > 0 needs module.eval()")
        params = (self.W_q.weight, self.W_k.weight, self.W_v.weight, self.W_o.weight)
        w_qkv, w_o = self._packed.get(params, x.dtype, x.device, lambda: (
            torch.stack([p.detach().to(x.device, x.dtype) for p in params[:3]]).contiguous(),
            self.W_o.weight.detach().to(x.device, x.dtype).contiguous()))
        return ops.softmax_attention(x, w_qkv, w_o, self.num_heads, out=out)


class MultiHeadConv1dAttention(nn.Module):
    """Conv1d half of MultiHeadBranchingConv (reference layers.py:452-500): Linear, per-head
    Conv1d(d_k, d_k, kernel_size, padding='same'), the reference's flat head reinterpretation,
    Linear.  Parameters as in the reference; the forward runs in libconvnn_b200."""

    def __init__(self, d_hidden, num_heads, kernel_size):
        super().__init__()
        assert d_hidden % num_heads == 0, "d_hidden must be divisible by num_heads"
        self.d_hidden, self.num_heads, self.d_k = d_hidden, num_heads, d_hidden // num_heads
        self.kernel_size, self.stride = kernel_size, 1
        self.W_x = nn.Linear(d_hidden, d_hidden)
        self.W_o = nn.Linear(d_hidden, d_hidden)
        self.in_channels = self.out_channels = self.d_k
        self.conv = nn.Conv1d(self.d_k, self.d_k, kernel_size=kernel_size, stride=1, padding="same")
        self._packed = _PackedParams()

    def forward(self, x, out: Optional[torch.Tensor] = None):
        _library_call(x, "MultiHeadConv1dAttention")
        params = (self.W_x.weight, self.W_x.bias, self.conv.weight, self.conv.bias, self.W_o.weight, self.W_o.bias)

        def build():
            cvt = lambda t: t.detach().to(x.device, x.dtype).contiguous()
            # (d_k out, d_k in, kernel_size) -> (d_k out, kernel_size, d_k in): a (d_k, kernel_size * d_k) matrix
            return (cvt(self.W_x.weight), cvt(self.W_x.bias), cvt(self.conv.weight.permute(0, 2, 1)),
                    cvt(self.conv.bias), cvt(self.W_o.weight), cvt(self.W_o.bias))
        w_x, b_x, w_c, b_c, w_o, b_o = self._packed.get(params, x.dtype, x.device, build)
        return ops.conv1d_attention(x, w_x, b_x, w_c, b_c, w_o, b_o, self.num_heads, self.kernel_size, out=out)


class _Branching(nn.Module):
    def _init_common(self, d_hidden, num_heads, attention_dropout, K, sampling_type, num_samples,
                     sample_padding, magnitude_type, seq_length, coordinate_encoding, convolution_type,
                     softmax_topk_val, branch_ratio):
        self.d_hidden = d_hidden
        self.num_heads = num_heads
        self.attention_dropout = attention_dropout
        self.K = K
        self.sampling_type = sampling_type
        self.num_samples = int(num_samples)
        self.sample_padding = int(sample_padding) if sampling_type == 'spatial' else 0
        self.magnitude_type = magnitude_type
        self.seq_length = seq_length
        self.coordinate_encoding = coordinate_encoding
        self.branch_ratio = branch_ratio
        self.d_hidden_convnn = int(branch_ratio * d_hidden)
        if branch_ratio != 0:
            self.convnn = MultiHeadConvNNAttention(
                d_hidden=self.d_hidden_convnn, num_heads=num_heads, attention_dropout=attention_dropout, K=K,
                sampling_type=sampling_type, num_samples=num_samples, sample_padding=sample_padding,
                magnitude_type=magnitude_type, seq_length=seq_length, coordinate_encoding=coordinate_encoding,
                convolution_type=convolution_type, softmax_topk_val=softmax_topk_val)

    def _two_branches(self, x, other, residual=None):
        """Both branches read their channel slice of x in place and write their slice of the
        concat buffer in place (no slice copy in, no cat copy out); then pointwise_linear with
        its bias, and the caller's skip connection if given, folded into one GEMM epilogue
        (reference layers.py:574-577, 648-651; vit.py:264)."""
        dc = self.d_hidden_convnn
        cat = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        self.convnn(x[:, :, :dc], out=cat[:, :, :dc])
        other(x[:, :, dc:], out=cat[:, :, dc:])
        pw = self.pointwise_linear
        return ops.linear(cat, pw.weight, pw.bias, residual=residual)


class MultiHeadBranchingAttention(_Branching):
    def __init__(self, d_hidden, num_heads, attention_dropout, K, sampling_type, num_samples, sample_padding,
                 magnitude_type, seq_length=197, coordinate_encoding=False, convolution_type='depthwise',
                 softmax_topk_val=True, branch_ratio=0.5):
        super().__init__()
        self._init_common(d_hidden, num_heads, attention_dropout, K, sampling_type, num_samples, sample_padding,
                          magnitude_type, seq_length, coordinate_encoding, convolution_type, softmax_topk_val,
                          branch_ratio)
        self.d_hidden_attention = d_hidden - self.d_hidden_convnn
        if branch_ratio != 1:
            self.attention = MultiHeadAttention(self.d_hidden_attention, num_heads, attention_dropout)
        self.pointwise_linear = nn.Linear(d_hidden, d_hidden)

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        # The reference swaps the degenerate cases (ratio 0 calls the ConvNN branch that was
        # not built and vice versa, layers.py:643-646) and fails with AttributeError; so do we.
        if self.branch_ratio == 0:
            y = self.convnn(x)
        elif self.branch_ratio == 1:
            y = self.attention(x)
        else:
            return self._two_branches(x, self.attention, residual)
        return y if residual is None else residual + y


class MultiHeadBranchingConv(_Branching):
    def __init__(self, d_hidden, num_heads, attention_dropout, kernel_size, K, sampling_type, num_samples,
                 sample_padding, magnitude_type, seq_length=197, coordinate_encoding=False,
                 convolution_type='depthwise', softmax_topk_val=True, branch_ratio=0.5):
        super().__init__()
        self.kernel_size = kernel_size
        self._init_common(d_hidden, num_heads, attention_dropout, K, sampling_type, num_samples, sample_padding,
                          magnitude_type, seq_length, coordinate_encoding, convolution_type, softmax_topk_val,
                          branch_ratio)
        self.d_hidden_conv1d = d_hidden - self.d_hidden_convnn
        if branch_ratio != 1:
            self.conv1d = MultiHeadConv1dAttention(self.d_hidden_conv1d, num_heads, kernel_size)
        self.pointwise_linear = nn.Linear(d_hidden, d_hidden)

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        if self.branch_ratio == 0:
            y = self.conv1d(x)
        elif self.branch_ratio == 1:
            y = self.convnn(x)
        else:
            return self._two_branches(x, self.conv1d, residual)
        return y if residual is None else residual + y
