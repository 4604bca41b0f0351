"""ViT harness around the ConvNN-Attention layers.

Mirrors the reference model's module tree and ``state_dict`` keys (reference vit.py:22-270)
so that a reference checkpoint loads with ``strict=True`` and whole-model throughput can be
measured without the reference checkout.  The ``nn.Module``s here only hold the parameters:
on CUDA, in float32 or bfloat16 and without autograd, every operation of the forward (patch
unfold and projection, LayerNorm, the attention block, both MLP layers with GELU and the skip
connections, the classifier) runs in libconvnn_b200.  Any other call (CPU tensors, autograd,
dropout in training mode) takes the modules' ordinary torch forward for the encoder shell and
is refused by the ConvNN layers themselves.
"""
from __future__ import annotations

import math
from types import SimpleNamespace

import torch
import torch.nn as nn

from . import ops
from .layers import MultiHeadBranchingAttention, MultiHeadBranchingConv, MultiHeadConvNNAttention, _PackedParams

_DEFAULTS = dict(layer="ConvNNAttention", patch_size=16, num_layers=12, num_heads=3, d_hidden=192, d_mlp=768,
                 dropout=0.1, attention_dropout=0.1, convolution_type="depthwise", softmax_topk_val=True, K=9,
                 sampling_type="all", num_samples=-1, sample_padding=0, magnitude_type="matmul",
                 coordinate_encoding=False, branch_ratio=0.5, kernel_size=9, device="cuda",
                 img_size=(3, 224, 224), num_classes=1000)


def make_args(**overrides) -> SimpleNamespace:
    """Namespace with the reference CLI's defaults (main.py:28-113) plus overrides."""
    a = dict(_DEFAULTS)
    a.update(overrides)
    return SimpleNamespace(**a)


class PatchEmbedding(nn.Module):
    def __init__(self, d_hidden, img_size, patch_size, n_channels=3):
        super().__init__()
        self.linear_projection = nn.Conv2d(n_channels, d_hidden, kernel_size=patch_size, stride=patch_size)
        self.norm = nn.LayerNorm(d_hidden)

    def forward(self, x):
        return self.norm(self.linear_projection(x).flatten(2).transpose(1, 2))


def _library_path(x: torch.Tensor) -> bool:
    """The fused encoder ops cover CUDA float32 / bfloat16 inference (and, for the model input,
    8-bit images that the patch unfold normalises on the way)."""
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.uint8) and not torch.is_grad_enabled()


class PositionalEncoding(nn.Module):
    def __init__(self, d_hidden, max_seq_length):
        super().__init__()
        self.cls_tokens = nn.Parameter(torch.randn(1, 1, d_hidden))
        pos = torch.arange(0, max_seq_length, dtype=torch.float).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_hidden, 2).float() * (-math.log(10000.0) / d_hidden))
        pe = torch.zeros(max_seq_length, d_hidden)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        self.register_buffer('pe', pe.unsqueeze(0))

    def forward(self, x):
        x = torch.cat((self.cls_tokens.expand(x.shape[0], -1, -1), x), dim=1)
        return x + self.pe[:, :x.size(1)]


class TransformerEncoder(nn.Module):
    def __init__(self, args, d_hidden, d_mlp, num_heads, dropout, attention_dropout):
        super().__init__()
        common = dict(K=args.K, sampling_type=args.sampling_type, num_samples=args.num_samples,
                      sample_padding=args.sample_padding, magnitude_type=args.magnitude_type,
                      coordinate_encoding=args.coordinate_encoding, convolution_type=args.convolution_type,
                      softmax_topk_val=args.softmax_topk_val)
        if args.layer == "ConvNNAttention":
            self.attention = MultiHeadConvNNAttention(d_hidden, num_heads, attention_dropout, **common)
        elif args.layer == "BranchConv":
            self.attention = MultiHeadBranchingConv(d_hidden, num_heads, attention_dropout,
                                                    kernel_size=args.kernel_size, branch_ratio=args.branch_ratio,
                                                    **common)
        elif args.layer == "BranchAttention":
            self.attention = MultiHeadBranchingAttention(d_hidden, num_heads, attention_dropout,
                                                         branch_ratio=args.branch_ratio, **common)
        else:
            raise ValueError("Invalid layer type. convnn_b200 provides ['ConvNNAttention', 'BranchConv', "
                             "'BranchAttention']")
        self.norm1 = nn.LayerNorm(d_hidden)
        self.norm2 = nn.LayerNorm(d_hidden)
        self.dropout1 = nn.Dropout(dropout)
        self.dropout2 = nn.Dropout(dropout)
        self.mlp = nn.Sequential(nn.Linear(d_hidden, d_mlp), nn.GELU(), nn.Dropout(dropout),
                                 nn.Linear(d_mlp, d_hidden))
        # bfloat16 library path: fold norm1 / norm2 into the GEMMs that consume them where the shapes
        # allow (set to False for a LayerNorm kernel followed by the plain GEMM, the reference's order
        # of roundings)
        self.fold_layernorm = True
        self.fuse_mlp = True          # with the fold: norm2 + mlp + skip connection as one kernel where it is built
        # ... and the attention layer's W_o + skip connection in front of it (one head).  Built and parity-green,
        # but not faster inside the model (1.70 ms against 1.675 ms per cfg-2 batch on the same GPU): off by default.
        self.fuse_out_proj = False
        self._fc1_folded = _PackedParams()

    def forward(self, x):
        if _library_path(x) and not (self.training and (self.dropout1.p > 0 or self.dropout2.p > 0)):
            return self._forward_library(x)[0]
        x = x + self.dropout1(self.attention(self.norm1(x)))
        return x + self.dropout2(self.mlp(self.norm2(x)))

    def folds_norm1(self, x) -> bool:
        """Whether this block consumes un-normalised rows plus their moments (norm1 folded into the
        K/V/Q projection): the block before it then emits the moments from its last GEMM."""
        return x.is_cuda and self.folds_norm1_shape(x.shape[0], x.shape[1], x.dtype)

    def folds_norm1_shape(self, B: int, T: int, dtype) -> bool:
        """``folds_norm1`` for a CUDA input (B, T, d_hidden) of ``dtype`` that does not exist yet."""
        return (self.fold_layernorm and isinstance(self.attention, MultiHeadConvNNAttention) and
                self.attention.prenorm_supported_shape(B, T, dtype))

    def _forward_library(self, x, moments=None, want_moments=False):
        """The same block in libconvnn_b200: both Linear layers (GELU and the skip connections folded
        into their stores), the attention layer with its output projection (+ skip), and the two
        LayerNorms either as kernels of their own or, where the shapes allow (``fold_layernorm``),
        folded into the GEMMs that consume them: those read the un-normalised rows and their moments
        (sum, sum of squares), which the GEMM that wrote the rows emits from its epilogue.
        Returns (x, moments of x or None)."""
        n1, n2, fc1, fc2 = self.norm1, self.norm2, self.mlp[0], self.mlp[3]
        bf16 = x.dtype == torch.bfloat16
        fold_mlp = (self.fold_layernorm and bf16 and
                    ops.prenorm_linear_supported(fc1.out_features, fc1.in_features, True))
        m1 = None
        if self.folds_norm1(x):
            if moments is None:
                moments = ops.row_moments(x)
            if (fold_mlp and self.fuse_mlp and self.fuse_out_proj and self.attention.num_heads == 1 and
                    ops.prenorm_mlp_supported(fc1.in_features, fc1.out_features, 1)):
                # attention up to the gather / conv, then ONE kernel for W_o + skip + norm2 + mlp + skip
                o, _ = self.attention.forward_prenorm(x, moments, n1, skip_out_proj=True)
                wf, wx = self._fc1_folded.get((fc1.weight, fc1.bias, n2.weight, n2.bias), x.dtype, x.device,
                                              lambda: ops.fold_layernorm(fc1.weight, fc1.bias, n2.weight, n2.bias))
                return ops.outproj_mlp(o, self.attention.packed_w_o, x, n2.eps, wf, wx, fc2.weight, fc2.bias,
                                       want_moments=want_moments)
            x, m1 = self.attention.forward_prenorm(x, moments, n1, residual=x, want_moments=fold_mlp)
        else:
            xn = ops.layernorm(x, n1.weight, n1.bias, n1.eps)
            x = self.attention(xn, residual=x)       # skip connection folded into the layer's last store
        if fold_mlp:
            if m1 is None:
                m1 = ops.row_moments(x)
            wf, wx = self._fc1_folded.get((fc1.weight, fc1.bias, n2.weight, n2.bias), x.dtype, x.device,
                                          lambda: ops.fold_layernorm(fc1.weight, fc1.bias, n2.weight, n2.bias))
            if self.fuse_mlp and ops.prenorm_mlp_supported(fc1.in_features, fc1.out_features, m1.shape[0]):
                # the whole block in one kernel: the hidden activations never reach HBM
                return ops.prenorm_mlp(x, m1, n2.eps, wf, wx, fc2.weight, fc2.bias, want_moments=want_moments)
            h = ops.prenorm_linear(x, m1, n2.eps, wf, wx, gelu=True)
        else:
            xn = ops.layernorm(x, n2.weight, n2.bias, n2.eps)
            h = ops.linear(xn, fc1.weight, fc1.bias, gelu=True)
        if want_moments and bf16:
            return ops.linear_moments(h, fc2.weight, fc2.bias, residual=x)
        return ops.linear(h, fc2.weight, fc2.bias, residual=x), None


class ViT(nn.Module):
    def __init__(self, args):
        super().__init__()
        assert args.img_size[1] % args.patch_size == 0 and args.img_size[2] % args.patch_size == 0, \
            "img_size dimensions must be divisible by patch_size dimensions"
        assert args.d_hidden % args.num_heads == 0, "d_hidden must be divisible by n_heads"
        self.args = args
        self.d_hidden = args.d_hidden
        self.n_patches = (args.img_size[1] * args.img_size[2]) // (args.patch_size * args.patch_size)
        self.max_seq_length = self.n_patches + 1
        self.patch_embedding = PatchEmbedding(args.d_hidden, args.img_size[1:], (args.patch_size, args.patch_size),
                                              args.img_size[0])
        self.positional_encoding = PositionalEncoding(args.d_hidden, self.max_seq_length)
        self.transformer_encoder = nn.Sequential(*[
            TransformerEncoder(args, args.d_hidden, args.d_mlp, args.num_heads, args.dropout,
                               args.attention_dropout) for _ in range(args.num_layers)])
        self.classifier = nn.Linear(args.d_hidden, args.num_classes)
        self.device = getattr(args, "device", "cuda")
        # Normalisation applied to uint8 inputs (plain attributes, not buffers: the state_dict stays
        # the reference's).  Defaults: the ImageNet statistics of the reference's loader (dataset.py:23).
        self.pixel_mean = (0.485, 0.456, 0.406)
        self.pixel_std = (0.229, 0.224, 0.225)
        self._pixel_stats = None
        self.name = f"VIT {args.layer}"
        self.to(self.device)

    def forward(self, x):
        if _library_path(x):
            pe_mod, pemb = self.positional_encoding, self.patch_embedding
            mean = inv_std = None
            if x.dtype == torch.uint8:
                key = (tuple(self.pixel_mean), tuple(self.pixel_std), x.device)
                if self._pixel_stats is None or self._pixel_stats[0] != key:
                    self._pixel_stats = (key, torch.tensor(self.pixel_mean, dtype=torch.float32, device=x.device),
                                         1.0 / torch.tensor(self.pixel_std, dtype=torch.float32, device=x.device))
                _, mean, inv_std = self._pixel_stats
            blocks = list(self.transformer_encoder)
            act = pemb.linear_projection.weight.dtype if x.dtype == torch.uint8 else x.dtype
            T = self.n_patches + 1
            # the first block's folded norm1 reads the row moments: the embedding's last kernel writes them
            first_folds = (bool(blocks) and act == torch.bfloat16 and x.dim() == 4 and
                           not (blocks[0].training and (blocks[0].dropout1.p > 0 or blocks[0].dropout2.p > 0)) and
                           blocks[0].folds_norm1_shape(x.shape[0], T, act))
            x = ops.patch_embed(x, pemb.linear_projection.weight, pemb.linear_projection.bias, pemb.norm.weight,
                                pemb.norm.bias, pe_mod.cls_tokens, pe_mod.pe, self.args.patch_size, pemb.norm.eps,
                                pixel_mean=mean, pixel_inv_std=inv_std, want_moments=first_folds)
            moments = None
            if first_folds:
                x, moments = x
            for i, blk in enumerate(blocks):
                if blk.training and (blk.dropout1.p > 0 or blk.dropout2.p > 0):
                    x, moments = blk(x), None
                    continue
                nxt = blocks[i + 1] if i + 1 < len(blocks) else None
                x, moments = blk._forward_library(x, moments, want_moments=nxt is not None and nxt.folds_norm1(x))
            return ops.linear(x[:, 0], self.classifier.weight, self.classifier.bias)
        x = self.positional_encoding(self.patch_embedding(x))
        x = self.transformer_encoder(x)
        return self.classifier(x[:, 0])

    def set_candidates(self, cand):
        """Fix the candidate set of every sampled-mode ConvNN layer (the reference redraws a
        permutation per layer call; ranks of a batch-sharded run must share one set)."""
        for m in self.modules():
            if isinstance(m, MultiHeadConvNNAttention):
                m.candidate_override = cand
