"""CPU oracle for the ViT that calls the ConvNN-Attention layer.  TEST INFRASTRUCTURE ONLY.

Functional restatement of the reference model forward (vit.py:67-72, 90-135, 260-270)
driven by a state_dict with the reference's key names, so that the same weights can be
loaded into the reference ``vit.ViT`` (when pinning here) and into the CUDA-backed
model.  Only tests, the smoke entry and the bench's CPU-baseline legs import this.

Parity status: PINNED against reference outputs by ``oracle/pin_against_reference.py``
and by the fixtures under ``tests/golden/``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .convnn_oracle import (ConvNNConfig, branching_attention, branching_conv,
                            conv_weight_shapes, convnn_attention)


@dataclass
class ViTConfig:
    """The subset of the reference CLI namespace (main.py:28-113) the model reads."""
    layer: str = "ConvNNAttention"          # ConvNNAttention | BranchAttention | BranchConv
    img_size: tuple = (3, 224, 224)
    patch_size: int = 16
    num_layers: int = 12
    num_heads: int = 1
    d_hidden: int = 192
    d_mlp: int = 768
    num_classes: int = 1000
    K: int = 9
    sampling_type: str = "all"
    num_samples: int = -1
    sample_padding: int = 0
    magnitude_type: str = "cosine"
    coordinate_encoding: bool = False
    convolution_type: str = "depthwise"
    softmax_topk_val: bool = True
    branch_ratio: float = 0.5
    kernel_size: int = 9
    dropout: float = 0.0
    attention_dropout: float = 0.0

    @property
    def n_patches(self) -> int:
        return (self.img_size[1] * self.img_size[2]) // (self.patch_size * self.patch_size)

    @property
    def seq_len(self) -> int:
        return self.n_patches + 1

    def convnn_cfg(self) -> ConvNNConfig:
        d = self.d_hidden if self.layer == "ConvNNAttention" else int(self.branch_ratio * self.d_hidden)
        return ConvNNConfig(d_hidden=d, num_heads=self.num_heads, K=self.K,
                            sampling_type=self.sampling_type, num_samples=self.num_samples,
                            sample_padding=self.sample_padding, magnitude_type=self.magnitude_type,
                            seq_length=197,  # vit.py:148-157 never passes seq_length
                            coordinate_encoding=self.coordinate_encoding,
                            convolution_type=self.convolution_type,
                            softmax_topk_val=self.softmax_topk_val)


def positional_table(T: int, D: int) -> torch.Tensor:
    """Fixed sin/cos table (vit.py:117-124), shape (1, T, D)."""
    pe = torch.zeros(T, D)
    pos = torch.arange(0, T, dtype=torch.float).unsqueeze(1)
    div = torch.exp(torch.arange(0, D, 2).float() * (-math.log(10000.0) / D))
    pe[:, 0::2] = torch.sin(pos * div)
    pe[:, 1::2] = torch.cos(pos * div)
    return pe.unsqueeze(0)


def attention_weight_shapes(cfg: ViTConfig) -> Dict[str, tuple]:
    """state_dict entries of one encoder's ``attention`` sub-module."""
    D, H = cfg.d_hidden, cfg.num_heads
    c = cfg.convnn_cfg()
    lin = lambda d: {"W_q.weight": (d, d), "W_k.weight": (d, d), "W_v.weight": (d, d), "W_o.weight": (d, d)}
    conv = conv_weight_shapes(c)
    if cfg.layer == "ConvNNAttention":
        return {**lin(D), **conv}
    dc = c.d_hidden
    dr = D - dc
    out = {f"convnn.{k}": s for k, s in {**lin(dc), **conv}.items()}
    if cfg.layer == "BranchAttention":
        out.update({f"attention.{k}": s for k, s in lin(dr).items()})
    elif cfg.layer == "BranchConv":
        dk = dr // H
        out.update({"conv1d.W_x.weight": (dr, dr), "conv1d.W_x.bias": (dr,),
                    "conv1d.W_o.weight": (dr, dr), "conv1d.W_o.bias": (dr,),
                    "conv1d.conv.weight": (dk, dk, cfg.kernel_size), "conv1d.conv.bias": (dk,)})
    else:
        raise ValueError(cfg.layer)
    out.update({"pointwise_linear.weight": (D, D), "pointwise_linear.bias": (D,)})
    return out


def make_vit_weights(cfg: ViTConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded random-init weights for every state_dict key of the reference ViT.
    Matrices ~ U(+-1/sqrt(fan_in)); LayerNorm gains near 1; conv taps ~ N(1/K, 0.08)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg.d_hidden
    sd: Dict[str, torch.Tensor] = {}

    def uni(shape, fan_in):
        b = 1.0 / math.sqrt(fan_in)
        return (torch.rand(shape, generator=g) * 2 - 1) * b

    p = cfg.patch_size
    sd["patch_embedding.linear_projection.weight"] = uni((D, cfg.img_size[0], p, p), cfg.img_size[0] * p * p)
    sd["patch_embedding.linear_projection.bias"] = uni((D,), cfg.img_size[0] * p * p)
    sd["patch_embedding.norm.weight"] = 1.0 + 0.05 * torch.randn(D, generator=g)
    sd["patch_embedding.norm.bias"] = 0.05 * torch.randn(D, generator=g)
    sd["positional_encoding.cls_tokens"] = torch.randn(1, 1, D, generator=g)
    sd["positional_encoding.pe"] = positional_table(cfg.seq_len, D)
    for i in range(cfg.num_layers):
        pre = f"transformer_encoder.{i}."
        for name, shape in attention_weight_shapes(cfg).items():
            if name.endswith("bias"):
                t = uni(shape, D)
            elif name in ("conv.weight", "conv.0.weight", "convnn.conv.weight", "convnn.conv.0.weight"):
                t = torch.randn(shape, generator=g) * 0.08 + 1.0 / shape[-1]
            else:
                fan = shape[1] * (shape[2] if len(shape) == 3 else 1)
                t = uni(shape, fan)
            sd[pre + "attention." + name] = t
        sd[pre + "norm1.weight"] = 1.0 + 0.05 * torch.randn(D, generator=g)
        sd[pre + "norm1.bias"] = 0.05 * torch.randn(D, generator=g)
        sd[pre + "norm2.weight"] = 1.0 + 0.05 * torch.randn(D, generator=g)
        sd[pre + "norm2.bias"] = 0.05 * torch.randn(D, generator=g)
        sd[pre + "mlp.0.weight"] = uni((cfg.d_mlp, D), D)
        sd[pre + "mlp.0.bias"] = uni((cfg.d_mlp,), D)
        sd[pre + "mlp.3.weight"] = uni((D, cfg.d_mlp), cfg.d_mlp)
        sd[pre + "mlp.3.bias"] = uni((D,), cfg.d_mlp)
    sd["classifier.weight"] = uni((cfg.num_classes, D), D)
    sd["classifier.bias"] = uni((cfg.num_classes,), D)
    return sd


def make_images(B: int, cfg: ViTConfig, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, *cfg.img_size, generator=g)


def _sub(w, prefix):
    n = len(prefix)
    return {k[n:]: t for k, t in w.items() if k.startswith(prefix)}


def embed(images: torch.Tensor, sd: Dict[str, torch.Tensor], cfg: ViTConfig) -> torch.Tensor:
    """PatchEmbedding + PositionalEncoding (vit.py:104-109, 126-135) -> (B, T, D)."""
    D = cfg.d_hidden
    x = F.conv2d(images, sd["patch_embedding.linear_projection.weight"],
                 sd["patch_embedding.linear_projection.bias"], stride=cfg.patch_size)
    x = x.flatten(2).transpose(1, 2)
    x = F.layer_norm(x, (D,), sd["patch_embedding.norm.weight"], sd["patch_embedding.norm.bias"])
    cls = sd["positional_encoding.cls_tokens"].expand(x.shape[0], -1, -1)
    x = torch.cat([cls, x], dim=1)
    return x + sd["positional_encoding.pe"][:, : x.shape[1]]


def attention_block(xn: torch.Tensor, w: Dict[str, torch.Tensor], cfg: ViTConfig,
                    policy: str, cand: Optional[torch.Tensor], generator=None) -> torch.Tensor:
    c = cfg.convnn_cfg()
    if cfg.layer == "ConvNNAttention":
        return convnn_attention(xn, w, c, cand, policy, generator).out
    if cfg.layer == "BranchAttention":
        return branching_attention(xn, w, c, cfg.d_hidden, cfg.branch_ratio, cand, policy, generator)
    if cfg.layer == "BranchConv":
        return branching_conv(xn, w, c, cfg.d_hidden, cfg.branch_ratio, cfg.kernel_size, cand, policy, generator)
    raise ValueError(cfg.layer)


def encoder(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: ViTConfig, policy: str,
            cand: Optional[torch.Tensor], generator=None) -> torch.Tensor:
    """TransformerEncoder.forward (vit.py:260-270), eval mode."""
    D = cfg.d_hidden
    xn = F.layer_norm(x, (D,), w["norm1.weight"], w["norm1.bias"])
    x = x + attention_block(xn, _sub(w, "attention."), cfg, policy, cand, generator)
    xn = F.layer_norm(x, (D,), w["norm2.weight"], w["norm2.bias"])
    h = F.gelu(xn @ w["mlp.0.weight"].t() + w["mlp.0.bias"])
    return x + (h @ w["mlp.3.weight"].t() + w["mlp.3.bias"])


def vit_forward(images: torch.Tensor, sd: Dict[str, torch.Tensor], cfg: ViTConfig,
                policy: str = "fp32", cand: Optional[torch.Tensor] = None,
                generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """ViT.forward (vit.py:67-72) -> logits (B, num_classes).  ``cand`` fixes the
    candidate set of the sampled modes for every layer (the reference redraws a random
    permutation per layer call; pass ``generator`` to reproduce that instead)."""
    x = embed(images.to(torch.float32), sd, cfg)
    for i in range(cfg.num_layers):
        x = encoder(x, _sub(sd, f"transformer_encoder.{i}."), cfg, policy, cand, generator)
    return x[:, 0] @ sd["classifier.weight"].t() + sd["classifier.bias"]
