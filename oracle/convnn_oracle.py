"""CPU oracle for the ConvNN-Attention forward path.  TEST INFRASTRUCTURE ONLY.

This module restates, token-major and in plain torch CPU ops, what the reference
computes in ``layers.py`` (``MultiHeadConvNNAttention.forward`` and its helpers,
``MultiHeadBranchingAttention`` / ``MultiHeadBranchingConv``).  It exists to check the
CUDA path: only the tests, the smoke entry and the CPU-baseline legs of the bench may
import it.  The product never routes through it.

Parity status: PINNED.  The reference has no tests or golden vectors of its own, so the
oracle is pinned against outputs of the reference itself: ``oracle/pin_against_reference.py``
runs the unmodified reference modules (imported from a reference checkout) against every
function here over the whole option grid, and ``tests/golden/make_golden.py`` stores
reference outputs as fixtures that ``tests/test_oracle_golden.py`` replays without the
reference present.

Conventions (reference: layers.py:261-321):
  x            (B, T, D) activations, D = H * d_k
  k, v         (B, H, T, C) per-head keys / values, C = d_k (+1 with coordinate channel)
  q            (B, H, S, C) candidate queries; S = T and candidates = all tokens for
               sampling 'all', otherwise the rows of x named by ``cand`` (S,)
  sim[i, j]    similarity of key token i (row) to candidate j (column)
  idx, val     (B, H, T, K) neighbour token indices and their pre-softmax values,
               best first; sampled modes put the token itself in slot 0 with value 1
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
import torch.nn.functional as F

METRICS = ("cosine", "matmul", "euclidean")
SAMPLINGS = ("all", "random", "spatial")
CONV_TYPES = ("depthwise", "standard", "depthwise-separable")


@dataclass
class ConvNNConfig:
    """Constructor arguments of the reference layer (layers.py:133-146)."""
    d_hidden: int
    num_heads: int = 1
    K: int = 9
    sampling_type: str = "all"
    num_samples: int = -1
    sample_padding: int = 0
    magnitude_type: str = "cosine"
    seq_length: int = 197
    coordinate_encoding: bool = False
    convolution_type: str = "depthwise"
    softmax_topk_val: bool = True

    @property
    def d_k(self) -> int:
        return self.d_hidden // self.num_heads

    @property
    def maximum(self) -> bool:  # layers.py:168
        return self.magnitude_type in ("cosine", "matmul")

    @property
    def in_channels(self) -> int:  # layers.py:181
        return self.d_k + 1 if self.coordinate_encoding else self.d_k


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to bfloat16, returned as float32."""
    return t.to(torch.bfloat16).to(torch.float32)


def spatial_candidates(T: int, num_samples: int, sample_padding: int) -> torch.Tensor:
    """Candidate token indices of sampling_type='spatial' (layers.py:297): a 1-D
    linspace over token positions truncated to integers."""
    return torch.linspace(0 + sample_padding, T - sample_padding - 1, num_samples).long()


def random_candidates(T: int, num_samples: int, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Candidate token indices of sampling_type='random' (layers.py:284): the first
    ``num_samples`` entries of a random permutation (``-1`` silently means T-1)."""
    return torch.randperm(T, generator=generator)[:num_samples]


def _split_heads(y: torch.Tensor, H: int) -> torch.Tensor:
    """(B, R, D) -> (B, H, R, d_k): head h owns channels [h*d_k, (h+1)*d_k)
    (layers.py:237-245; the reference additionally transposes to channel-major)."""
    B, R, D = y.shape
    return y.view(B, R, H, D // H).permute(0, 2, 1, 3).contiguous()


def _append_coordinate(t: torch.Tensor) -> torch.Tensor:
    """Append one channel linspace(-1, 1, rows) (layers.py:439-450).  For sampled
    queries the coordinate runs over the S candidates, not their true positions."""
    B, H, R, C = t.shape
    coord = torch.linspace(-1.0, 1.0, R, dtype=t.dtype).view(1, 1, R, 1).expand(B, H, R, 1)
    return torch.cat([t, coord], dim=-1)


def project_qkv(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: ConvNNConfig,
                cand: Optional[torch.Tensor], policy: str = "fp32"):
    """Q/K/V projections (layers.py:264-265, 274, 286, 299) in per-head token-major form.

    policy 'bf16' rounds q, k, v to bfloat16 after the fp32 projection, which is the
    rounding point of the CUDA bf16 path (x and the weights are expected to be
    bf16-representable already)."""
    H = cfg.num_heads
    k = _split_heads(x @ w["W_k.weight"].t(), H)
    v = _split_heads(x @ w["W_v.weight"].t(), H)
    xq = x if cand is None else x[:, cand, :]
    q = _split_heads(xq @ w["W_q.weight"].t(), H)
    if cfg.coordinate_encoding:
        q, k, v = _append_coordinate(q), _append_coordinate(k), _append_coordinate(v)
    if policy == "bf16":   # the stored tensors, coordinate channel included, are bfloat16
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    return q, k, v


def similarity(q: torch.Tensor, k: torch.Tensor, cfg: ConvNNConfig,
               cand: Optional[torch.Tensor], dtype=torch.float32) -> torch.Tensor:
    """sim (B, H, T, S) per layers.py:323-340 plus the sampled-mode self mask
    (layers.py:291-292, 304-305).  ``dtype=torch.float64`` gives a high-precision copy
    for near-tie analysis."""
    q = q.to(dtype)
    k = k.to(dtype)
    if cfg.magnitude_type == "cosine":
        kn = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        qn = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        sim = kn @ qn.transpose(-1, -2)
    elif cfg.magnitude_type == "matmul":
        sim = (k @ q.transpose(-1, -2)) / (cfg.d_k ** 0.5)
    elif cfg.magnitude_type == "euclidean":
        k2 = (k * k).sum(-1, keepdim=True)                    # (B,H,T,1)
        q2 = (q * q).sum(-1, keepdim=True).transpose(-1, -2)  # (B,H,1,S)
        sim = torch.sqrt(k2 + q2 - 2.0 * (k @ q.transpose(-1, -2)))
    else:
        raise ValueError(f"unknown magnitude_type {cfg.magnitude_type!r}")
    if cand is not None:
        cols = torch.arange(cand.numel())
        sim[:, :, cand, cols] = 1.1 if cfg.magnitude_type == "euclidean" else -0.1
    return sim


def select_neighbours(sim: torch.Tensor, cfg: ConvNNConfig, cand: Optional[torch.Tensor]):
    """Hard top-K selection (layers.py:344, 363, 391, 410).  Returns idx (int64 token
    indices) and val (pre-softmax values), both (B, H, T, K), best first."""
    B, H, T, S = sim.shape
    if cand is None:
        val, idx = torch.topk(sim, k=cfg.K, dim=-1, largest=cfg.maximum)
    else:
        v1, i1 = torch.topk(sim, k=cfg.K - 1, dim=-1, largest=cfg.maximum)
        own = torch.arange(T).view(1, 1, T, 1).expand(B, H, T, 1)
        idx = torch.cat([own, cand[i1]], dim=-1)
        val = torch.cat([torch.ones(B, H, T, 1, dtype=sim.dtype), v1], dim=-1)
    return idx, val


def neighbour_weights(val: torch.Tensor, cfg: ConvNNConfig) -> torch.Tensor:
    """Per-neighbour scalar weights (layers.py:352-355, 382-385, 394-397, 426-429)."""
    if cfg.softmax_topk_val:
        return torch.softmax(val if cfg.maximum else -val, dim=-1)
    return val if cfg.maximum else 1.0 / (val + 1e-8)


def neighbour_conv(v: torch.Tensor, idx: torch.Tensor, p: torch.Tensor,
                   w: Dict[str, torch.Tensor], cfg: ConvNNConfig) -> torch.Tensor:
    """Gather + weighting + Conv1d(kernel K, stride K) (layers.py:402-405, 313,
    187-228), written as a contraction over the K neighbour taps.
    Returns o (B, H, T, d_k)."""
    B, H, T, C = v.shape
    K = cfg.K
    bi = torch.arange(B).view(B, 1, 1, 1)
    hi = torch.arange(H).view(1, H, 1, 1)
    nb = v[bi, hi, idx]                          # (B,H,T,K,C) neighbour rows
    P = nb * p.unsqueeze(-1)                     # weighted neighbour block
    if cfg.convolution_type == "depthwise":
        wc = w["conv.weight"]                    # (C,1,K); one conv shared by all heads
        return torch.einsum("bhtjc,cj->bhtc", P, wc[:, 0, :])
    if cfg.convolution_type == "standard":
        wc = w["conv.weight"]                    # (d_k, C, K)
        return torch.einsum("bhtjc,ocj->bhto", P, wc)
    if cfg.convolution_type == "depthwise-separable":
        w0 = w["conv.0.weight"]                  # (C,1,K)
        w1 = w["conv.1.weight"]                  # (d_k,C,1)
        dw = torch.einsum("bhtjc,cj->bhtc", P, w0[:, 0, :])
        return torch.einsum("bhtc,oc->bhto", dw, w1[:, :, 0])
    raise ValueError(f"unknown convolution_type {cfg.convolution_type!r}")


def merge_heads(o: torch.Tensor, cfg: ConvNNConfig) -> torch.Tensor:
    """(B, H, T, d_k) -> (B, T, D) exactly as layers.py:317, 320, 247-259 do it.

    H == 1 is the identity.  H > 1 reproduces the reference's flat reinterpretation:
    per (b, h) the (T, d_k) block is read back as if it were (d_k, T), so
    y[b, t', h*d_k + c'] = flat(o[b, h])[c'*T + t'].  It requires T == seq_length."""
    B, H, T, dk = o.shape
    if H == 1:
        return o[:, 0]
    if T != cfg.seq_length:
        raise RuntimeError(f"shape '[{B}, -1, {dk}, {cfg.seq_length}]' is invalid for input of size {o.numel()}")
    y = o.reshape(B, H, dk, T)            # reinterpret, no data movement
    return y.permute(0, 3, 1, 2).reshape(B, T, H * dk)


@dataclass
class ConvNNTrace:
    """Everything the tests compare against, stage by stage."""
    out: torch.Tensor
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    sim: torch.Tensor
    idx: torch.Tensor
    val: torch.Tensor
    o: torch.Tensor
    cand: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)


def resolve_candidates(cfg: ConvNNConfig, T: int, cand: Optional[torch.Tensor] = None,
                       generator: Optional[torch.Generator] = None) -> Optional[torch.Tensor]:
    if cfg.sampling_type == "all":
        return None
    if cand is not None:
        return cand.long()
    if cfg.sampling_type == "spatial":
        pad = cfg.sample_padding
        return spatial_candidates(T, cfg.num_samples, pad)
    if cfg.sampling_type == "random":
        return random_candidates(T, cfg.num_samples, generator)
    raise ValueError("Invalid sampling_type. Must be one of ['all', 'random', 'spatial']")


def convnn_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: ConvNNConfig,
                     cand: Optional[torch.Tensor] = None, policy: str = "fp32",
                     generator: Optional[torch.Generator] = None) -> ConvNNTrace:
    """Forward of MultiHeadConvNNAttention (layers.py:261-321), eval mode.

    ``policy``: 'fp32' computes everything in float32 like the reference on CPU;
    'bf16' additionally rounds q, k, v to bfloat16 after projection (the CUDA bf16
    path's rounding point).  ``cand`` overrides the candidate draw of the sampled modes.
    """
    x = x.to(torch.float32)
    w = {n: t.to(torch.float32) for n, t in w.items()}
    B, T, D = x.shape
    cand = resolve_candidates(cfg, T, cand, generator)
    q, k, v = project_qkv(x, w, cfg, cand, policy)
    sim = similarity(q, k, cfg, cand)
    idx, val = select_neighbours(sim, cfg, cand)
    p = neighbour_weights(val, cfg)
    o = neighbour_conv(v, idx, p, w, cfg)
    y = merge_heads(o, cfg)
    out = y @ w["W_o.weight"].t()
    return ConvNNTrace(out=out, q=q, k=k, v=v, sim=sim, idx=idx, val=val, o=o, cand=cand)


def from_neighbours(v: torch.Tensor, idx: torch.Tensor, val: torch.Tensor,
                    w: Dict[str, torch.Tensor], cfg: ConvNNConfig) -> torch.Tensor:
    """Everything downstream of the selection, for a given (idx, val): used to compare
    outputs on rows where a near-tie made the CUDA path pick another neighbour."""
    w = {n: t.to(torch.float32) for n, t in w.items()}
    p = neighbour_weights(val.to(torch.float32), cfg)
    o = neighbour_conv(v.to(torch.float32), idx.long(), p, w, cfg)
    return merge_heads(o, cfg) @ w["W_o.weight"].t()


# --------------------------------------------------------------------------------------
# Near-tie analysis
# --------------------------------------------------------------------------------------

def near_tie_rows(sim: torch.Tensor, cfg: ConvNNConfig, sampled: bool, tol: float) -> torch.Tensor:
    """Boolean (B, H, T): rows whose selection or ordering is decided by a gap smaller
    than ``tol`` (scaled by max(1, |value|)).  The top-(n+1) sorted values are inspected,
    n = K ('all') or K-1 (sampled): any adjacent gap below tol can legitimately flip
    either set membership (last gap) or tap order (the others)."""
    n = cfg.K - 1 if sampled else cfg.K
    S = sim.shape[-1]
    m = min(n + 1, S)
    if m < 2:
        return torch.zeros(sim.shape[:-1], dtype=torch.bool)
    top, _ = torch.topk(sim.double(), k=m, dim=-1, largest=cfg.maximum)
    gaps = (top[..., 1:] - top[..., :-1]).abs()
    scale = top[..., :-1].abs().clamp_min(1.0)
    return (gaps < tol * scale).any(dim=-1)


def swap_possible_rows(sim: torch.Tensor, cfg: ConvNNConfig, sampled: bool, delta: torch.Tensor) -> torch.Tensor:
    """Boolean (B, H, T): rows in which a perturbation of every similarity by at most
    ``delta`` (per row, shape (B, H, T), absolute) can change the ordered top-n list.  If two
    similarity matrices differ by at most delta on a row and their exact selections differ,
    two columns have swapped order, so some adjacent gap among the top-(n+1) sorted values
    of either matrix is at most 2*delta.  Used to check that every row on which a bfloat16
    run and the oracle disagree is explained by the measured difference of their q / k."""
    n = cfg.K - 1 if sampled else cfg.K
    m = min(n + 1, sim.shape[-1])
    if m < 2:
        return torch.zeros(sim.shape[:-1], dtype=torch.bool)
    top, _ = torch.topk(sim.double(), k=m, dim=-1, largest=cfg.maximum)
    gaps = (top[..., 1:] - top[..., :-1]).abs()
    return (gaps <= 2.0 * delta.double().unsqueeze(-1)).any(dim=-1)


# --------------------------------------------------------------------------------------
# Branching wrappers (ConvNN branch is the hot path; the other halves are plain torch)
# --------------------------------------------------------------------------------------

def softmax_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], H: int) -> torch.Tensor:
    """MultiHeadAttention.forward (layers.py:105-130), eval mode, no mask."""
    B, T, D = x.shape
    dk = D // H
    q = _split_heads(x @ w["W_q.weight"].t(), H)
    k = _split_heads(x @ w["W_k.weight"].t(), H)
    v = _split_heads(x @ w["W_v.weight"].t(), H)
    a = torch.softmax((q @ k.transpose(-1, -2)) / math.sqrt(dk), dim=-1)
    o = (a @ v).permute(0, 2, 1, 3).reshape(B, T, D)
    return o @ w["W_o.weight"].t()


def conv1d_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], H: int, kernel_size: int) -> torch.Tensor:
    """MultiHeadConv1dAttention.forward (layers.py:477-500): Linear -> per-head
    Conv1d(d_k, d_k, kernel_size, padding='same') -> the same flat reinterpretation as
    the ConvNN layer (applied for every H, with seq_length = T) -> Linear."""
    B, T, D = x.shape
    dk = D // H
    y = x @ w["W_x.weight"].t() + w["W_x.bias"]
    y = _split_heads(y, H)                                    # (B,H,T,dk)
    yc = y.permute(0, 1, 3, 2).reshape(B * H, dk, T)          # channel-major
    z = F.conv1d(yc, w["conv.weight"], w["conv.bias"], padding="same")  # (B*H,dk,T)
    o = z.permute(0, 2, 1).reshape(B, H, T, dk)               # token-major (B,H,T,dk)
    yq = o.reshape(B, H, dk, T).permute(0, 3, 1, 2).reshape(B, T, D)
    return yq @ w["W_o.weight"].t() + w["W_o.bias"]


def _sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    n = len(prefix)
    return {k[n:]: t for k, t in w.items() if k.startswith(prefix)}


def branching_attention(x, w, cfg: ConvNNConfig, d_total: int, branch_ratio: float,
                        cand=None, policy="fp32", generator=None) -> torch.Tensor:
    """MultiHeadBranchingAttention.forward (layers.py:642-652) for 0 < ratio < 1.
    ``cfg.d_hidden`` must be int(branch_ratio * d_total); both halves use cfg.num_heads."""
    dc = int(branch_ratio * d_total)
    assert cfg.d_hidden == dc
    x = x.to(torch.float32)
    w = {n: t.to(torch.float32) for n, t in w.items()}
    x1 = convnn_attention(x[:, :, :dc].contiguous(), _sub(w, "convnn."), cfg, cand, policy, generator).out
    x2 = softmax_attention(x[:, :, dc:].contiguous(), _sub(w, "attention."), cfg.num_heads)
    cat = torch.cat([x1, x2], dim=2)
    return cat @ w["pointwise_linear.weight"].t() + w["pointwise_linear.bias"]


def branching_conv(x, w, cfg: ConvNNConfig, d_total: int, branch_ratio: float, kernel_size: int,
                   cand=None, policy="fp32", generator=None) -> torch.Tensor:
    """MultiHeadBranchingConv.forward (layers.py:568-578) for 0 < ratio < 1."""
    dc = int(branch_ratio * d_total)
    assert cfg.d_hidden == dc
    x = x.to(torch.float32)
    w = {n: t.to(torch.float32) for n, t in w.items()}
    x1 = convnn_attention(x[:, :, :dc].contiguous(), _sub(w, "convnn."), cfg, cand, policy, generator).out
    x2 = conv1d_attention(x[:, :, dc:].contiguous(), _sub(w, "conv1d."), cfg.num_heads, kernel_size)
    cat = torch.cat([x1, x2], dim=2)
    return cat @ w["pointwise_linear.weight"].t() + w["pointwise_linear.bias"]


# --------------------------------------------------------------------------------------
# Seeded synthetic inputs / weights shared by fixtures, tests and the bench
# --------------------------------------------------------------------------------------

def conv_weight_shapes(cfg: ConvNNConfig) -> Dict[str, tuple]:
    C, dk, K = cfg.in_channels, cfg.d_k, cfg.K
    if cfg.convolution_type == "depthwise":
        return {"conv.weight": (C, 1, K)}
    if cfg.convolution_type == "standard":
        return {"conv.weight": (dk, C, K)}
    return {"conv.0.weight": (C, 1, K), "conv.1.weight": (dk, C, 1)}


def make_layer_weights(cfg: ConvNNConfig, seed: int, conv_init: str = "random") -> Dict[str, torch.Tensor]:
    """Deterministic weights keyed by the reference's state_dict names.  Linear weights
    ~ U(-1/sqrt(D), 1/sqrt(D)) like nn.Linear's default; conv weights ~ N(0, 0.08) so
    that tap order matters ('ones' reproduces the depthwise all-ones init,
    layers.py:206)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg.d_hidden
    b = 1.0 / math.sqrt(D)
    w = {}
    for name in ("W_q.weight", "W_k.weight", "W_v.weight", "W_o.weight"):
        w[name] = (torch.rand(D, D, generator=g) * 2 - 1) * b
    for name, shape in conv_weight_shapes(cfg).items():
        if conv_init == "ones":
            w[name] = torch.ones(shape)
        else:
            w[name] = torch.randn(shape, generator=g) * 0.08 + (1.0 / shape[-1] if name != "conv.1.weight" else 0.0)
    return w


def make_input(B: int, T: int, D: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, T, D, generator=g)
