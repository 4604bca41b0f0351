"""Stage-level and whole-layer calls into libconvnn_b200 on torch CUDA tensors.

torch is plumbing here: it owns device memory and the current stream.  All arithmetic
happens in the library's kernels; nothing in this file computes on the host or falls
back to torch ops.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _capi


@dataclass(frozen=True)
class LayerSpec:
    """Static configuration of one ConvNN-Attention layer (reference layers.py:133-146)."""
    d_hidden: int
    num_heads: int
    K: int
    sampling_type: str = "all"
    magnitude_type: str = "cosine"
    convolution_type: str = "depthwise"
    softmax_topk_val: bool = True
    coordinate_encoding: bool = False
    seq_length: int = 197

    @property
    def d_k(self) -> int:
        return self.d_hidden // self.num_heads

    @property
    def in_channels(self) -> int:
        return self.d_k + (1 if self.coordinate_encoding else 0)


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return _capi.F32
    if dt == torch.bfloat16:
        return _capi.BF16
    raise TypeError(f"convnn_b200 computes in float32 or bfloat16, got {dt}")


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("convnn_b200 runs on CUDA tensors only: there is no CPU path")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def descriptor(spec: LayerSpec, B: int, T: int, S: int, dtype: torch.dtype) -> _capi.ConvnnDesc:
    return _capi.make_desc(B, T, S, spec.d_hidden, spec.num_heads, spec.K, _dtype_code(dtype),
                           spec.magnitude_type, spec.sampling_type != "all", spec.convolution_type,
                           spec.softmax_topk_val, spec.coordinate_encoding, spec.seq_length)


def _rows_view(x: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """(B, T, D) tensor whose rows are contiguous and evenly strided -> (tensor, ld).
    A channel slice x[:, :, :d] of a wider contiguous tensor qualifies as it is."""
    B, T, D = x.shape
    if x.stride(2) == 1 and x.stride(0) == T * x.stride(1) and x.stride(1) >= D:
        return x, x.stride(1)
    x = x.contiguous()
    return x, D


def pack_weights(spec: LayerSpec, w_q, w_k, w_v, w_o, conv_weights, dtype, device):
    """Re-layout the module parameters into what the kernels read (see the header):
    w_qkv (3, D, D) = [W_k; W_v; W_q]; depthwise taps tap-major, standard taps (d_k, K*C); all in ``dtype``."""
    def cvt(t):
        return t.detach().to(device=device, dtype=dtype).contiguous()
    w_qkv = torch.stack([cvt(w_k), cvt(w_v), cvt(w_q)], dim=0).contiguous()
    w_pw = None
    if spec.convolution_type == "depthwise":
        (wc,) = conv_weights                       # (C, 1, K) -> (K, C)
        w_conv = cvt(wc[:, 0, :].t())
    elif spec.convolution_type == "standard":
        (wc,) = conv_weights                       # (d_k, C, K) -> (d_k, K, C)
        w_conv = cvt(wc.permute(0, 2, 1))
    elif spec.convolution_type == "depthwise-separable":
        w0, w1 = conv_weights                      # (C, 1, K) -> (K, C); (d_k, C, 1) -> (d_k, C)
        w_conv = cvt(w0[:, 0, :].t())
        w_pw = cvt(w1[:, :, 0])
    else:
        raise ValueError(f"unknown convolution_type {spec.convolution_type!r}")
    return w_qkv, w_conv, w_pw, cvt(w_o)


def check_candidates(cand: torch.Tensor, T: Optional[int] = None) -> torch.Tensor:
    """Range check of caller-supplied candidate token indices: the kernels use them as row
    numbers without looking, so a value outside [0, T) must be stopped on the host.  Raises
    IndexError as the reference's ``x[:, rand_idx, :]`` (layers.py:285) does.  Reads the
    tensor (a device tensor is synchronised), so it runs where a candidate set is fixed, not
    on every forward."""
    if cand.numel() == 0:
        raise IndexError("the candidate set is empty")
    lo, hi = int(cand.min()), int(cand.max())
    if lo < 0 or (T is not None and hi >= T):
        bad = lo if lo < 0 else hi
        raise IndexError(f"index {bad} is out of bounds for dimension 1 with size {T}")
    return cand


def _cand_arg(spec: LayerSpec, cand: Optional[torch.Tensor], T: int, device) -> Tuple[Optional[torch.Tensor], int]:
    if spec.sampling_type == "all":
        return None, T
    if cand is None:
        raise ValueError("sampled modes need candidate indices")
    if not cand.is_cuda:
        check_candidates(cand, T)          # host tensors are cheap to check on every call
    cand = cand.to(device=device, dtype=torch.int32).contiguous()
    return cand, int(cand.numel())


def qkv_proj(spec: LayerSpec, x: torch.Tensor, w_qkv: torch.Tensor, cand: Optional[torch.Tensor] = None):
    """-> q (B,S,H,Cp), k, v (B,T,H,Cp), qstat (B,H,S), kstat (B,H,T)."""
    _require_cuda(x, w_qkv)
    L = _capi.lib()
    x, ldx = _rows_view(x)
    B, T, _ = x.shape
    cand, S = _cand_arg(spec, cand, T, x.device)
    d = descriptor(spec, B, T, S, x.dtype)
    Cp = L.convnn_b200_head_channels(d)
    _capi.check(min(Cp, 0))
    H = spec.num_heads
    q = torch.empty(B, S, H, Cp, dtype=x.dtype, device=x.device)
    k = torch.empty(B, T, H, Cp, dtype=x.dtype, device=x.device)
    v = torch.empty(B, T, H, Cp, dtype=x.dtype, device=x.device)
    qstat = torch.empty(B, H, S, dtype=torch.float32, device=x.device)
    kstat = torch.empty(B, H, T, dtype=torch.float32, device=x.device)
    scratch = torch.empty(L.convnn_b200_stage_scratch_bytes(d), dtype=torch.uint8, device=x.device)
    _capi.check(L.convnn_b200_qkv_proj(d, x.data_ptr(), ldx, w_qkv.data_ptr(), _capi.ptr(cand), q.data_ptr(),
                                       k.data_ptr(), v.data_ptr(), qstat.data_ptr(), kstat.data_ptr(),
                                       scratch.data_ptr(), _stream(x)))
    return q, k, v, qstat, kstat


def sim_topk(spec: LayerSpec, q, k, qstat, kstat, cand: Optional[torch.Tensor] = None):
    """-> idx int32 (B,H,T,K), val float32 (B,H,T,K), best first."""
    _require_cuda(q, k)
    L = _capi.lib()
    B, T, H, _ = k.shape
    cand, S = _cand_arg(spec, cand, T, k.device)
    d = descriptor(spec, B, T, q.shape[1], k.dtype)
    idx = torch.empty(B, H, T, spec.K, dtype=torch.int32, device=k.device)
    val = torch.empty(B, H, T, spec.K, dtype=torch.float32, device=k.device)
    _capi.check(L.convnn_b200_sim_topk(d, q.data_ptr(), k.data_ptr(), _capi.ptr(qstat), _capi.ptr(kstat),
                                       _capi.ptr(cand), idx.data_ptr(), val.data_ptr(), _stream(k)))
    return idx, val


def gather_conv(spec: LayerSpec, v, idx, val, w_conv, w_pw=None, S: Optional[int] = None):
    """-> o (B,H,T,d_k)."""
    _require_cuda(v, idx, val, w_conv)
    L = _capi.lib()
    B, T, H, _ = v.shape
    d = descriptor(spec, B, T, T if spec.sampling_type == "all" else (S or T), v.dtype)
    o = torch.empty(B, H, T, spec.d_k, dtype=v.dtype, device=v.device)
    scratch = None
    if spec.convolution_type != "depthwise":
        scratch = torch.empty(L.convnn_b200_stage_scratch_bytes(d), dtype=torch.uint8, device=v.device)
    _capi.check(L.convnn_b200_gather_conv(d, v.data_ptr(), idx.data_ptr(), val.data_ptr(), w_conv.data_ptr(),
                                          _capi.ptr(w_pw), o.data_ptr(), _capi.ptr(scratch), _stream(v)))
    return o


def _residual_arg(residual, like):
    if residual is None:
        return None, 0
    r, ldr = _rows_view(residual)
    if r.dtype != like.dtype or not r.is_cuda:
        raise TypeError("residual must be a CUDA tensor of the activation dtype")
    return r, ldr


def out_proj(spec: LayerSpec, o, w_o, out: Optional[torch.Tensor] = None, S: Optional[int] = None,
             residual: Optional[torch.Tensor] = None):
    """-> out (B,T,D) [= residual + proj]; ``out`` may be a channel slice of a wider tensor."""
    _require_cuda(o, w_o)
    L = _capi.lib()
    B, H, T, dk = o.shape
    d = descriptor(spec, B, T, T if spec.sampling_type == "all" else (S or T), o.dtype)
    if out is None:
        out = torch.empty(B, T, spec.d_hidden, dtype=o.dtype, device=o.device)
    view, ldo = _rows_view(out)
    if view is not out:
        raise ValueError("out must have unit channel stride and evenly strided rows")
    scratch = torch.empty(L.convnn_b200_stage_scratch_bytes(d), dtype=torch.uint8, device=o.device)
    res, ldr = _residual_arg(residual, o)
    _capi.check(L.convnn_b200_out_proj(d, o.data_ptr(), w_o.data_ptr(), _capi.ptr(res), ldr, out.data_ptr(), ldo,
                                       scratch.data_ptr(), _stream(o)))
    return out


def workspace_bytes(spec: LayerSpec, B: int, T: int, S: int, dtype: torch.dtype) -> int:
    d = descriptor(spec, B, T, S, dtype)
    n = _capi.lib().convnn_b200_workspace_bytes(d)
    if n == 0:
        # re-run validation through an entry point that reports the reason
        _capi.check(min(_capi.lib().convnn_b200_head_channels(d), 0))
    return int(n)


def forward(spec: LayerSpec, x: torch.Tensor, packed, cand: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Whole-layer forward through ``convnn_b200_forward`` (out = [residual +] layer(x))."""
    w_qkv, w_conv, w_pw, w_o = packed
    _require_cuda(x, w_qkv)
    L = _capi.lib()
    x, ldx = _rows_view(x)
    B, T, D = x.shape
    cand, S = _cand_arg(spec, cand, T, x.device)
    d = descriptor(spec, B, T, S, x.dtype)
    need = L.convnn_b200_workspace_bytes(d)
    if need == 0:
        _capi.check(min(L.convnn_b200_head_channels(d), 0))
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty(B, T, D, dtype=x.dtype, device=x.device)
    oview, ldo = _rows_view(out)
    if oview is not out:
        raise ValueError("out must have unit channel stride and evenly strided rows")
    res, ldr = _residual_arg(residual, x)
    _capi.check(L.convnn_b200_forward(d, x.data_ptr(), ldx, w_qkv.data_ptr(), w_conv.data_ptr(), _capi.ptr(w_pw),
                                      w_o.data_ptr(), _capi.ptr(cand), _capi.ptr(res), ldr, out.data_ptr(), ldo,
                                      workspace.data_ptr(), workspace.numel(), _stream(x)))
    return out


# ---- LayerNorm folded into the GEMM that consumes it (bfloat16) --------------------------------

def prenorm_linear_supported(N: int, K: int, gelu: bool) -> bool:
    return bool(_capi.lib().convnn_b200_prenorm_linear_supported(N, K, int(gelu)))


def prenorm_forward_supported(spec: LayerSpec, B: int, T: int, dtype) -> bool:
    if dtype != torch.bfloat16 or spec.sampling_type != "all":
        return False
    return bool(_capi.lib().convnn_b200_prenorm_forward_supported(descriptor(spec, B, T, T, dtype)))


def row_moments(x: torch.Tensor) -> torch.Tensor:
    """(1, stride, 2) float32 (sum, sum of squares) of every row of a bfloat16 ``x`` (..., D); stride =
    the row count rounded up to the plane stride of moments buffers (``convnn_b200_moment_stride``)."""
    _require_cuda(x)
    xv, rows, ldx = _flat_rows(x)
    out = torch.empty(1, _capi.lib().convnn_b200_moment_stride(rows), 2, dtype=torch.float32, device=x.device)
    _capi.check(_capi.lib().convnn_b200_row_moments(xv.data_ptr(), ldx, rows, x.shape[-1], out.data_ptr(), _stream(x)))
    return out


def fold_layernorm(weight: torch.Tensor, bias: Optional[torch.Tensor], gamma: torch.Tensor,
                   beta: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(w_folded (N, K), w_extra (N, 16)) for ``prenorm_linear`` / ``prenorm_forward``: the Linear's
    weight with the LayerNorm's gamma multiplied in, and the mean / beta / bias correction rows."""
    _require_cuda(weight, gamma, beta, bias)
    w = weight.detach().contiguous()
    N, K = w.shape
    wf = torch.empty(N, K, dtype=torch.bfloat16, device=w.device)
    wx = torch.empty(N, 16, dtype=torch.bfloat16, device=w.device)
    _capi.check(_capi.lib().convnn_b200_fold_layernorm(w.data_ptr(), _capi.ptr(bias), gamma.data_ptr(), beta.data_ptr(),
                                                       N, K, wf.data_ptr(), wx.data_ptr(), _stream(w)))
    return wf, wx


def prenorm_linear(a: torch.Tensor, moments: torch.Tensor, eps: float, w_folded: torch.Tensor,
                   w_extra: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    """[GELU](LayerNorm(a) @ W.T + bias) from the un-normalised rows ``a`` and their moments."""
    _require_cuda(a, moments, w_folded, w_extra)
    av, M, lda = _flat_rows(a)
    N, K = w_folded.shape
    out = torch.empty(*a.shape[:-1], N, dtype=a.dtype, device=a.device)
    _capi.check(_capi.lib().convnn_b200_prenorm_linear(av.data_ptr(), lda, moments.data_ptr(), moments.shape[0],
                                                       float(eps), w_folded.data_ptr(), w_extra.data_ptr(),
                                                       out.data_ptr(), N, M, N, K, int(gelu), _stream(a)))
    return out


def linear_moments(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                   residual: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(residual + a @ weight.T + bias, moments of its rows) through ``convnn_b200_linear_moments``."""
    _require_cuda(a, weight, bias, residual)
    L = _capi.lib()
    av, M, lda = _flat_rows(a)
    N, K = weight.shape
    w = weight if weight.is_contiguous() else weight.contiguous()
    out = torch.empty(*a.shape[:-1], N, dtype=a.dtype, device=a.device)
    mom = torch.empty(L.convnn_b200_moment_planes(N), L.convnn_b200_moment_stride(M), 2, dtype=torch.float32,
                      device=a.device)
    res, _, ldr = _flat_rows(residual)
    _capi.check(L.convnn_b200_linear_moments(av.data_ptr(), lda, w.data_ptr(), _capi.ptr(bias), res.data_ptr(), ldr,
                                             out.data_ptr(), N, M, N, K, mom.data_ptr(), _stream(a)))
    return out, mom


def prenorm_forward(spec: LayerSpec, x: torch.Tensor, moments: torch.Tensor, eps: float, packed_folded,
                    residual: Optional[torch.Tensor] = None, want_moments: bool = False,
                    workspace: Optional[torch.Tensor] = None):
    """``[residual +] layer(LayerNorm(x))`` through ``convnn_b200_prenorm_forward``; ``packed_folded`` =
    (w_qkv_folded (3D, D), w_qkv_extra (3D, 16), w_conv, w_pw, w_o).  Returns (out, moments of out or None)."""
    w_qkv, w_qkv_x, w_conv, w_pw, w_o = packed_folded      # w_o None: stop before the output projection
    _require_cuda(x, w_qkv, moments)
    L = _capi.lib()
    x, ldx = _rows_view(x)
    B, T, D = x.shape
    d = descriptor(spec, B, T, T, x.dtype)
    need = L.convnn_b200_workspace_bytes(d)
    if need == 0:
        _capi.check(min(L.convnn_b200_head_channels(d), 0))
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    out = torch.empty(B, T, D, dtype=x.dtype, device=x.device)
    res, ldr = _residual_arg(residual, x)
    mom = None
    if want_moments:
        mom = torch.empty(L.convnn_b200_moment_planes(D), L.convnn_b200_moment_stride(B * T), 2, dtype=torch.float32,
                          device=x.device)
    _capi.check(L.convnn_b200_prenorm_forward(d, x.data_ptr(), ldx, moments.data_ptr(), moments.shape[0], float(eps),
                                              w_qkv.data_ptr(), w_qkv_x.data_ptr(), w_conv.data_ptr(), _capi.ptr(w_pw),
                                              _capi.ptr(w_o), _capi.ptr(res), ldr, out.data_ptr(), D,
                                              _capi.ptr(mom), workspace.data_ptr(), workspace.numel(), _stream(x)))
    return out, mom


def prenorm_mlp_supported(D: int, DM: int, planes: int) -> bool:
    return bool(_capi.lib().convnn_b200_prenorm_mlp_supported(D, DM, planes))


def prenorm_mlp(x: torch.Tensor, moments: torch.Tensor, eps: float, w1_folded: torch.Tensor, w1_extra: torch.Tensor,
                w2: torch.Tensor, b2: Optional[torch.Tensor], want_moments: bool = False):
    """``x + (GELU(LayerNorm(x) @ W1.T + b1) @ W2.T + b2)`` in one kernel (``convnn_b200_prenorm_mlp``).
    Returns (out, moments of out (planes, stride, 2) or None)."""
    _require_cuda(x, moments, w1_folded, w1_extra, w2, b2)
    L = _capi.lib()
    xv, M, ldx = _flat_rows(x)
    DM, D = w1_folded.shape
    w2c = w2 if w2.is_contiguous() else w2.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    mom = None
    if want_moments:
        mom = torch.empty(L.convnn_b200_prenorm_mlp_moment_planes(), L.convnn_b200_moment_stride(M), 2,
                          dtype=torch.float32, device=x.device)
    _capi.check(L.convnn_b200_prenorm_mlp(xv.data_ptr(), ldx, moments.data_ptr(), moments.shape[0], float(eps),
                                          w1_folded.data_ptr(), w1_extra.data_ptr(), w2c.data_ptr(), _capi.ptr(b2),
                                          out.data_ptr(), D, M, D, DM, _capi.ptr(mom), _stream(x)))
    return out, mom


def outproj_mlp(o: torch.Tensor, w_o: torch.Tensor, x: torch.Tensor, eps: float, w1_folded: torch.Tensor,
                w1_extra: torch.Tensor, w2: torch.Tensor, b2: Optional[torch.Tensor], want_moments: bool = False):
    """``x1 = x + o @ W_o.T; x1 + mlp(LayerNorm(x1))`` in one kernel (``convnn_b200_outproj_mlp``); ``o`` is the
    attention layer's head-merged output before its output projection.  Returns (out, moments of out or None)."""
    _require_cuda(o, w_o, x, w1_folded, w1_extra, w2, b2)
    L = _capi.lib()
    ov, M, ld_o = _flat_rows(o)
    xv, _, ldx = _flat_rows(x)
    DM, D = w1_folded.shape
    w2c = w2 if w2.is_contiguous() else w2.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    mom = None
    if want_moments:
        mom = torch.empty(L.convnn_b200_prenorm_mlp_moment_planes(), L.convnn_b200_moment_stride(M), 2,
                          dtype=torch.float32, device=x.device)
    _capi.check(L.convnn_b200_outproj_mlp(ov.data_ptr(), ld_o, w_o.data_ptr(), xv.data_ptr(), ldx, float(eps),
                                          w1_folded.data_ptr(), w1_extra.data_ptr(), w2c.data_ptr(), _capi.ptr(b2),
                                          out.data_ptr(), D, M, D, DM, _capi.ptr(mom), _stream(x)))
    return out, mom


# ---- the other halves of the branching wrappers ------------------------------------------------

def _out_slice(out: Optional[torch.Tensor], like: torch.Tensor) -> Tuple[torch.Tensor, int]:
    B, T, D = like.shape
    if out is None:
        out = torch.empty(B, T, D, dtype=like.dtype, device=like.device)
    view, ldo = _rows_view(out)
    if view is not out:
        raise ValueError("out must have unit channel stride and evenly strided rows")
    return out, ldo


def softmax_attention(x: torch.Tensor, w_qkv: torch.Tensor, w_o: torch.Tensor, num_heads: int,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """MultiHeadAttention.forward (reference layers.py:105-130) through
    ``convnn_b200_softmax_attention``; ``w_qkv`` = (3, D, D) [W_q; W_k; W_v]."""
    _require_cuda(x, w_qkv, w_o)
    L = _capi.lib()
    x, ldx = _rows_view(x)
    B, T, D = x.shape
    out, ldo = _out_slice(out, x)
    dt = _dtype_code(x.dtype)
    ws = torch.empty(L.convnn_b200_attention_workspace_bytes(dt, B, T, D), dtype=torch.uint8, device=x.device)
    _capi.check(L.convnn_b200_softmax_attention(dt, x.data_ptr(), ldx, w_qkv.data_ptr(), w_o.data_ptr(), out.data_ptr(),
                                                ldo, B, T, D, num_heads, ws.data_ptr(), ws.numel(), _stream(x)))
    return out


def conv1d_attention(x: torch.Tensor, w_x, b_x, w_conv, b_conv, w_o, b_o, num_heads: int, kernel_size: int,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """MultiHeadConv1dAttention.forward (reference layers.py:477-500) through
    ``convnn_b200_conv1d_attention``; ``w_conv`` packed (d_k, kernel_size, d_k)."""
    _require_cuda(x, w_x, w_conv, w_o)
    L = _capi.lib()
    x, ldx = _rows_view(x)
    B, T, D = x.shape
    out, ldo = _out_slice(out, x)
    dt = _dtype_code(x.dtype)
    ws = torch.empty(L.convnn_b200_conv1d_attention_workspace_bytes(dt, B, T, D, kernel_size), dtype=torch.uint8,
                     device=x.device)
    _capi.check(L.convnn_b200_conv1d_attention(dt, x.data_ptr(), ldx, w_x.data_ptr(), _capi.ptr(b_x), w_conv.data_ptr(),
                                               _capi.ptr(b_conv), w_o.data_ptr(), _capi.ptr(b_o), out.data_ptr(), ldo,
                                               B, T, D, num_heads, kernel_size, ws.data_ptr(), ws.numel(), _stream(x)))
    return out


# ---- the encoder ops around the layer ---------------------------------------------------

def _flat_rows(t: torch.Tensor) -> Tuple[torch.Tensor, int, int]:
    """(..., D) tensor -> (tensor, rows, ld) with contiguous rows of a common stride."""
    D = t.shape[-1]
    if t.dim() >= 2 and t.stride(-1) == 1 and t.is_contiguous():
        return t, t.numel() // D, D
    if t.dim() == 3:
        v, ld = _rows_view(t)
        return v, v.shape[0] * v.shape[1], ld
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= D:
        return t, t.shape[0], t.stride(0)          # evenly strided rows, e.g. the class-token rows x[:, 0]
    t = t.contiguous()
    return t, t.numel() // D, D


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    _require_cuda(x, weight, bias)
    L = _capi.lib()
    xv, rows, ldx = _flat_rows(x)
    D = x.shape[-1]
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _capi.check(L.convnn_b200_layernorm(_dtype_code(x.dtype), xv.data_ptr(), ldx, weight.data_ptr(), bias.data_ptr(),
                                        float(eps), y.data_ptr(), D, rows, D, _stream(x)))
    return y


def linear(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[GELU](a @ weight.T + bias) [+ residual] through ``convnn_b200_linear``."""
    _require_cuda(a, weight, bias, residual)
    L = _capi.lib()
    av, M, lda = _flat_rows(a)
    N, K = weight.shape
    w = weight if weight.is_contiguous() else weight.contiguous()
    out = torch.empty(*a.shape[:-1], N, dtype=a.dtype, device=a.device)
    res, ldr = (None, 0)
    if residual is not None:
        res, _, ldr = _flat_rows(residual)
    _capi.check(L.convnn_b200_linear(_dtype_code(a.dtype), av.data_ptr(), lda, w.data_ptr(), _capi.ptr(bias),
                                     _capi.ptr(res), ldr, out.data_ptr(), N, M, N, K, int(gelu), _stream(a)))
    return out


def patch_embed(images: torch.Tensor, conv_weight: torch.Tensor, conv_bias: torch.Tensor, norm_weight, norm_bias,
                cls: torch.Tensor, pe: torch.Tensor, patch: int, eps: float = 1e-5,
                pixel_mean: Optional[torch.Tensor] = None, pixel_inv_std: Optional[torch.Tensor] = None,
                want_moments: bool = False):
    """PatchEmbedding + PositionalEncoding (reference vit.py:104-109, 126-135): unfold, GEMM
    with the (D, C*P*P) weight view, LayerNorm, class token and positional table -> (B, T, D).
    uint8 images are normalised on the way ((img / 255 - pixel_mean[c]) * pixel_inv_std[c], the
    loader's ToTensor + Normalize, reference dataset.py:22-23) and computed in the weights' dtype.
    want_moments: also return the (1, moment_stride(B*T), 2) float32 row moments of the result (what
    row_moments would compute from it), written by the same kernel."""
    _require_cuda(images, conv_weight)
    L = _capi.lib()
    B, C, Hh, Ww = images.shape
    D = conv_weight.shape[0]
    Np = (Hh // patch) * (Ww // patch)
    act = conv_weight.dtype if images.dtype == torch.uint8 else images.dtype
    dt = _dtype_code(act)
    images = images.contiguous()
    cols = torch.empty(B * Np, C * patch * patch, dtype=act, device=images.device)
    if images.dtype == torch.uint8:
        if pixel_mean is None or pixel_inv_std is None:
            raise ValueError("uint8 images need pixel_mean and pixel_inv_std (float32, one value per channel)")
        _capi.check(L.convnn_b200_patchify_u8(dt, images.data_ptr(), pixel_mean.data_ptr(), pixel_inv_std.data_ptr(),
                                              cols.data_ptr(), B, C, Hh, Ww, patch, _stream(images)))
    else:
        _capi.check(L.convnn_b200_patchify(dt, images.data_ptr(), cols.data_ptr(), B, C, Hh, Ww, patch, _stream(images)))
    proj = linear(cols, conv_weight.reshape(D, -1), conv_bias)
    out = torch.empty(B, Np + 1, D, dtype=act, device=images.device)
    pe2 = pe.reshape(-1, D)[: Np + 1].contiguous()
    moments = None
    if want_moments:
        moments = torch.empty(1, L.convnn_b200_moment_stride(B * (Np + 1)), 2, dtype=torch.float32,
                              device=images.device)
    _capi.check(L.convnn_b200_embed_tokens_moments(dt, proj.data_ptr(), norm_weight.data_ptr(), norm_bias.data_ptr(),
                                                   float(eps), cls.reshape(-1).contiguous().data_ptr(), pe2.data_ptr(),
                                                   out.data_ptr(), B, Np, D,
                                                   moments.data_ptr() if want_moments else None, _stream(images)))
    return (out, moments) if want_moments else out
