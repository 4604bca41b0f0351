"""CPU-side checks of the boundary: the library loads and exports every declared symbol,
argument validation mirrors the reference's failures, and the drop-in modules keep the
reference's state_dict layout.  No kernel is launched here."""
import ctypes
import os
import re
import sys
import types

import pytest
import torch

import convnn_b200
from convnn_b200 import _capi
from golden_util import MANIFEST

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(convnn_b200_\w+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_capi.library_path()) if os.path.exists(_capi.library_path()) else _capi.lib()
    syms = declared_symbols()
    assert len(syms) >= 10
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/ but not exported"
    assert set(syms) == set(_capi.SIGNATURES), "ctypes binding and header disagree"
    assert _capi.lib().convnn_b200_abi_version() == 1


def desc(**kw):
    base = dict(B=2, T=65, S=65, D=48, H=1, K=9, dtype=_capi.F32, metric="cosine", sampled=False,
                conv_type="depthwise", softmax=True, coord=False, seq_length=197)
    base.update(kw)
    return _capi.make_desc(**base)


def test_workspace_and_head_channels():
    L = _capi.lib()
    d = desc()
    assert L.convnn_b200_head_channels(d) == 48
    assert L.convnn_b200_workspace_bytes(d) >= 2 * 65 * 48 * 4 * 4
    d = desc(coord=True, conv_type="standard")
    assert L.convnn_b200_head_channels(d) == 56      # 48 + 1 rounded up to a multiple of 8
    d16 = desc(dtype=_capi.BF16)
    assert L.convnn_b200_workspace_bytes(d16) < L.convnn_b200_workspace_bytes(desc())


@pytest.mark.parametrize("kw,status,text", [
    (dict(K=66), _capi.E_TOPK_RANGE, "selected index k out of range"),          # torch.topk's message
    (dict(sampled=True, S=8, K=10), _capi.E_TOPK_RANGE, "out of range"),
    (dict(H=3, T=65, S=65), _capi.E_SEQ_LENGTH, "is invalid for input of size"),  # reference reshape error
    (dict(D=50, H=3), _capi.E_INVALID, "divisible"),
    (dict(S=64), _capi.E_INVALID, "S == T"),
    (dict(coord=True), _capi.E_INVALID, "depthwise"),
    (dict(K=33, T=100, S=100), _capi.E_UNSUPPORTED, "limit"),
    (dict(dtype=7), _capi.E_INVALID, "dtype"),
])
def test_validation_statuses(kw, status, text):
    L = _capi.lib()
    d = desc(**kw)
    assert L.convnn_b200_workspace_bytes(d) == 0
    rc = L.convnn_b200_head_channels(d)
    assert rc == status
    assert text in L.convnn_b200_last_error().decode()
    with pytest.raises(ValueError if status == _capi.E_INVALID else RuntimeError):
        _capi.check(rc)


def test_sampled_k_minus_one_equal_s_is_legal():
    assert _capi.lib().convnn_b200_head_channels(desc(sampled=True, S=8, K=9)) == 48


def test_null_pointer_rejected_before_any_launch():
    L = _capi.lib()
    rc = L.convnn_b200_sim_topk(desc(), None, None, None, None, None, None, None, None)
    assert rc == _capi.E_NULL
    rc = L.convnn_b200_forward(desc(), None, 48, None, None, None, None, None, None, 0, None, 48, None, 0, None)
    assert rc == _capi.E_NULL
    assert L.convnn_b200_layernorm(_capi.F32, None, 8, None, None, 1e-5, None, 8, 4, 8, None) == _capi.E_NULL
    assert L.convnn_b200_linear(_capi.F32, None, 8, None, None, None, 0, None, 8, 4, 8, 8, 0, None) == _capi.E_NULL
    assert L.convnn_b200_linear(7, None, 8, None, None, None, 0, None, 8, 4, 8, 8, 0, None) == _capi.E_INVALID


def _keys(module):
    return {k: list(v.shape) for k, v in module.state_dict().items()}


def test_state_dict_layout_matches_reference():
    C = convnn_b200
    want = MANIFEST["state_dict"]
    assert _keys(C.MultiHeadConvNNAttention(48, 3, 0.0, 9, "all", -1, 0, "cosine")) == want["convnn_depthwise"]
    assert _keys(C.MultiHeadConvNNAttention(48, 3, 0.0, 9, "all", -1, 0, "cosine", 197, True, "standard")) == \
        want["convnn_standard_coord"]
    assert _keys(C.MultiHeadConvNNAttention(48, 3, 0.0, 9, "all", -1, 0, "cosine", 197, False,
                                            "depthwise-separable")) == want["convnn_dwsep"]
    assert _keys(C.MultiHeadBranchingAttention(96, 3, 0.0, 9, "all", -1, 0, "cosine", 197, False, "standard",
                                               True, 0.5)) == want["branch_attention"]
    assert _keys(C.MultiHeadBranchingConv(96, 3, 0.0, 5, 9, "all", -1, 0, "cosine", 197, False, "depthwise",
                                          True, 0.5)) == want["branch_conv"]
    args = C.make_args(layer="ConvNNAttention", img_size=(3, 32, 32), patch_size=4, num_layers=12, num_heads=1,
                       d_hidden=192, d_mlp=768, num_classes=10, K=9, magnitude_type="cosine", device="cpu")
    assert _keys(C.ViT(args)) == want["vit_tiny_convnn"]


def test_depthwise_init_is_all_ones_and_coord_depthwise_raises():
    m = convnn_b200.MultiHeadConvNNAttention(48, 1, 0.0, 9, "all", -1, 0, "cosine")
    assert torch.all(m.conv.weight == 1.0)                       # reference layers.py:206
    with pytest.raises(ValueError):                              # groups mismatch at construction
        convnn_b200.MultiHeadConvNNAttention(48, 1, 0.0, 9, "all", -1, 0, "cosine", 197, True, "depthwise")


def test_no_cpu_path_and_forward_only():
    m = convnn_b200.MultiHeadConvNNAttention(48, 1, 0.0, 9, "all", -1, 0, "cosine").eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.randn(2, 65, 48))


def test_branching_degenerate_ratios_fail_like_reference():
    m = convnn_b200.MultiHeadBranchingAttention(96, 3, 0.0, 9, "all", -1, 0, "cosine", branch_ratio=0)
    with pytest.raises(AttributeError):                          # reference layers.py:643-644
        m(torch.randn(1, 197, 96))


def test_spatial_candidates_match_reference_formula():
    m = convnn_b200.MultiHeadConvNNAttention(48, 1, 0.0, 5, "spatial", 16, 3, "cosine")
    got = m.candidates(65, torch.device("cpu"))
    want = torch.linspace(3, 65 - 3 - 1, 16).long()
    assert torch.equal(got, want)
    r = convnn_b200.MultiHeadConvNNAttention(48, 1, 0.0, 5, "random", -1, 0, "cosine")
    assert r.candidates(65, torch.device("cpu")).numel() == 64   # num_samples=-1 -> T-1 (layers.py:284)


def test_dropin_install_rebinds_reference_names():
    fake_layers = types.ModuleType("layers")
    fake_vit = types.ModuleType("vit")
    for mod in (fake_layers, fake_vit):
        for n in ("MultiHeadConvNNAttention", "MultiHeadBranchingAttention", "MultiHeadBranchingConv"):
            setattr(mod, n, object)
        mod.MultiHeadAttention = "untouched"
    sys.modules["layers"], sys.modules["vit"] = fake_layers, fake_vit
    try:
        convnn_b200.install()
        assert fake_vit.MultiHeadConvNNAttention is convnn_b200.MultiHeadConvNNAttention
        assert fake_layers.MultiHeadBranchingConv is convnn_b200.MultiHeadBranchingConv
        assert fake_vit.MultiHeadAttention == "untouched"
        convnn_b200.uninstall()
        assert fake_vit.MultiHeadConvNNAttention is object
    finally:
        del sys.modules["layers"], sys.modules["vit"]


def test_candidate_indices_are_range_checked_on_the_host():
    """A candidate index outside [0, T) would become an out-of-bounds row number inside the
    kernels; the reference raises IndexError on `x[:, rand_idx, :]` (layers.py:285), and so do
    the places where a caller fixes the candidate set."""
    from convnn_b200 import ops
    ops.check_candidates(torch.tensor([0, 5, 64]), 65)
    with pytest.raises(IndexError, match="out of bounds"):
        ops.check_candidates(torch.tensor([0, 5, 65]), 65)
    with pytest.raises(IndexError, match="out of bounds"):
        ops.check_candidates(torch.tensor([-1, 5]), 65)
    m = convnn_b200.MultiHeadConvNNAttention(48, 1, 0.0, 5, "random", 16, 0, "cosine")
    with pytest.raises(IndexError):
        m.candidate_override = torch.tensor([3, -2, 7])
    m.candidate_override = torch.tensor([3, 70, 7])              # upper bound needs T
    with pytest.raises(IndexError):
        m.candidates(65, torch.device("cpu"))
    assert torch.equal(m.candidates(71, torch.device("cpu")), torch.tensor([3, 70, 7]))
    spec = ops.LayerSpec(48, 1, 5, "random")
    with pytest.raises(IndexError):
        ops._cand_arg(spec, torch.tensor([1, 99]), 65, torch.device("cpu"))
