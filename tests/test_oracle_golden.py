"""The oracle replays the committed reference outputs (no reference, no GPU needed)."""
import pytest
import torch

from oracle.convnn_oracle import convnn_attention, near_tie_rows, similarity, project_qkv
from oracle.vit_oracle import vit_forward
from golden_util import LAYER_NAMES, VIT_NAMES, layer_case, rel_err, vit_case


@pytest.mark.parametrize("name", LAYER_NAMES)
def test_layer_matches_reference(name):
    cfg, w, x, want, cand = layer_case(name)
    tr = convnn_attention(x, w, cfg, cand=cand)
    assert tr.out.shape == want.shape
    assert rel_err(tr.out, want) < 1e-5


@pytest.mark.parametrize("name", VIT_NAMES)
def test_vit_matches_reference(name):
    cfg, sd, img, want = vit_case(name)
    got = vit_forward(img, sd, cfg)
    assert rel_err(got, want) < 1e-5


def test_sampled_slot0_is_self_with_value_one():
    cfg, w, x, _, cand = layer_case("cos_spatial_dw_h1")
    tr = convnn_attention(x, w, cfg, cand=cand)
    T = x.shape[1]
    assert torch.equal(tr.idx[..., 0], torch.arange(T).expand_as(tr.idx[..., 0]))
    assert torch.all(tr.val[..., 0] == 1.0)
    # a token never selects itself through the candidate columns (finite sentinel mask)
    assert not (tr.idx[..., 1:] == torch.arange(T).view(1, 1, T, 1)).any()


def test_near_tie_detector_flags_exact_ties():
    cfg, w, x, _, _ = layer_case("cos_all_dw_h1")
    q, k, v = project_qkv(x, w, cfg, None)
    k[:, :, 5] = k[:, :, 4]            # tokens 4 and 5 become identical keys ...
    q[:, :, 5] = q[:, :, 4]            # ... and identical candidates: every row has a tie
    sim = similarity(q, k, cfg, None)
    flagged = near_tie_rows(sim, cfg, sampled=False, tol=1e-6)
    top = torch.topk(sim, cfg.K, dim=-1).indices
    has_pair = ((top == 4).any(-1) | (top == 5).any(-1))
    assert bool((flagged | ~has_pair).all())
