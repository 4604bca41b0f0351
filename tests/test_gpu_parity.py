"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle and the
committed reference outputs.

Tolerances (from the task statement): float32 — neighbour index lists identical except on
rows decided by a similarity gap below 1e-6, outputs within 1e-4 relative; bfloat16 —
outputs within 2e-2 relative against the oracle run with the same rounding points
(q, k, v rounded to bfloat16 after projection).
"""
import pytest
import torch

from convnn_b200 import ops
from oracle.convnn_oracle import (ConvNNConfig, bf16_round, convnn_attention, from_neighbours, make_input,
                                  make_layer_weights, near_tie_rows, neighbour_conv, neighbour_weights,
                                  select_neighbours, similarity, swap_possible_rows)
from golden_util import LAYER_NAMES, layer_case
from gpu_util import DEV, heads_to_oracle, module_of, pack, rel_err, spec_of

pytestmark = pytest.mark.gpu

FP32_TIE = 1e-6
FP32_OUT = 1e-4
BF16_OUT = 2e-2


def run_stages(cfg, w, x, cand, dtype):
    spec = spec_of(cfg)
    packed = pack(cfg, w, dtype)
    xg = x.to(DEV, dtype)
    cg = None if cand is None else cand.to(DEV)
    q, k, v, qs, ks = ops.qkv_proj(spec, xg, packed[0], cg)
    idx, val = ops.sim_topk(spec, q, k, qs, ks, cg)
    o = ops.gather_conv(spec, v, idx, val, packed[1], packed[2], S=q.shape[1])
    out = ops.out_proj(spec, o, packed[3], S=q.shape[1])
    torch.cuda.synchronize()
    return q, k, v, qs, ks, idx, val, o, out


@pytest.mark.parametrize("name", LAYER_NAMES)
def test_fp32_stages_against_oracle_and_reference(name):
    cfg, w, x, want, cand = layer_case(name)
    tr = convnn_attention(x, w, cfg, cand=cand)
    cand = tr.cand                     # spatial candidates are resolved by the oracle
    q, k, v, qs, ks, idx, val, o, out = run_stages(cfg, w, x, cand, torch.float32)
    C = cfg.in_channels
    assert rel_err(heads_to_oracle(q, C), tr.q) < 1e-5
    assert rel_err(heads_to_oracle(k, C), tr.k) < 1e-5
    assert rel_err(heads_to_oracle(v, C), tr.v) < 1e-5
    # selection: identical, in order, wherever no gap is below 1e-6
    ties = near_tie_rows(tr.sim, cfg, cand is not None, FP32_TIE)
    same = (idx.cpu().long() == tr.idx).all(-1)
    assert bool((same | ties).all()), f"{int((~(same | ties)).sum())} rows differ without a near-tie"
    assert float(ties.float().mean()) < 0.02
    dv = (val.cpu() - tr.val).abs() / tr.val.abs().clamp_min(1.0)
    assert float(dv[same].max()) < 5e-6
    # downstream of the selection, on the kernel's own neighbours
    p = neighbour_weights(val.cpu(), cfg)
    o_want = neighbour_conv(tr.v, idx.cpu().long(), p, w, cfg)
    assert rel_err(o, o_want) < FP32_OUT
    assert rel_err(out, from_neighbours(tr.v, idx.cpu(), val.cpu(), w, cfg)) < FP32_OUT
    if bool(same.all()):
        assert rel_err(out, want) < FP32_OUT          # the reference's own output


@pytest.mark.parametrize("name", LAYER_NAMES)
def test_fp32_module_forward_equals_staged_calls(name):
    cfg, w, x, want, cand = layer_case(name)
    m = module_of(cfg, w, torch.float32)
    m.candidate_override = cand
    with torch.no_grad():
        y1 = m(x.to(DEV))
        y2 = m(x.to(DEV))
    out = run_stages(cfg, w, x, m.candidates(x.shape[1], torch.device(DEV)), torch.float32)[-1]
    assert torch.equal(y1, y2), "two runs differ bit-wise"
    assert torch.equal(y1, out)


BASELINE_SHAPES = {
    # the layer shapes of the baseline configs at a reduced batch
    "cfg2_tiny": (2, 197, dict(d_hidden=192, num_heads=1, K=9, magnitude_type="cosine")),
    "cfg3_small": (2, 197, dict(d_hidden=384, num_heads=1, K=9, magnitude_type="euclidean", sampling_type="random",
                                num_samples=64, convolution_type="depthwise-separable")),
    "cfg4_branch_half": (2, 197, dict(d_hidden=384, num_heads=12, K=9, magnitude_type="cosine",
                                      convolution_type="standard")),
    "cfg5_long_all": (1, 1024, dict(d_hidden=768, num_heads=1, K=25, magnitude_type="cosine")),
    "cfg5_long_spatial": (1, 1024, dict(d_hidden=768, num_heads=1, K=9, magnitude_type="cosine",
                                        sampling_type="spatial", num_samples=256)),
    "h3_matmul": (2, 197, dict(d_hidden=192, num_heads=3, K=9, magnitude_type="matmul")),
    # kernel variants the baseline shapes leave out: standard conv over 192 channels (24 channel
    # groups), separable conv on 64-channel heads (one slice per head in the streaming kernel),
    # a head three GEMM tiles wide with the cosine statistic, a long sequence on the pair kernel
    "std_d192": (2, 197, dict(d_hidden=192, num_heads=1, K=9, magnitude_type="cosine", convolution_type="standard")),
    "dwsep_h3": (2, 197, dict(d_hidden=192, num_heads=3, K=9, magnitude_type="euclidean",
                              convolution_type="depthwise-separable")),
    "d768_cosine_short": (2, 197, dict(d_hidden=768, num_heads=1, K=9, magnitude_type="cosine")),
    "long_pair": (1, 1536, dict(d_hidden=128, num_heads=1, K=9, magnitude_type="cosine", seq_length=1536)),
    # the long-sequence sweep's own shape: 4096 tokens of 768 channels through all four stages (the
    # CTA-pair similarity kernel with 12 channel chunks per tile over a 5-stage ring)
    "cfg5_n4096_all": (1, 4096, dict(d_hidden=768, num_heads=1, K=9, magnitude_type="cosine", seq_length=4096)),
    "cfg5_n4096_spatial_k25": (1, 4096, dict(d_hidden=768, num_heads=1, K=25, magnitude_type="cosine",
                                             sampling_type="spatial", num_samples=1024, seq_length=4096)),
}


def _named_case(name):
    if name in BASELINE_SHAPES:
        B, T, kw = BASELINE_SHAPES[name]
        cfg = ConvNNConfig(**kw)
        cand = None
        if cfg.sampling_type == "random":
            cand = torch.randperm(T, generator=torch.Generator().manual_seed(17))[: cfg.num_samples]
        return cfg, make_layer_weights(cfg, seed=7), make_input(B, T, cfg.d_hidden, seed=11), None, cand
    return layer_case(name)


def rows_explained_by_rounding(sim_kernel, sim_oracle, idx_kernel, cfg, cand):
    """Rows (B, H, T) on which the kernel's exact selection over ITS similarities may differ from
    the oracle's exact selection over the oracle's.  Both lists are the best of the column set
    U = (oracle's top n+1) + (kernel's picks); if they differ, two columns of U have swapped
    order although their similarities moved by at most delta = max over U of |sim_kernel -
    sim_oracle|, so an adjacent gap of the oracle's top-(n+1) values is at most 2 delta.
    Returns (mask, delta)."""
    sampled = cand is not None
    n = cfg.K - 1 if sampled else cfg.K
    m = min(n + 1, sim_oracle.shape[-1])
    top_cols = torch.topk(sim_oracle, k=m, dim=-1, largest=cfg.maximum).indices
    if sampled:
        inv = torch.full((sim_oracle.shape[-2],), 0, dtype=torch.long)
        inv[cand] = torch.arange(cand.numel())
        picked = inv[idx_kernel[..., 1:]]
    else:
        picked = idx_kernel
    cols = torch.cat([top_cols, picked], dim=-1)
    delta = (sim_kernel - sim_oracle).abs().gather(-1, cols).amax(-1) + 1e-6
    return swap_possible_rows(sim_oracle, cfg, sampled, delta), delta


@pytest.mark.parametrize("name", LAYER_NAMES + sorted(BASELINE_SHAPES))
def test_bf16_stages_against_oracle(name):
    cfg, w, x, _, cand = _named_case(name)
    x = bf16_round(x)
    w = {n: bf16_round(t) for n, t in w.items()}
    tr = convnn_attention(x, w, cfg, cand=cand, policy="bf16")
    cand = tr.cand
    q, k, v, qs, ks, idx, val, o, out = run_stages(cfg, w, x, cand, torch.bfloat16)
    C, dk = cfg.in_channels, cfg.d_k
    # projections: equal up to one bfloat16 rounding step where the fp32 sums differ in order
    for got, ref in ((q, tr.q), (k, tr.k), (v, tr.v)):
        g = heads_to_oracle(got, C)
        assert float(((g - ref).abs() <= ref.abs() * 2.0 ** -7 + 1e-6).float().mean()) == 1.0
        assert float((g[..., :dk] == ref[..., :dk]).float().mean()) > 0.97
    # selection on the kernel's own q / k: fp32-exact products, so only sub-1e-6 gaps may differ
    qo, ko, vo = heads_to_oracle(q, C), heads_to_oracle(k, C), heads_to_oracle(v, C)
    sim = similarity(qo, ko, cfg, tr.cand)
    idx_want, val_want = select_neighbours(sim, cfg, tr.cand)
    ties = near_tie_rows(sim, cfg, cand is not None, FP32_TIE)
    same = (idx.cpu().long() == idx_want).all(-1)
    assert bool((same | ties).all()), f"{int((~(same | ties)).sum())} rows differ without a near-tie"
    dv = (val.cpu() - val_want).abs() / val_want.abs().clamp_min(1.0)
    assert float(dv[same].max()) < 5e-6
    # gather / conv / projection
    p = neighbour_weights(val.cpu(), cfg)
    assert rel_err(o, neighbour_conv(vo, idx.cpu().long(), p, w, cfg)) < BF16_OUT
    assert rel_err(out, from_neighbours(vo, idx.cpu(), val.cpu(), w, cfg)) < BF16_OUT
    # End to end against the oracle with the same rounding policy.  q and k of the two runs differ
    # where an fp32 sum rounded the other way (one bfloat16 step, checked above), which moves the
    # similarities a row's decision depends on by at most delta; every row whose ordered list
    # differs from the oracle's must be explained by that (see rows_explained_by_rounding).
    agree = (idx.cpu().long() == tr.idx).all(-1)
    explained, delta = rows_explained_by_rounding(sim, tr.sim, idx.cpu().long(), cfg, tr.cand)
    assert bool((agree | explained).all()), \
        f"{int((~(agree | explained)).sum())} rows differ from the oracle beyond what the q/k rounding explains"
    print(f"[{name}] rows agreeing with the bf16-policy oracle: {float(agree.float().mean()):.4f}; "
          f"delta median {float(delta.median()):.2e} max {float(delta.max()):.2e}")
    # (with thousands of candidates per row the top values crowd together and more rows sit within
    # 2 delta of a swap; the fraction is reported, the bound above is what must hold)
    assert float(agree.float().mean()) > (0.85 if x.shape[1] <= 2048 else 0.2)
    # per-head conv output on the agreeing rows (valid for every H: the head merge mixes rows)
    assert rel_err(o.float().cpu()[agree], tr.o[agree]) < BF16_OUT
    if cfg.num_heads == 1:
        rows = agree[:, 0]
        assert rel_err(out.float().cpu()[rows], tr.out[rows]) < BF16_OUT


def test_input_channel_slice_and_output_slice_are_used_in_place():
    """x[:, :, :d] of a wider tensor goes in through ldx, the result lands in a slice (ldo)."""
    cfg, w, x, want, _ = layer_case("cos_all_dw_h1")
    wide = torch.randn(x.shape[0], x.shape[1], 80, device=DEV)
    wide[:, :, :48] = x.to(DEV)
    dst = torch.full((x.shape[0], x.shape[1], 100), 7.0, device=DEV)
    m = module_of(cfg, w, torch.float32)
    with torch.no_grad():
        m(wide[:, :, :48], out=dst[:, :, :48])
    assert rel_err(dst[:, :, :48], want) < FP32_OUT
    assert bool((dst[:, :, 48:] == 7.0).all())


@pytest.mark.parametrize("T,K,H", [(1, 1, 1), (2, 2, 1), (9, 9, 1), (40, 32, 1), (129, 9, 1), (257, 4, 1),
                                   (197, 9, 3), (64, 16, 1)])
def test_small_and_ragged_shapes_fp32(T, K, H):
    D = 24 * H
    cfg = ConvNNConfig(d_hidden=D, num_heads=H, K=K, magnitude_type="cosine", seq_length=197)
    w = make_layer_weights(cfg, seed=3)
    x = make_input(3, T, D, seed=4)
    tr = convnn_attention(x, w, cfg)
    *_, idx, val, o, out = run_stages(cfg, w, x, None, torch.float32)
    ties = near_tie_rows(tr.sim, cfg, False, FP32_TIE)
    same = (idx.cpu().long() == tr.idx).all(-1)
    assert bool((same | ties).all())
    assert rel_err(out, from_neighbours(tr.v, idx.cpu(), val.cpu(), w, cfg)) < FP32_OUT


def test_exact_ties_keep_the_lower_candidate_column():
    """Duplicated tokens give exactly equal similarities; the documented rule is that the
    lower column wins (torch.topk's own order for ties is unspecified)."""
    cfg = ConvNNConfig(d_hidden=32, num_heads=1, K=4, magnitude_type="matmul")
    w = make_layer_weights(cfg, seed=3)
    x = make_input(1, 12, 32, seed=4)
    x[:, 6:] = x[:, :6]                       # token t+6 is a copy of token t
    *_, idx, val, o, out = run_stages(cfg, w, x, None, torch.float32)
    idx = idx.cpu()[0, 0]
    val = val.cpu()[0, 0]
    for r in range(12):
        for j in range(0, 4, 2):
            assert val[r, j] == val[r, j + 1]
            assert idx[r, j] + 6 == idx[r, j + 1]


def test_errors_match_reference_behaviour():
    cfg, w, x, _, _ = layer_case("cos_all_dw_h1")
    big = ConvNNConfig(d_hidden=48, num_heads=1, K=30, magnitude_type="cosine")
    m = module_of(big, make_layer_weights(big, seed=1), torch.float32)
    with torch.no_grad(), pytest.raises(RuntimeError, match="selected index k out of range"):
        m(torch.randn(1, 20, 48, device=DEV))
    h3 = ConvNNConfig(d_hidden=48, num_heads=3, K=5, magnitude_type="cosine")
    m = module_of(h3, make_layer_weights(h3, seed=1), torch.float32)
    with torch.no_grad(), pytest.raises(RuntimeError, match="is invalid for input of size"):
        m(torch.randn(2, 65, 48, device=DEV))
    with pytest.raises(RuntimeError, match="forward-only"):
        m(torch.randn(2, 197, 48, device=DEV))
    with torch.no_grad(), pytest.raises(TypeError):
        module_of(cfg, w, torch.float16)(x.to(DEV, torch.float16))


def test_random_sampling_consumes_the_generator_like_the_reference():
    """sampling_type='random' draws torch.randperm(T, device=x.device)[:n] per call."""
    cfg = ConvNNConfig(d_hidden=48, num_heads=1, K=5, sampling_type="random", num_samples=20,
                       magnitude_type="cosine")
    w = make_layer_weights(cfg, seed=2)
    x = make_input(2, 65, 48, seed=5)
    m = module_of(cfg, w, torch.float32)
    torch.manual_seed(99)
    cand = torch.randperm(65, device=DEV)[:20]
    torch.manual_seed(99)
    with torch.no_grad():
        y = m(x.to(DEV))
    tr = convnn_attention(x, w, cfg, cand=cand.cpu())
    assert rel_err(y, tr.out) < 1e-3           # near-ties aside, the same candidates were used
