"""The tcgen05 similarity/top-K kernel on shapes that exercise every tiling path:
several row tiles, several column tiles with a ragged last tile, the 128/64/32-byte
swizzle chunkings (d_k multiple of 64 / 32 / 16), K up to 32, sampled masks, and the
CTA-pair kernel that takes over on long sequences."""
import pytest
import torch

from convnn_b200 import _capi, ops
from oracle.convnn_oracle import ConvNNConfig, near_tie_rows, select_neighbours, similarity
from gpu_util import DEV, spec_of

pytestmark = pytest.mark.gpu

CASES = [
    # B, T, S, D, H, K, metric, sampling
    (3, 197, 197, 192, 1, 9, "cosine", "all"),
    (2, 300, 300, 64, 1, 25, "cosine", "all"),
    (2, 700, 700, 128, 2, 9, "matmul", "all"),
    (2, 197, 64, 384, 1, 9, "euclidean", "random"),
    (1, 1024, 256, 96, 1, 9, "cosine", "spatial"),
    (2, 197, 197, 384, 12, 9, "cosine", "all"),
    (1, 130, 130, 48, 1, 32, "euclidean", "all"),
    (1, 1030, 1030, 64, 1, 4, "cosine", "all"),
    (2, 50, 17, 32, 1, 16, "matmul", "random"),
    # short candidate lists: full 256-candidate set, tiny candidate sets, several row tiles, one pick
    (1, 256, 256, 64, 2, 12, "euclidean", "all"),
    (2, 300, 40, 64, 1, 9, "cosine", "random"),
    (1, 20, 20, 32, 1, 16, "matmul", "all"),
    (3, 700, 33, 160, 5, 2, "cosine", "spatial"),
    (2, 197, 197, 96, 3, 1, "matmul", "all"),
    # long key and candidate lists: the CTA-pair kernel (256-row units, 256-column tiles, ragged ends)
    (2, 1536, 1200, 128, 2, 9, "euclidean", "random"),
    (1, 2048, 2048, 192, 1, 16, "matmul", "all"),
    (1, 1300, 1300, 64, 1, 9, "cosine", "all"),
    (1, 1100, 1100, 64, 1, 25, "cosine", "all"),      # long lists on short sequences stay on the single-CTA kernel
    (1, 8200, 4100, 64, 1, 25, "cosine", "spatial"),  # ... and move to the pair kernel on long ones
    (1, 8192, 4096, 64, 1, 32, "euclidean", "random"),
    # the pair kernel at the channel count of the long-sequence sweep: d_k = 768 is 12 chunks per
    # tile wrapping around the 5-stage (4-stage for lists longer than 24) shared-memory ring
    (1, 2048, 2048, 768, 1, 9, "cosine", "all"),
    (1, 4096, 1024, 768, 1, 9, "cosine", "spatial"),
    (1, 8192, 4096, 768, 1, 25, "cosine", "spatial"),
]


@pytest.mark.parametrize("B,T,S,D,H,K,metric,sampling", CASES)
def test_tensor_core_topk_matches_oracle(B, T, S, D, H, K, metric, sampling):
    g = torch.Generator().manual_seed(B * 1000 + T)
    dk = D // H
    q = torch.randn(B, S, H, dk, generator=g).to(torch.bfloat16)
    k = torch.randn(B, T, H, dk, generator=g).to(torch.bfloat16)
    cand = None
    if sampling != "all":
        cand = torch.randperm(T, generator=g)[:S] if sampling == "random" else torch.linspace(0, T - 1, S).long()
    cfg = ConvNNConfig(d_hidden=D, num_heads=H, K=K, sampling_type=sampling, num_samples=S, magnitude_type=metric,
                       seq_length=T)
    qo, ko = q.float().permute(0, 2, 1, 3), k.float().permute(0, 2, 1, 3)     # (B,H,rows,dk)
    if metric == "cosine":
        qstat, kstat = 1.0 / qo.norm(dim=-1).clamp_min(1e-12), 1.0 / ko.norm(dim=-1).clamp_min(1e-12)
    else:
        qstat, kstat = (qo * qo).sum(-1), (ko * ko).sum(-1)
    sim = similarity(qo, ko, cfg, cand, dtype=torch.float64)
    idx_want, val_want = select_neighbours(sim, cfg, cand)
    spec = spec_of(cfg)
    idx, val = ops.sim_topk(spec, q.to(DEV), k.to(DEV), qstat.contiguous().to(DEV), kstat.contiguous().to(DEV),
                            None if cand is None else cand.to(DEV))
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    ties = near_tie_rows(sim, cfg, cand is not None, 2e-6)
    same = (idx.cpu().long() == idx_want).all(-1)
    assert bool((same | ties).all()), f"{int((~(same | ties)).sum())} rows differ without a near-tie"
    assert float(ties.float().mean()) < 0.08    # (25 gaps per row among thousands of candidates: ~5 % at 2e-6)
    dv = (val.cpu().double() - val_want).abs() / val_want.abs().clamp_min(1.0)
    assert float(dv[same].max()) < 1e-5


@pytest.mark.parametrize("S,K,sampling", [(16384, 9, "all"), (4096, 25, "spatial")])
def test_pair_kernel_at_16384_tokens_against_float64_rows(S, K, sampling):
    """The largest shape of the long-sequence sweep (16384 tokens of 768 channels): the whole
    launch runs, and a seeded sample of 256 key rows is compared with a float64 similarity over
    all candidates (the full 16384 x 16384 matrix is never formed, here or in the kernel)."""
    T, D, n_rows = 16384, 768, 256
    g = torch.Generator().manual_seed(S + K)
    q = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, T, 1, D, generator=g).to(torch.bfloat16)
    cand = None if sampling == "all" else torch.linspace(0, T - 1, S).long()
    cfg = ConvNNConfig(d_hidden=D, num_heads=1, K=K, sampling_type=sampling, num_samples=S, magnitude_type="cosine",
                       seq_length=T)
    qo, ko = q.float().permute(0, 2, 1, 3), k.float().permute(0, 2, 1, 3)
    qstat, kstat = 1.0 / qo.norm(dim=-1).clamp_min(1e-12), 1.0 / ko.norm(dim=-1).clamp_min(1e-12)
    idx, val = ops.sim_topk(spec_of(cfg), q.to(DEV), k.to(DEV), qstat.contiguous().to(DEV), kstat.contiguous().to(DEV),
                            None if cand is None else cand.to(DEV))
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    idx, val = idx.cpu().long(), val.cpu().double()
    # properties of every row
    n = K if cand is None else K - 1
    own = 0 if cand is None else 1
    assert int(idx.min()) >= 0 and int(idx.max()) < T
    assert bool((val[..., own:-1] >= val[..., own + 1:]).all()), "values not sorted best first"
    srt = idx[..., own:].sort(-1).values
    assert bool((srt[..., 1:] != srt[..., :-1]).all()), "duplicate neighbour in a row"
    # float64 check of the sampled rows
    rows = torch.randperm(T, generator=g)[:n_rows].sort().values
    kd = ko[0, 0, rows].double()
    qd = qo[0, 0].double()
    sim = (kd / kd.norm(dim=-1, keepdim=True)) @ (qd / qd.norm(dim=-1, keepdim=True)).t()     # (n_rows, S)
    if cand is not None:
        own_col = (cand.view(1, -1) == rows.view(-1, 1))
        sim = torch.where(own_col, torch.full_like(sim, -0.1), sim)
    top, cols = torch.topk(sim, n + 1, dim=-1)
    want = cols[:, :n] if cand is None else cand[cols[:, :n]]
    gaps = (top[:, :-1] - top[:, 1:]).abs()
    ties = (gaps < 2e-6).any(-1)
    got = idx[0, 0, rows][:, own:]
    same = (got == want).all(-1)
    assert bool((same | ties).all()), f"{int((~(same | ties)).sum())} of {n_rows} rows differ without a near-tie"
    assert float(ties.float().mean()) < 0.1
    dv = (val[0, 0, rows][:, own:] - top[:, :n]).abs()
    assert float(dv[same].max()) < 1e-5
    if cand is not None:
        assert bool((idx[0, 0, :, 0] == torch.arange(T)).all()) and bool((val[0, 0, :, 0] == 1.0).all())


def test_tensor_core_and_simt_kernels_agree_bitwise_on_indices():
    """Same q / k through the SIMT float path (q, k upcast) and the tensor-core path."""
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 197, 1, 192, generator=g).to(torch.bfloat16)
    k = torch.randn(2, 197, 1, 192, generator=g).to(torch.bfloat16)
    cfg = ConvNNConfig(d_hidden=192, num_heads=1, K=9, magnitude_type="matmul")
    spec = spec_of(cfg)
    i16, v16 = ops.sim_topk(spec, q.to(DEV), k.to(DEV), None, None)
    i32, v32 = ops.sim_topk(spec, q.float().to(DEV), k.float().to(DEV), None, None)
    same = (i16 == i32).all(-1)
    assert float(same.float().mean()) > 0.999
    assert float((v16 - v32).abs().max()) < 1e-4


def test_short_sequence_exact_ties_keep_the_lower_column():
    """The ViT shapes on the tensor-core kernel: identical candidate rows in the same and in
    different column tiles, a key row of zeros (every similarity ties) and a row with ties exactly
    at the K-th place.  Expected order: by value, equal values by ascending column."""
    g = torch.Generator().manual_seed(21)
    T = S = 197
    q = torch.randn(2, S, 1, 64, generator=g).to(torch.bfloat16)
    k = torch.randn(2, T, 1, 64, generator=g).to(torch.bfloat16)
    q[0, 150] = q[0, 20]           # lower and upper column range
    q[0, 30] = q[0, 21]            # both in the lower range
    k[0, 5] = q[0, 20]
    k[0, 100] = q[0, 21]
    k[0, 7] = 0                    # all 197 similarities are exactly 0
    q[1, 40:60] = q[1, 40]         # twenty equal candidates: ties at and around the K-th place
    k[1, 3] = q[1, 40]
    cfg = ConvNNConfig(d_hidden=64, num_heads=1, K=9, magnitude_type="matmul", seq_length=T)
    idx, val = ops.sim_topk(spec_of(cfg), q.to(DEV), k.to(DEV), None, None)
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    sim = (k[:, :, 0].double() @ q[:, :, 0].double().transpose(1, 2)) / 8.0          # exact in float64
    order = torch.sort(sim, dim=-1, descending=True, stable=True).indices[..., :9]
    top = sim.gather(-1, order)
    nxt = torch.sort(sim, dim=-1, descending=True, stable=True).values[..., :10]
    gaps = (nxt[..., :-1] - nxt[..., 1:])
    loose = ((gaps > 0) & (gaps < 2e-6)).any(-1)      # near-ties (not exact ties) may go either way
    same = (idx[:, 0].cpu().long() == order).all(-1)
    assert bool((same | loose).all()), f"{int((~(same | loose)).sum())} rows break the tie rule"
    assert idx[0, 0, 5, :2].tolist() == [20, 150] and idx[0, 0, 100, :2].tolist() == [21, 30]
    assert idx[0, 0, 7].tolist() == list(range(9)) and bool((val[0, 0, 7] == 0).all())
    assert idx[1, 0, 3].tolist() == list(range(40, 49))
    assert float((val[:, 0].cpu().double() - top)[same].abs().max()) < 1e-5


def test_pair_kernel_orders_exact_ties_by_column():
    """Two identical candidate rows whose columns fall into different column halves of
    different tiles (130: upper half of tile 0, 300: lower half of tile 1): both are selected
    by the key rows that resemble them, and the lower column comes first."""
    g = torch.Generator().manual_seed(11)
    T = S = 1024
    q = torch.randn(1, S, 1, 64, generator=g).to(torch.bfloat16)
    k = torch.randn(1, T, 1, 64, generator=g).to(torch.bfloat16)
    q[0, 300] = q[0, 130]
    k[0, 5] = q[0, 130]
    k[0, 700] = q[0, 130]
    cfg = ConvNNConfig(d_hidden=64, num_heads=1, K=9, magnitude_type="matmul", seq_length=T)
    idx, val = ops.sim_topk(spec_of(cfg), q.to(DEV), k.to(DEV), None, None)
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    for row in (5, 700):
        got = idx[0, 0, row].tolist()
        assert got[0] == 130 and got[1] == 300, got
        assert float(val[0, 0, row, 0]) == float(val[0, 0, row, 1])


def test_pair_kernel_and_simt_kernel_agree_on_long_sequences():
    """Same q / k through the float32 SIMT path (q, k upcast) and the CTA-pair tensor-core path."""
    g = torch.Generator().manual_seed(7)
    q = torch.randn(1, 2100, 1, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 2100, 1, 128, generator=g).to(torch.bfloat16)
    cfg = ConvNNConfig(d_hidden=128, num_heads=1, K=9, magnitude_type="matmul", seq_length=2100)
    spec = spec_of(cfg)
    i16, v16 = ops.sim_topk(spec, q.to(DEV), k.to(DEV), None, None)
    i32, v32 = ops.sim_topk(spec, q.float().to(DEV), k.float().to(DEV), None, None)
    same = (i16 == i32).all(-1)
    assert float(same.float().mean()) > 0.999
    assert float((v16 - v32).abs().max()) < 1e-4


def test_long_sequence_layer_replays_from_a_cuda_graph():
    """The cluster launch of the pair kernel (and everything else in the layer) can be captured:
    a replayed graph reproduces the eager result bit for bit."""
    import convnn_b200
    layer = convnn_b200.MultiHeadConvNNAttention(128, 1, 0.0, 9, "all", -1, 0, "cosine", seq_length=1280)
    layer = layer.eval().to(DEV, torch.bfloat16)
    x = torch.randn(2, 1280, 128, generator=torch.Generator().manual_seed(9)).to(DEV, torch.bfloat16)
    with torch.no_grad():
        want = layer(x)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            layer(x)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            got = layer(x)
        g.replay()
        torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert _capi.device_status() == 0
