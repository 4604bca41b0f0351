"""LayerNorm folded into the GEMM that consumes it (vit.py:262-269 of the reference computed without
materialising the normalised rows): the folded entry points against float64 arithmetic on the same
bfloat16 inputs, and against the library's own LayerNorm + GEMM order."""
import pytest
import torch
import torch.nn.functional as F

import convnn_b200
from convnn_b200 import _capi, ops
from oracle.convnn_oracle import ConvNNConfig, make_input, make_layer_weights
from gpu_util import DEV, module_of, rel_err

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def rnd(*shape, seed, scale=1.0, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale + shift).to(BF).to(DEV)


@pytest.mark.parametrize("rows,D", [(1, 192), (777, 192), (300, 768), (65, 64)])
def test_row_moments(rows, D):
    x = rnd(rows, D, seed=1, shift=0.5)
    m = ops.row_moments(x)
    assert m.shape == (1, rows + rows % 2, 2)
    xd = x.double()
    assert torch.allclose(m[0, :rows, 0].double(), xd.sum(1), rtol=1e-5, atol=1e-4)
    assert torch.allclose(m[0, :rows, 1].double(), (xd * xd).sum(1), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("M,N,K,bias", [(777, 192, 768, True), (50432, 192, 768, True), (1000, 192, 192, False),
                                         (300, 768, 768, True), (130, 80, 64, True)])
def test_linear_moments_is_linear_plus_row_sums(M, N, K, bias):
    """Same bits as convnn_b200_linear with the skip connection; the planes add up to the moments of
    the stored rows."""
    a, w, res = rnd(M, K, seed=2), rnd(N, K, seed=3, scale=K ** -0.5), rnd(M, N, seed=4)
    b = rnd(N, seed=5) if bias else None
    want = ops.linear(a, w, b, residual=res)
    got, mom = ops.linear_moments(a, w, b, res)
    assert torch.equal(got, want)
    assert mom.shape == (_capi.lib().convnn_b200_moment_planes(N), M + M % 2, 2)
    gd = got.double()
    tot = mom.double()[:, :M].sum(0)
    assert torch.allclose(tot[:, 0], gd.sum(1), rtol=1e-5, atol=1e-3)
    assert torch.allclose(tot[:, 1], (gd * gd).sum(1), rtol=1e-5, atol=1e-3)
    assert _capi.device_status() == 0


def layernorm_linear_f64(x, gamma, beta, w, b, eps, gelu):
    y = F.layer_norm(x.double(), (x.shape[-1],), gamma.double(), beta.double(), eps)
    out = y @ w.double().t()
    if b is not None:
        out = out + b.double()
    return F.gelu(out) if gelu else out


@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("M,N,K,shift", [(777, 768, 192, 0.0), (1, 768, 192, 0.0), (50432, 768, 192, 0.0), (1000, 192, 192, 3.0),
                                          (129, 576, 192, -1.0), (4000, 256, 64, 0.5)])
def test_prenorm_linear_against_float64(M, N, K, shift, gelu):
    """[GELU](LayerNorm(x) W^T + b) from the raw rows and their moments: within the bfloat16 output
    tolerance (2e-2, relative to the output's scale) of float64 arithmetic on the same inputs, and no
    worse than LayerNorm kernel + GEMM; rows with a mean several times their spread included."""
    assert ops.prenorm_linear_supported(N, K, gelu)
    x = rnd(M, K, seed=6, shift=shift)
    gamma, beta = rnd(K, seed=7, scale=0.2, shift=1.0), rnd(K, seed=8, scale=0.2)
    w, b = rnd(N, K, seed=9, scale=K ** -0.5), rnd(N, seed=10, scale=0.3)
    wf, wx = ops.fold_layernorm(w, b, gamma, beta)
    got = ops.prenorm_linear(x, ops.row_moments(x), 1e-5, wf, wx, gelu=gelu)
    want = layernorm_linear_f64(x, gamma, beta, w, b, 1e-5, gelu)
    unfused = ops.linear(ops.layernorm(x, gamma, beta, 1e-5), w, b, gelu=gelu)
    scale = want.abs().max().item()
    err = (got.double().cpu() - want.cpu()).abs().max().item() / scale
    err_unfused = (unfused.double().cpu() - want.cpu()).abs().max().item() / scale
    print(f"max err / scale: folded {err:.2e}, LayerNorm + GEMM {err_unfused:.2e}")
    assert err < 2e-2
    assert rel_err(got, want) < 6e-3
    assert _capi.device_status() == 0


def test_prenorm_linear_takes_moments_in_several_planes():
    """The consumer adds the planes up: moments split arbitrarily over three planes give the same bits."""
    M, N, K = 500, 768, 192
    x, gamma, beta = rnd(M, K, seed=11), rnd(K, seed=12, shift=1.0, scale=0.1), rnd(K, seed=13, scale=0.1)
    w = rnd(N, K, seed=14, scale=K ** -0.5)
    wf, wx = ops.fold_layernorm(w, None, gamma, beta)
    m = ops.row_moments(x)
    parts = torch.stack([m[0] * 0.25, m[0] * 0.5, m[0] * 0.25]).contiguous()
    a = ops.prenorm_linear(x, m, 1e-5, wf, wx)
    b = ops.prenorm_linear(x, parts, 1e-5, wf, wx)
    assert torch.equal(a, b)


def test_unsupported_shapes_are_refused_not_computed():
    assert not ops.prenorm_linear_supported(3072, 768, True)       # the W tile does not fit in shared memory
    x = rnd(64, 768, seed=15)
    wf, wx = torch.zeros(3072, 768, dtype=BF, device=DEV), torch.zeros(3072, 16, dtype=BF, device=DEV)
    with pytest.raises(_capi.ConvnnError):
        ops.prenorm_linear(x, ops.row_moments(x), 1e-5, wf, wx, gelu=True)


@pytest.mark.parametrize("metric,H", [("cosine", 1), ("euclidean", 1), ("matmul", 1), ("cosine", 3)])
def test_prenorm_forward_matches_layernorm_then_forward(metric, H):
    """norm1 folded into the K/V/Q projection: the layer output (with the skip connection) agrees with
    LayerNorm kernel + convnn_b200_forward except on rows whose neighbour choice sits on a near-tie, and
    the emitted moments are those of the stored rows."""
    B, T, D = 8, 197, 192
    cfg = ConvNNConfig(d_hidden=D, num_heads=H, K=9, magnitude_type=metric, seq_length=T)
    layer = module_of(cfg, make_layer_weights(cfg, seed=21), BF)
    norm = torch.nn.LayerNorm(D).to(DEV, BF)
    with torch.no_grad():
        norm.weight.copy_(rnd(D, seed=22, scale=0.1, shift=1.0))
        norm.bias.copy_(rnd(D, seed=23, scale=0.1))
        x = rnd(B, T, D, seed=24, shift=0.3)
        assert layer.prenorm_supported(x)
        got, mom = layer.forward_prenorm(x, ops.row_moments(x), norm, residual=x, want_moments=True)
        want = layer(ops.layernorm(x, norm.weight, norm.bias, norm.eps), residual=x)
    assert _capi.device_status() == 0
    diff = (got.float() - want.float()).abs().amax(-1)
    scale = want.float().abs().amax().item()
    close = (diff < 2e-2 * scale).float().mean().item()
    print(f"rows within 2e-2 of the unfused order: {close:.4f}")
    assert close > 0.97
    gd = got.double().view(B * T, D)
    tot = mom.double()[:, : B * T].sum(0)
    assert torch.allclose(tot[:, 0], gd.sum(1), rtol=1e-5, atol=1e-3)
    assert torch.allclose(tot[:, 1], (gd * gd).sum(1), rtol=1e-5, atol=1e-3)


def test_vit_with_and_without_the_fold():
    """Whole model (ViT-Tiny shape, 4 layers): folding both LayerNorms of every block changes where
    bfloat16 roundings happen, not what is computed."""
    from oracle.vit_oracle import ViTConfig, make_images, make_vit_weights
    from oracle.convnn_oracle import bf16_round
    cfg = ViTConfig(layer="ConvNNAttention", d_hidden=192, d_mlp=768, num_heads=1, num_layers=4,
                    magnitude_type="cosine", convolution_type="depthwise")
    sd = {k: bf16_round(v) for k, v in make_vit_weights(cfg, seed=5).items()}
    args = convnn_b200.make_args(**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__}, device=DEV)
    model = convnn_b200.ViT(args).eval()
    model.load_state_dict(sd, strict=True)
    model = model.to(DEV, BF)
    img = bf16_round(make_images(4, cfg, seed=6)).to(DEV, BF)
    lib = _capi.lib()
    with torch.no_grad():
        model(img)                                   # builds the folded weights (two launches per block, once)
        n0 = lib.convnn_b200_launch_count()
        folded = model(img).float()
        n1 = lib.convnn_b200_launch_count()
        for blk in model.transformer_encoder:
            blk.fold_layernorm = False
        plain = model(img).float()
        n2 = lib.convnn_b200_launch_count()
    assert _capi.device_status() == 0
    # per block: two LayerNorm launches and (fused MLP) one GEMM launch fewer; the first block's row
    # moments come from the embedding's last kernel, not from a launch of their own
    assert (n2 - n1) - (n1 - n0) == 3 * cfg.num_layers
    err = rel_err(folded, plain)
    print(f"logits, folded against unfused: rel err {err:.3e}")
    assert err < 0.1


def test_patch_embed_emits_the_moments_of_the_rows_it_stores():
    """The embedding's last kernel (LayerNorm + class token + positional table) also writes (sum, sum of
    squares) of every stored row, class-token rows included: the same numbers row_moments computes from
    the result, and the result itself is unchanged by asking for them."""
    B, C, HW, P, D = 5, 3, 64, 16, 192
    Np = (HW // P) ** 2
    img = rnd(B, C, HW, HW, seed=71)
    w, b = rnd(D, C, P, P, seed=72, scale=(C * P * P) ** -0.5), rnd(D, seed=73, scale=0.1)
    g, bt = rnd(D, seed=74, scale=0.2, shift=1.0), rnd(D, seed=75, scale=0.2)
    cls, pe = rnd(1, 1, D, seed=76), rnd(1, Np + 1, D, seed=77)
    plain = ops.patch_embed(img, w, b, g, bt, cls, pe, P)
    out, mom = ops.patch_embed(img, w, b, g, bt, cls, pe, P, want_moments=True)
    torch.cuda.synchronize()
    assert torch.equal(out, plain)
    M = B * (Np + 1)
    assert mom.shape == (1, _capi.lib().convnn_b200_moment_stride(M), 2)
    want = ops.row_moments(out)
    assert torch.allclose(mom[0, :M], want[0, :M], rtol=1e-5, atol=1e-4)
    od = out.double().view(M, D)
    assert torch.allclose(mom[0, :M, 0].double(), od.sum(1), rtol=1e-5, atol=1e-3)
    assert torch.allclose(mom[0, :M, 1].double(), (od * od).sum(1), rtol=1e-5, atol=1e-3)


def mlp_f64(x, gamma, beta, w1, b1, w2, b2, eps):
    xd = x.double()
    y = F.layer_norm(xd, (x.shape[-1],), gamma.double(), beta.double(), eps)
    h = F.gelu(y @ w1.double().t() + b1.double())
    out = h @ w2.double().t()
    if b2 is not None:
        out = out + b2.double()
    return xd + out


@pytest.mark.parametrize("M,D,DM,shift,bias2", [(777, 192, 768, 0.0, True), (1, 192, 768, 0.0, True), (256, 192, 768, 2.0, False),
                                                (50432, 192, 768, 0.0, True), (5000, 192, 768, -1.0, True),
                                                (1000, 128, 512, 0.5, True), (1000, 64, 256, 0.0, True),
                                                (300, 192, 1536, 0.0, True),
                                                # odd and single super-chunk counts, several tiles per cluster
                                                (60000, 192, 384, 0.0, True), (60000, 128, 128, 0.0, True),
                                                (40000, 64, 640, 0.3, False)])
def test_prenorm_mlp_against_float64(M, D, DM, shift, bias2):
    """The whole MLP block in one kernel (norm2 folded, GELU, both Linear layers, skip connection): within
    the bfloat16 tolerance of float64 arithmetic on the same inputs and as close as the two-kernel path
    (prenorm_linear + linear_moments); the emitted moments are those of the stored rows; ragged last
    tiles, a single row, rows with a large mean, every supported width."""
    assert ops.prenorm_mlp_supported(D, DM, 1)
    x = rnd(M, D, seed=31, shift=shift)
    gamma, beta = rnd(D, seed=32, scale=0.2, shift=1.0), rnd(D, seed=33, scale=0.2)
    w1, b1 = rnd(DM, D, seed=34, scale=D ** -0.5), rnd(DM, seed=35, scale=0.3)
    w2, b2 = rnd(D, DM, seed=36, scale=DM ** -0.5), (rnd(D, seed=37, scale=0.3) if bias2 else None)
    wf, wx = ops.fold_layernorm(w1, b1, gamma, beta)
    mom = ops.row_moments(x)
    got, mo = ops.prenorm_mlp(x, mom, 1e-5, wf, wx, w2, b2, want_moments=True)
    again, _ = ops.prenorm_mlp(x, mom, 1e-5, wf, wx, w2, b2)
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    assert torch.equal(got, again)
    want = mlp_f64(x, gamma, beta, w1, b1, w2, b2, 1e-5)
    two = ops.linear(ops.prenorm_linear(x, mom, 1e-5, wf, wx, gelu=True), w2, b2, residual=x)
    scale = want.abs().max().item()
    err = (got.double() - want).abs().max().item() / scale
    err_two = (two.double() - want).abs().max().item() / scale
    print(f"max err / scale: one kernel {err:.2e}, two kernels {err_two:.2e}")
    assert err < 2e-2 and err < 1.5 * err_two + 1e-3
    assert rel_err(got, want) < 6e-3
    gd = got.double()
    tot = mo.double()[:, :M].sum(0)
    assert torch.allclose(tot[:, 0], gd.sum(1), rtol=1e-5, atol=1e-3)
    assert torch.allclose(tot[:, 1], (gd * gd).sum(1), rtol=1e-5, atol=1e-3)


def test_prenorm_mlp_takes_moments_in_several_planes_and_refuses_other_shapes():
    M, D, DM = 600, 192, 768
    x, gamma, beta = rnd(M, D, seed=41), rnd(D, seed=42, shift=1.0, scale=0.1), rnd(D, seed=43, scale=0.1)
    w1, b1, w2 = rnd(DM, D, seed=44, scale=D ** -0.5), rnd(DM, seed=45), rnd(D, DM, seed=46, scale=DM ** -0.5)
    wf, wx = ops.fold_layernorm(w1, b1, gamma, beta)
    m = ops.row_moments(x)
    parts = torch.stack([m[0] * 0.25, m[0] * 0.5, m[0] * 0.25]).contiguous()
    a, _ = ops.prenorm_mlp(x, m, 1e-5, wf, wx, w2, None)
    b, _ = ops.prenorm_mlp(x, parts, 1e-5, wf, wx, w2, None)
    assert torch.equal(a, b)
    assert not ops.prenorm_mlp_supported(768, 3072, 2) and not ops.prenorm_mlp_supported(192, 704, 2)
    with pytest.raises(_capi.ConvnnError):
        ops.prenorm_mlp(rnd(64, 768, seed=47), ops.row_moments(rnd(64, 768, seed=47)), 1e-5,
                        torch.zeros(3072, 768, dtype=BF, device=DEV), torch.zeros(3072, 16, dtype=BF, device=DEV),
                        torch.zeros(768, 3072, dtype=BF, device=DEV), None)


@pytest.mark.parametrize("M,D,DM,shift", [(777, 192, 768, 0.0), (1, 192, 768, 0.0), (50432, 192, 768, 1.0),
                                          (1000, 128, 512, 0.0), (1000, 64, 256, -0.5), (600, 192, 256, 0.0)])
def test_outproj_mlp_against_float64_and_the_separate_kernels(M, D, DM, shift):
    """W_o + skip + norm2 + mlp + skip in one kernel: x1 = x + o W_o^T is formed inside (and its moments with
    it); the result agrees with float64 arithmetic from the rounded x1 as well as linear(+skip) followed by
    the one-kernel MLP does, and the emitted moments are those of the stored rows."""
    x, o = rnd(M, D, seed=51, shift=shift), rnd(M, D, seed=52)
    wo = rnd(D, D, seed=53, scale=D ** -0.5)
    gamma, beta = rnd(D, seed=54, scale=0.2, shift=1.0), rnd(D, seed=55, scale=0.2)
    w1, b1 = rnd(DM, D, seed=56, scale=D ** -0.5), rnd(DM, seed=57, scale=0.3)
    w2, b2 = rnd(D, DM, seed=58, scale=DM ** -0.5), rnd(D, seed=59, scale=0.3)
    wf, wx = ops.fold_layernorm(w1, b1, gamma, beta)
    got, mo = ops.outproj_mlp(o, wo, x, 1e-5, wf, wx, w2, b2, want_moments=True)
    again, _ = ops.outproj_mlp(o, wo, x, 1e-5, wf, wx, w2, b2)
    torch.cuda.synchronize()
    assert _capi.device_status() == 0
    assert torch.equal(got, again)
    x1 = ops.linear(o, wo, None, residual=x)
    sep, _ = ops.prenorm_mlp(x1, ops.row_moments(x1), 1e-5, wf, wx, w2, b2)
    want = mlp_f64(x1, gamma, beta, w1, b1, w2, b2, 1e-5)
    scale = want.abs().max().item()
    err = (got.double() - want).abs().max().item() / scale
    err_sep = (sep.double() - want).abs().max().item() / scale
    print(f"max err / scale: one kernel {err:.2e}, output projection + MLP kernel {err_sep:.2e}")
    assert err < 2e-2 and err < 1.5 * err_sep + 1e-3
    gd = got.double()
    tot = mo.double()[:, :M].sum(0)
    assert torch.allclose(tot[:, 0], gd.sum(1), rtol=1e-5, atol=1e-3)
    assert torch.allclose(tot[:, 1], (gd * gd).sum(1), rtol=1e-5, atol=1e-3)


def test_vit_with_the_output_projection_inside_the_mlp_kernel():
    """`fuse_out_proj` (off by default): same model, W_o + skip handled by the MLP kernel; logits agree with the
    default path and one more launch per block disappears."""
    from oracle.vit_oracle import ViTConfig, make_images, make_vit_weights
    from oracle.convnn_oracle import bf16_round
    cfg = ViTConfig(layer="ConvNNAttention", d_hidden=192, d_mlp=768, num_heads=1, num_layers=3,
                    magnitude_type="cosine", convolution_type="depthwise")
    sd = {k: bf16_round(v) for k, v in make_vit_weights(cfg, seed=7).items()}
    args = convnn_b200.make_args(**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__}, device=DEV)
    model = convnn_b200.ViT(args).eval()
    model.load_state_dict(sd, strict=True)
    model = model.to(DEV, BF)
    img = bf16_round(make_images(3, cfg, seed=8)).to(DEV, BF)
    lib = _capi.lib()
    with torch.no_grad():
        model(img)
        n0 = lib.convnn_b200_launch_count()
        base = model(img).float()
        n1 = lib.convnn_b200_launch_count()
        for blk in model.transformer_encoder:
            blk.fuse_out_proj = True
        fused = model(img).float()
        n2 = lib.convnn_b200_launch_count()
    assert _capi.device_status() == 0
    assert (n1 - n0) - (n2 - n1) == cfg.num_layers
    err = rel_err(fused, base)
    print(f"logits, W_o inside the MLP kernel against the default path: rel err {err:.3e}")
    assert err < 0.05
