"""The allocation-free forward (convnn_b200_forward_noalloc), collected last on purpose.

Some callers may not allocate device memory at the point where they run the layer (inside a
serving loop where cudaMalloc would stall the GPU, from a plugin whose host owns the
allocator, on a GPU whose memory is already handed out).  For them the library keeps the layer's intermediates in a
fixed 32 MiB array of its own.  This test calls that entry point through the C ABI twice in a
row, with different inputs, and requires the same output as the ordinary entry point that is
given a workspace; it also checks that a shape too large for the built-in array is refused.
"""
import pytest
import torch

from convnn_b200 import _capi, ops
from oracle.convnn_oracle import ConvNNConfig, bf16_round, make_input, make_layer_weights
from gpu_util import DEV, pack, spec_of

pytestmark = pytest.mark.gpu


def _call_noalloc(spec, x, packed, cand=None):
    L = _capi.lib()
    w_qkv, w_conv, w_pw, w_o = packed
    B, T, D = x.shape
    S = T if cand is None else int(cand.numel())
    d = ops.descriptor(spec, B, T, S, x.dtype)
    out = torch.empty_like(x)
    rc = L.convnn_b200_forward_noalloc(d, x.data_ptr(), D, w_qkv.data_ptr(), w_conv.data_ptr(), _capi.ptr(w_pw),
                                       w_o.data_ptr(), _capi.ptr(cand), None, 0, out.data_ptr(), D,
                                       torch.cuda.current_stream().cuda_stream)
    return rc, out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_forward_matches_workspace_forward_twice(dtype):
    cfg = ConvNNConfig(d_hidden=192, num_heads=1, K=9, magnitude_type="cosine")
    w = {n: bf16_round(t) for n, t in make_layer_weights(cfg, seed=5).items()}
    spec, packed = spec_of(cfg), pack(cfg, w, dtype)
    for seed in (1, 2):                                    # two calls in a row share the built-in array
        x = make_input(8, 197, 192, seed=seed).to(DEV, dtype)
        want = ops.forward(spec, x, packed)
        rc, got = _call_noalloc(spec, x, packed)
        _capi.check(rc)
        torch.cuda.synchronize()
        assert torch.equal(got, want)                      # same kernels, same order: bit-identical
    assert _capi.device_status() == 0


def test_noalloc_forward_takes_no_device_memory_after_warm_up():
    """The built-in array is reserved when its CUDA module is first touched on a device, which
    convnn_b200_noalloc_capacity() does (the start-up warm-up the header asks for).  After that
    a forward must leave the device's free memory exactly as it found it."""
    L = _capi.lib()
    assert L.convnn_b200_noalloc_capacity() == 32 << 20           # warm-up: resolves the address
    cfg = ConvNNConfig(d_hidden=192, num_heads=1, K=9, magnitude_type="cosine")
    spec, packed = spec_of(cfg), pack(cfg, make_layer_weights(cfg, seed=5), torch.bfloat16)
    w_qkv, w_conv, w_pw, w_o = packed
    x = make_input(8, 197, 192, seed=1).to(DEV, torch.bfloat16)
    out = torch.empty_like(x)
    d = ops.descriptor(spec, 8, 197, 197, x.dtype)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        return L.convnn_b200_forward_noalloc(d, x.data_ptr(), 192, w_qkv.data_ptr(), w_conv.data_ptr(), None,
                                             w_o.data_ptr(), None, None, 0, out.data_ptr(), 192, stream)
    _capi.check(call())                                           # kernels loaded, attributes set
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    _capi.check(call())
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.equal(out, ops.forward(spec, x, packed))


def test_noalloc_forward_sampled_mode_and_heads():
    cfg = ConvNNConfig(d_hidden=96, num_heads=3, K=9, magnitude_type="euclidean", sampling_type="spatial",
                       num_samples=49, convolution_type="depthwise-separable")
    w = make_layer_weights(cfg, seed=3)
    spec, packed = spec_of(cfg), pack(cfg, w, torch.float32)
    cand = torch.linspace(0, 196, 49).long().to(DEV, torch.int32)
    for seed in (4, 5):
        x = make_input(2, 197, 96, seed=seed).to(DEV)
        want = ops.forward(spec, x, packed, cand)
        rc, got = _call_noalloc(spec, x, packed, cand)
        _capi.check(rc)
        assert torch.equal(got, want)


def test_noalloc_forward_refuses_shapes_beyond_its_capacity():
    L = _capi.lib()
    cap = L.convnn_b200_noalloc_capacity()
    assert cap == 32 << 20
    cfg = ConvNNConfig(d_hidden=192, num_heads=1, K=9, magnitude_type="cosine")
    spec, packed = spec_of(cfg), pack(cfg, make_layer_weights(cfg, seed=5), torch.bfloat16)
    x = torch.zeros(256, 197, 192, device=DEV, dtype=torch.bfloat16)      # needs ~120 MB of intermediates
    assert ops.workspace_bytes(spec, 256, 197, 197, torch.bfloat16) > cap
    rc, _ = _call_noalloc(spec, x, packed)
    assert rc == _capi.E_WORKSPACE
    assert "built-in workspace" in L.convnn_b200_last_error().decode()
