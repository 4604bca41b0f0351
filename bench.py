"""Benchmark of the ConvNN-Attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1 and per GPU at N>1, weak scaling): ViT-Tiny with ConvNN-Attention layers,
bfloat16 inference, batch 256 x 3 x 224 x 224 synthetic N(0,1) images, patch 16 -> 197
tokens, d=192, 12 layers, 1000 classes, K=9, cosine similarity, sampling 'all', depthwise
conv, random-init weights.  A step is one forward of the whole model on one batch per GPU.

A step is `inner_iters` batches per GPU (stated in `config`), chosen so that the timed region
of `steps` steps lasts about a second; `ms_per_step` x `steps` is the timed region.

One JSON line on stdout (rank 0).  `value` = images/s with inputs resident in HBM, timed
with CUDA events on the launching stream, max over ranks.  `e2e` = the same through the
public module call with HOST (pinned, bfloat16) images: the host->device copy and the
device->host read of the logits are inside the timed region.  `roofline` describes the layer
kernel with the largest share of device time, timed with CUDA events around the stage calls.
At N=1 the line also carries `configs` (whole-model images/s of the baseline's ViT-Small and
ViT-Base BranchAttention configurations) and `layer_sweep` (the standalone layer on 4096 and
16384 tokens of 768 channels: tokens/s, similarity TFLOP/s and gather/conv GB/s against the
measured peaks, each case with its own clock record); at N>1 a `strong` record (global batch
256 split over the ranks).
`cpu_baseline` / `--impl reference` time the model on the host cores: the reference's own
vit.ViT when a checkout is reachable ($CONVNN_REF_PATH, ../reference, baseline/_ref), else
the CPU oracle port of the same model (the reference is eager PyTorch; its checkout does not
travel to the GPU box).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOAD = dict(layer="ConvNNAttention", img_size=(3, 224, 224), patch_size=16, num_layers=12, num_heads=1,
                d_hidden=192, d_mlp=768, num_classes=1000, K=9, magnitude_type="cosine", sampling_type="all",
                convolution_type="depthwise", softmax_topk_val=True, dropout=0.0, attention_dropout=0.0)
BATCH_PER_GPU = 256
METRIC, UNIT = "ConvNN-ViT images/sec", "images/s"
WORKLOAD_NAME = ("cfg-2 ViT-Tiny ConvNNAttention inference 224x224 patch16 (197 tokens) d=192 heads=1 12 layers "
                 "1000 classes K=9 cosine/all/depthwise")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            m = json.load(f)
        return dict(hbm=m["hbm_gbs"], tf_burst=m["bf16_tflops"], tf_sustained=m["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference model on the host cores
# ---------------------------------------------------------------------------------------

def find_reference_checkout():
    for p in (os.environ.get("CONVNN_REF_PATH"), os.path.join(os.path.dirname(ROOT), "reference"),
              os.path.join(ROOT, "baseline", "_ref")):
        if p and os.path.exists(os.path.join(p, "vit.py")) and os.path.exists(os.path.join(p, "layers.py")):
            return p
    return None


def cpu_model_throughput(batch: int, steps: int, warmup: int, budget_s: float = 30.0):
    """images/s of the model on the host cores (fp32, all host threads), ``batch`` images per
    step: the reference's own vit.ViT when its checkout is reachable, else the oracle port.
    -> (images/s, seconds per step, threads, steps done, kind)."""
    from oracle.vit_oracle import ViTConfig, make_images, make_vit_weights, vit_forward
    cfg = ViTConfig(**WORKLOAD)
    sd = make_vit_weights(cfg, seed=1)
    img = make_images(batch, cfg, seed=2)
    cores = torch.get_num_threads()
    kind, fwd = "port", (lambda: vit_forward(img, sd, cfg))
    ref = find_reference_checkout()
    if ref is not None:
        try:
            import types
            from oracle.pin_against_reference import load_reference
            _, ref_vit = load_reference(ref)
            a = {f: getattr(cfg, f) for f in cfg.__dataclass_fields__}
            a.update(device="cpu", img_size=tuple(cfg.img_size))
            model = ref_vit.ViT(types.SimpleNamespace(**a)).eval()
            model.load_state_dict(sd, strict=True)
            kind, fwd = "reference", (lambda: model(img))
        except Exception as e:  # noqa: BLE001
            print(f"reference checkout at {ref} could not be used ({type(e).__name__}: {e}); timing the port",
                  file=sys.stderr)
    with torch.no_grad():
        for _ in range(warmup):
            fwd()
        times = []
        t_start = time.perf_counter()
        for _ in range(steps):
            t0 = time.perf_counter()
            fwd()
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - t_start > budget_s:
                break
    per = sum(times) / len(times)
    return batch / per, per, cores, len(times), kind


def inner_iters_for(steps: int) -> int:
    """Batches per step such that `steps` steps last about a second at ~1.6-2 ms per batch."""
    return max(1, -(-640 // max(1, steps)))


def config_record(world: int, inner: int, lanes: int = 2) -> dict:
    return {"workload": WORKLOAD_NAME, "batch_per_gpu": BATCH_PER_GPU, "global_batch": BATCH_PER_GPU * world,
            "inner_iters": inner, "images_per_step": BATCH_PER_GPU * world * inner,
            "parallelism": f"batch-shard x{world}",
            "l2": f"{3 if lanes == 1 else 2 * lanes} distinct resident input batches (77 MB each) rotate, larger than L2",
            "launch": "cuda_graph (one per resident input batch; a replay reads its batch in place)",
            "batches_in_flight": f"{lanes} (convnn_b200.ForwardLanes: a CUDA graph holds the forwards of that many batches "
                                 "as parallel branches)",
            "e2e_host_images": "uint8 (normalised on the GPU); `e2e_bf16_images`: pre-normalised bfloat16",
            "collective": "none (one rank)" if world == 1 else
                          "one NCCL all_gather_into_tensor of the logits per group of batches (default: per step), "
                          "on a side stream under the following forwards"}


def run_reference_arm(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    batch = 32
    warm = max(1, min(args.warmup, 3))
    v, per, cores, done, kind = cpu_model_throughput(batch, args.steps, warm, budget_s=150.0)
    what = "the reference's own vit.ViT" if kind == "reference" else "the CPU oracle port of the model"
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": warm, "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_record(int(os.environ.get("WORLD_SIZE", "1")), args.inner_iters, max(1, args.lanes)),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{done} forwards of {batch} images (a sample of the workload's 256-image batches), "
                                   f"fp32, torch CPU, {what}"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

class ClockSampler:
    """SM clock / throttle-reason samples taken while a timed region runs: an NVML polling thread
    (about one sample per 2 ms; the main thread sits in cudaStreamSynchronize meanwhile), or an
    nvidia-smi subprocess at 20 ms where NVML cannot be loaded.  Read-only."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    _nvml = None

    @classmethod
    def _handle(cls, dev_index: int):
        import pynvml
        if cls._nvml is None:
            pynvml.nvmlInit()
            cls._nvml = pynvml
        props = torch.cuda.get_device_properties(dev_index)
        bus = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        return pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())

    def __init__(self, index: int, period_s: float = 0.002):
        import threading
        self.rows, self.p, self.f, self.thread = [], None, None, None
        self.stop_flag = threading.Event()
        try:
            h = self._handle(index)
            nv = self._nvml
            self.smax = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

            def poll():
                while not self.stop_flag.is_set():
                    try:
                        mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                        r = int(reasons_fn(h))
                        self.rows.append((mhz, {n for n, b in bits.items() if r & b}))
                    except Exception:  # noqa: BLE001
                        pass
                    time.sleep(period_s)
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            self.how = "nvml thread"
        except Exception:  # noqa: BLE001
            self.thread = None
            self.how = "nvidia-smi -lms 20"
            self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            try:
                self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                           "-lms", "20", "-i", str(index)], stdout=self.f, stderr=subprocess.DEVNULL)
            except OSError:
                self.p = None

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = sorted(r[0] for r in self.rows)
            reasons = set().union(*[r[1] for r in self.rows]) if self.rows else set()
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                    "sm_max_mhz": self.smax, "samples": len(sm), "reasons": sorted(reasons), "how": self.how}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        rows = [r.strip().split(", ") for r in self.f.read().strip().splitlines() if r.strip()]
        self.f.close()
        os.unlink(self.f.name)
        sm, smax, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                smax = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None, "sm_max_mhz": smax,
                "samples": len(sm), "reasons": sorted(reasons), "how": self.how}


class StageTimer:
    """Collects CUDA events between the stage calls of every ConvNN layer."""

    def __init__(self):
        self.marks = []

    def __call__(self, label):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.marks.append((label, e))

    def totals(self):
        tot, cnt = {}, {}
        for (l0, e0), (l1, e1) in zip(self.marks, self.marks[1:]):
            if l1 == "begin":
                continue
            tot[l1] = tot.get(l1, 0.0) + e0.elapsed_time(e1)
            cnt[l1] = cnt.get(l1, 0) + 1
        return tot, cnt


def stage_profile(model, B, cfg, dev, sets=4, reps=5):
    """Device time per launch of each stage of one ConvNN layer at the bench shape.

    Each stage is captured in a CUDA graph that runs it once on each of ``sets`` distinct
    buffer sets (together larger than L2, so no launch finds its inputs cached by the
    previous one) and the graph is timed with CUDA events on the launching stream."""
    import convnn_b200
    from convnn_b200 import ops
    layer = next(m for m in model.modules() if isinstance(m, convnn_b200.MultiHeadConvNNAttention))
    spec = layer._spec()
    w_qkv, w_conv, w_pw, w_o = layer.packed_weights(torch.bfloat16, dev)
    T, D = cfg.seq_len, cfg.d_hidden
    g = torch.Generator(device="cpu").manual_seed(7)
    data = []
    for _ in range(sets):
        x = torch.randn(B, T, D, generator=g).to(dev, torch.bfloat16)
        q, k, v, qs, ks = ops.qkv_proj(spec, x, w_qkv)
        idx, val = ops.sim_topk(spec, q, k, qs, ks)
        o = ops.gather_conv(spec, v, idx, val, w_conv, w_pw)
        data.append(dict(x=x, q=q, k=k, v=v, qs=qs, ks=ks, idx=idx, val=val, o=o))
    fns = {
        "qkv_proj": lambda d: ops.qkv_proj(spec, d["x"], w_qkv),
        "sim_topk": lambda d: ops.sim_topk(spec, d["q"], d["k"], d["qs"], d["ks"]),
        "gather_conv": lambda d: ops.gather_conv(spec, d["v"], d["idx"], d["val"], w_conv, w_pw),
        "out_proj": lambda d: ops.out_proj(spec, d["o"], w_o, residual=d["x"]),
    }
    # the encoder's MLP block as the model runs it: one kernel where the fused form is built
    blk = model.transformer_encoder[0]
    n2, fc1, fc2 = blk.norm2, blk.mlp[0], blk.mlp[3]
    if blk.fold_layernorm and blk.fuse_mlp and ops.prenorm_mlp_supported(fc1.in_features, fc1.out_features, 2):
        wf, wx = ops.fold_layernorm(fc1.weight, fc1.bias, n2.weight, n2.bias)
        for d in data:
            d["mom"] = ops.linear_moments(d["o"], w_o, None, d["x"])[1]      # two planes, as the output projection emits
        fns["mlp_block"] = lambda d: ops.prenorm_mlp(d["x"], d["mom"], n2.eps, wf, wx, fc2.weight, fc2.bias,
                                                     want_moments=True)
    out = {}
    torch.cuda.synchronize()
    for name, fn in fns.items():
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = [fn(d) for d in data]
        for _ in range(2):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / (reps * sets)
        del keep, graph
    return out


def run_forward_of(args) -> int:
    """One eager forward (after a warm-up forward) of a whole model of the baseline's configurations,
    for launch lists: python bench.py --forward-of cfg-4 [--stage-batch 32].  Prints the number of
    library kernels the forward launched."""
    import convnn_b200
    from convnn_b200 import _capi
    from oracle.vit_oracle import ViTConfig, make_vit_weights
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    table = {"cfg-2": (BATCH_PER_GPU, WORKLOAD)}
    for name, (B, kw) in OTHER_CONFIGS.items():
        table[name.split()[0]] = (B, kw)
    B, kw = table[args.forward_of]
    B = args.stage_batch if args.stage_batch != BATCH_PER_GPU else B
    cfg = ViTConfig(**kw)
    model = convnn_b200.ViT(convnn_b200.make_args(**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__},
                                                  device=dev)).eval()
    model.load_state_dict(make_vit_weights(cfg, seed=1), strict=True)
    model = model.to(dev, torch.bfloat16)
    if cfg.sampling_type == "random":
        model.set_candidates(torch.randperm(cfg.seq_len, generator=torch.Generator().manual_seed(17))
                             [: cfg.num_samples].to(dev))
    x = torch.randn(B, 3, 224, 224, device=dev).to(torch.bfloat16)
    lib = _capi.lib()
    with torch.no_grad():
        model(x)
        torch.cuda.synchronize()
        n0 = lib.convnn_b200_launch_count()
        model(x)
        torch.cuda.synchronize()
    print(json.dumps({"forward_of": args.forward_of, "batch": B, "library_launches_per_forward":
                      int(lib.convnn_b200_launch_count() - n0), "device_status": _capi.device_status()}))
    return 0


def run_single_stage(args) -> int:
    """Launch one stage of the layer a few times at the bench shape (for ncu captures and
    quick timing): python bench.py --stage sim_topk [--stage-batch 64] [--stage-iters 3]."""
    import convnn_b200
    from convnn_b200 import ops
    from oracle.vit_oracle import ViTConfig
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = ViTConfig(**WORKLOAD)
    B, T, D = args.stage_batch, cfg.seq_len, cfg.d_hidden
    layer = convnn_b200.MultiHeadConvNNAttention(D, cfg.num_heads, 0.0, cfg.K, cfg.sampling_type, cfg.num_samples,
                                                 cfg.sample_padding, cfg.magnitude_type).eval().to(dev, torch.bfloat16)
    spec = layer._spec()
    w_qkv, w_conv, w_pw, w_o = layer.packed_weights(torch.bfloat16, dev)
    x = torch.randn(B, T, D, device=dev).to(torch.bfloat16)
    q, k, v, qs, ks = ops.qkv_proj(spec, x, w_qkv)
    idx, val = ops.sim_topk(spec, q, k, qs, ks)
    o = ops.gather_conv(spec, v, idx, val, w_conv, w_pw)
    F = cfg.d_mlp
    h = torch.randn(B, T, F, device=dev).to(torch.bfloat16)
    W1 = (torch.randn(F, D, device=dev) / 14).to(torch.bfloat16)
    W2 = (torch.randn(D, F, device=dev) / 28).to(torch.bfloat16)
    b1, b2 = torch.randn(F, device=dev).to(torch.bfloat16), torch.randn(D, device=dev).to(torch.bfloat16)
    gam, bet = torch.ones(D, device=dev).to(torch.bfloat16), torch.zeros(D, device=dev).to(torch.bfloat16)
    fns = {"qkv_proj": lambda: ops.qkv_proj(spec, x, w_qkv),
           "sim_topk": lambda: ops.sim_topk(spec, q, k, qs, ks),
           "gather_conv": lambda: ops.gather_conv(spec, v, idx, val, w_conv, w_pw),
           "out_proj": lambda: ops.out_proj(spec, o, w_o),
           # the encoder's kernels around the layer (same GEMM kernel, other epilogues)
           "out_proj_skip": lambda: ops.out_proj(spec, o, w_o, residual=x),
           "mlp0": lambda: ops.linear(x, W1, b1, gelu=True),
           "mlp3": lambda: ops.linear(h, W2, b2, residual=x),
           "layernorm": lambda: ops.layernorm(x, gam, bet)}
    if args.stage in ("mlp_fused", "mlp0_prenorm", "qkv_prenorm", "mlp3_moments"):
        # the kernels of the folded-LayerNorm encoder path
        mom = ops.row_moments(x)
        wf1, wx1 = ops.fold_layernorm(W1, b1, gam, bet)
        wfq, wxq = ops.fold_layernorm(w_qkv.view(-1, D), None, gam, bet)
        fns.update({"mlp_fused": lambda: ops.prenorm_mlp(x, mom, 1e-5, wf1, wx1, W2, b2, want_moments=True),
                    "mlp0_prenorm": lambda: ops.prenorm_linear(x, mom, 1e-5, wf1, wx1, gelu=True),
                    "qkv_prenorm": lambda: ops.prenorm_linear(x, mom, 1e-5, wfq, wxq),
                    "mlp3_moments": lambda: ops.linear_moments(h, W2, b2, x)})
    if args.stage in ("attention", "conv1d_attention"):
        # the other halves of the ViT-Base branching wrappers (cfg-4): 384 channels, 12 heads
        Dh, Hh = 384, 12
        xa = torch.randn(B, T, 2 * Dh, device=dev).to(torch.bfloat16)[:, :, Dh:]
        if args.stage == "attention":
            m = convnn_b200.MultiHeadAttention(Dh, Hh, 0.0).eval().to(dev, torch.bfloat16)
        else:
            m = convnn_b200.MultiHeadConv1dAttention(Dh, Hh, 9).eval().to(dev, torch.bfloat16)
        with torch.no_grad():
            m(xa)
        fns[args.stage] = lambda: m(xa)
    fn = fns[args.stage]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.stage_iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"stage": args.stage, "batch": B, "iters": args.stage_iters,
                      "ms_per_call_incl_host": e0.elapsed_time(e1) / args.stage_iters}))
    return 0


def timed_loop(fn, min_reps: int, min_ms: float):
    """Average device time of fn() in ms: CUDA events on the launching stream around a loop of at
    least `min_reps` calls lasting at least `min_ms` (sized from a short trial)."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    est = max(e0.elapsed_time(e1) / 3, 1e-3)
    reps = max(min_reps, int(min_ms / est) + 1)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, reps


def layer_sweep(dev, sweep_n, min_reps=20, min_ms=120.0):
    """Standalone ConvNN layer on long sequences (cfg-5 of the baseline): x ~ N(0,1) of shape
    8 x N x 768 bf16, cosine, depthwise, sampling 'all' and 'spatial' (N/4 candidates), K in {9, 25}.
    One record per case: per-stage device time (>= 20 launches and >= 120 ms each, inputs of a
    few hundred MB, larger than L2), tokens/s, roofline fractions and the clocks sampled meanwhile."""
    import convnn_b200
    from convnn_b200 import ops
    pk = peaks()
    B, D = 8, 768
    out = []
    for N in sweep_n:
        for K in (9, 25):
            for sampling in ("all", "spatial"):
                S = N if sampling == "all" else N // 4
                layer = convnn_b200.MultiHeadConvNNAttention(D, 1, 0.0, K, sampling, S if sampling != "all" else -1,
                                                             0, "cosine", seq_length=N).eval().to(dev, torch.bfloat16)
                spec = layer._spec()
                w_qkv, w_conv, w_pw, w_o = layer.packed_weights(torch.bfloat16, dev)
                cand = layer.candidates(N, dev)
                # distinct buffer sets visited in turn, together larger than L2 (one set is 4 x 50 MB at
                # N=4096, 4 x 201 MB at N=16384); each stage is captured in a CUDA graph that runs it once
                # per set, so back-to-back launches carry no host time and find nothing cached
                sets = 1 if N >= 16384 else 3
                data = []
                for _ in range(sets):
                    x = torch.randn(B, N, D, device=dev).to(torch.bfloat16)
                    q, k, v, qs, ks = ops.qkv_proj(spec, x, w_qkv, cand)
                    idx, val = ops.sim_topk(spec, q, k, qs, ks, cand)
                    o = ops.gather_conv(spec, v, idx, val, w_conv, w_pw, S=S)
                    data.append(dict(x=x, q=q, k=k, v=v, qs=qs, ks=ks, idx=idx, val=val, o=o))
                fns = {"qkv_proj": lambda d: ops.qkv_proj(spec, d["x"], w_qkv, cand),
                       "sim_topk": lambda d: ops.sim_topk(spec, d["q"], d["k"], d["qs"], d["ks"], cand),
                       "gather_conv": lambda d: ops.gather_conv(spec, d["v"], d["idx"], d["val"], w_conv, w_pw, S=S),
                       "out_proj": lambda d: ops.out_proj(spec, d["o"], w_o, S=S)}
                torch.cuda.synchronize()
                sampler = ClockSampler(dev.index or 0)
                times, reps = {}, {}
                for name, fn in fns.items():
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        keep = [fn(d) for d in data]
                    ms, n = timed_loop(graph.replay, -(-min_reps // sets), min_ms)
                    times[name], reps[name] = ms / sets, n * sets
                    del keep, graph
                clocks = sampler.stop()
                work = algorithmic_work(B, N, S, D, 1, K)
                total = sum(times.values())
                sim_tf = work["sim_topk"]["flops"] / times["sim_topk"] / 1e9
                gc_gbs = work["gather_conv"]["bytes"] / times["gather_conv"] / 1e6
                out.append({
                    "case": f"N={N} K={K} {sampling} S={S}", "tokens_per_s": B * N / (total / 1e3),
                    "ms": {k2: round(v2, 4) for k2, v2 in times.items()}, "launches_timed": reps,
                    "sim_topk_TFLOPs": sim_tf, "sim_topk_frac_of_tensor_peak_burst": sim_tf / pk["tf_burst"],
                    "sim_topk_frac_of_tensor_peak_sustained": sim_tf / pk["tf_sustained"],
                    "gather_conv_GBps": gc_gbs, "gather_conv_frac_of_hbm_peak": gc_gbs / pk["hbm"],
                    "peak_source": pk["source"], "clocks": clocks})
                del layer, data, x, q, k, v, idx, val, o, fns
                torch.cuda.empty_cache()
    return out


def run_layer_sweep(args) -> int:
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    with torch.no_grad():
        for rec in layer_sweep(dev, args.sweep_n):
            print(json.dumps(rec))
    return 0


# Other configurations of the baseline, whole model, bfloat16 (cfg-3: ViT-Small, euclidean, 64 random
# candidates shared by all layers, separable conv; cfg-4: ViT-Base BranchAttention, 12 heads, standard conv).
OTHER_CONFIGS = {
    "cfg-3 ViT-Small ConvNNAttention euclidean/random-64/depthwise-separable B=256": (256, dict(
        layer="ConvNNAttention", d_hidden=384, d_mlp=1536, num_heads=1, num_layers=12, magnitude_type="euclidean",
        sampling_type="random", num_samples=64, convolution_type="depthwise-separable")),
    "cfg-4 ViT-Base BranchAttention 12 heads cosine/all/standard B=128": (128, dict(
        layer="BranchAttention", d_hidden=768, d_mlp=3072, num_heads=12, num_layers=12, magnitude_type="cosine",
        convolution_type="standard", branch_ratio=0.5)),
}


def other_configs(dev, min_ms=400.0):
    """Whole-model images/s of the baseline's other ViT configurations (device-resident inputs, two
    distinct input batches alternating, CUDA graph, >= 10 forwards and >= 400 ms each)."""
    import convnn_b200
    from oracle.vit_oracle import ViTConfig, make_vit_weights  # seeded weights only (not on the timed path)
    out = {}
    for name, (B, kw) in OTHER_CONFIGS.items():
        cfg = ViTConfig(**kw)
        model = convnn_b200.ViT(convnn_b200.make_args(**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__},
                                                      device=dev)).eval()
        model.load_state_dict(make_vit_weights(cfg, seed=1), strict=True)
        model = model.to(dev, torch.bfloat16)
        if cfg.sampling_type == "random":
            model.set_candidates(torch.randperm(cfg.seq_len, generator=torch.Generator().manual_seed(17))
                                 [: cfg.num_samples].to(dev))
        xs = [torch.randn(B, 3, 224, 224, device=dev).to(torch.bfloat16) for _ in range(4)]
        fl = convnn_b200.ForwardLanes(model, xs, lanes=2)          # two forwards per graph, inputs read in place
        i = [0]

        def fwd():
            fl.replay(i[0] & 1)
            i[0] += 1
        sampler = ClockSampler(dev.index or 0)
        ms, reps = timed_loop(fwd, 10, min_ms)
        out[name] = {"images_per_s": 2 * B / (ms / 1e3), "ms_per_forward": ms / 2, "batch": B, "batches_in_flight": 2,
                     "forwards_timed": 2 * reps, "dtype": "bf16", "clocks": sampler.stop()}
        del fl
        del model, xs
        torch.cuda.empty_cache()
    return out


# dram__bytes_read + dram__bytes_write of one launch of each stage at the bench shape, from the
# ncu captures summarised under profiles/ (outputs that are still in L2 when the kernel ends are
# not in these figures, which is why they sit below the algorithmic bytes).
NCU_TRAFFIC_BYTES = {"qkv_proj": 19.69e6 + 10.28e6, "sim_topk": 39.2e6 + 0.009e6, "gather_conv": 23.04e6,
                     "out_proj": 19.5e6, "mlp_block": 20.47e6}


def algorithmic_work(B, T, S, D, H, K, DM=0, elt=2):
    """Compulsory bytes / flops per launch of each stage (one layer call)."""
    idxval = 8 * B * H * T * K
    return {
        "qkv_proj": dict(bytes=elt * (B * T * D + 3 * D * D + B * (2 * T + S) * D) + 4 * B * H * (T + S),
                         flops=2 * B * (2 * T + S) * D * D),
        "sim_topk": dict(bytes=elt * (B * T * D + B * S * D) + idxval + 4 * B * H * (T + S), flops=2 * B * T * S * D),
        "gather_conv": dict(bytes=elt * (2 * B * T * D + K * D) + idxval, flops=2 * B * T * D * K),
        # (with the skip connection read: one more activation-sized tensor)
        "out_proj": dict(bytes=elt * (3 * B * T * D + D * D), flops=2 * B * T * D * D),
        # norm2 + mlp.0 + GELU + mlp.3 + skip in one kernel: x in, x out, both weights, moments in (2 planes) / out (4)
        "mlp_block": dict(bytes=elt * (2 * B * T * D + 2 * D * DM) + 8 * B * T * 6, flops=4 * B * T * D * DM),
    }


def run_ours(args) -> int:
    import torch.distributed as dist
    import convnn_b200
    from convnn_b200 import _capi
    from oracle.vit_oracle import ViTConfig, make_vit_weights  # seeded weights only (not on the timed path)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the ConvNN path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from convnn_b200.sharded import bind_host_to_device
    numa_bound = bind_host_to_device(dev) if world > 1 else False   # before any pinned allocation
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _capi.lib()
    inner = args.inner_iters

    cfg = ViTConfig(**WORKLOAD)
    margs = convnn_b200.make_args(**WORKLOAD, device=dev)
    model = convnn_b200.ViT(margs).eval()
    model.load_state_dict(make_vit_weights(cfg, seed=1), strict=True)
    model = model.to(dev, torch.bfloat16)
    B = BATCH_PER_GPU
    classes = WORKLOAD["num_classes"]
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    LANES = max(1, args.lanes)
    inner += (-inner) % LANES               # whole groups of LANES batches per step (recorded in `config`)
    NBUF = 3 if LANES == 1 else 2 * LANES   # >= 3 x 77 MB of distinct resident inputs > 126 MB L2; whole groups of LANES
    host = [torch.randn(B, 3, 224, 224, generator=g).to(torch.bfloat16).pin_memory() for _ in range(NBUF)]
    resident = [h.to(dev) for h in host]
    total = B * world

    # One CUDA graph of the whole forward per resident input batch (ctypes launches on the capturing
    # stream are captured): a replay reads its batches where they lie, no staging copy in between.  A graph
    # holds the forwards of LANES batches as parallel branches (convnn_b200.ForwardLanes): the second
    # batch's kernels fill the tails of the first one's.
    with torch.no_grad():
        model(resident[0])                # builds the packed / folded weights (launches of their own, once)
        torch.cuda.synchronize()
        n_cap = lib.convnn_b200_launch_count()
        model(resident[0])
        torch.cuda.synchronize()
        per_forward = lib.convnn_b200_launch_count() - n_cap
        fl = convnn_b200.ForwardLanes(model, resident, lanes=LANES)
    from convnn_b200.sharded import LogitsGather
    per_flush = args.gather_every if args.gather_every > 0 else inner
    gather = LogitsGather(world, per_flush, B, classes, torch.bfloat16, dev)    # default: one collective per step


    def group_step(i):
        """Batches i .. i + LANES - 1 (one graph replay)."""
        for y in fl.replay((i // LANES) % fl.n_groups):
            gather.add(y)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        # ---- device-resident timing -------------------------------------------------------
        n = 0
        for _ in range(args.warmup):
            for _ in range(inner // LANES):
                group_step(n)
                n += LANES
        gather.drain()
        barrier()
        sampler = ClockSampler(local) if rank == 0 else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            for _ in range(inner // LANES):
                group_step(n)
                n += LANES
        gather.drain()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if sampler else None

        # ---- end to end: pinned host images in, logits out ------------------------------------
        copy_stream = torch.cuda.Stream(dev)
        d2h_stream = torch.cuda.Stream(dev)
        out_host = torch.empty(world * inner * B, classes, dtype=torch.bfloat16).pin_memory()   # one step's logits

        def e2e_timed(host_batches):
            """ms for args.steps x inner batches from pinned host batches: two staging buffers per lane on
            the device, each with its own graph of the forward, filled in turn by the copy stream."""
            NS = 2 * LANES
            staging = [host_batches[k % len(host_batches)].to(dev) for k in range(NS)]
            lf = convnn_b200.ForwardLanes(model, staging, lanes=LANES)
            ready = [torch.cuda.Event() for _ in range(NS)]

            def run(n_batches):
                cur = torch.cuda.current_stream()
                copy_stream.wait_stream(cur)
                for i in range(0, n_batches, LANES):
                    gi = (i // LANES) % lf.n_groups
                    with torch.cuda.stream(copy_stream):
                        copy_stream.wait_event(lf.done[gi])    # the forwards that last read these buffers
                        for j, k in enumerate(lf.groups[gi]):
                            staging[k].copy_(host_batches[(i + j) % len(host_batches)], non_blocking=True)
                            ready[k].record(copy_stream)
                    for y in lf.replay(gi, after=[ready[k] for k in lf.groups[gi]]):
                        group = gather.add(y)
                        if group is not None:
                            # a step's logits are complete (and gathered): read them back on a stream of their
                            # own (behind the input copies they would hold up the next batch)
                            logits, done = group
                            with torch.cuda.stream(d2h_stream):
                                d2h_stream.wait_event(done)
                                out_host[: logits.numel() // classes].view(logits.shape).copy_(logits, non_blocking=True)
                gather.drain()
                cur.wait_stream(copy_stream)
                cur.wait_stream(d2h_stream)

            run(max(2, args.warmup) * LANES)
            barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            run(args.steps * inner)
            f1.record()
            barrier()
            return f0.elapsed_time(f1)

        ms_e2e = e2e_timed(host)

        # ---- the same with 8-bit host images (what an image decoder hands over), ToTensor + Normalize inside
        # the patch unfold: more work in the timed region, half the bytes of bfloat16 images (a quarter of
        # float32) over PCIe.  This is the `e2e` record; the bfloat16 figure is kept beside it.
        host_u8 = [torch.randint(0, 256, (B, 3, 224, 224), generator=g, dtype=torch.uint8).pin_memory() for _ in range(NBUF)]
        ms_e2e_u8 = e2e_timed(host_u8)

        # ---- strong scaling: the 256-image batch of the baseline split over the ranks ----------
        ms_strong = 0.0
        if world > 1:
            Bs = BATCH_PER_GPU // world
            xs = [r[:Bs].contiguous() for r in resident]
            s_fwd = convnn_b200.ForwardLanes(model, xs, lanes=LANES)
            s_gather = LogitsGather(world, per_flush, Bs, classes, torch.bfloat16, dev)

            def strong_step(i):
                for y in s_fwd.replay((i // LANES) % s_fwd.n_groups):
                    s_gather.add(y)
            for i in range(0, 12 * LANES, LANES):
                strong_step(i)
            s_gather.drain()
            barrier()
            n_strong = max(50, args.steps * inner)
            n_strong -= n_strong % LANES
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for i in range(0, n_strong, LANES):
                strong_step(i)
            s_gather.drain()
            g1.record()
            barrier()
            ms_strong = g0.elapsed_time(g1) / n_strong
            del s_fwd

        # ---- per-stage device time for the roofline ----------------------------------------
        stage_ms = stage_profile(model, B, cfg, dev)

    t = torch.tensor([ms, ms_e2e, ms_strong, ms_e2e_u8], dtype=torch.float64, device=dev)
    per_rank = [[float(v) for v in t]]
    if world > 1:
        every = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank = [[float(v) for v in r] for r in every]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_strong, ms_e2e_u8 = float(t[0]), float(t[1]), float(t[2]), float(t[3])

    if rank == 0:
        pk = peaks()
        T = cfg.seq_len
        work = algorithmic_work(B, T, T, cfg.d_hidden, cfg.num_heads, cfg.K, cfg.d_mlp)
        dom = max(stage_ms, key=stage_ms.get)
        per_launch_ms = stage_ms[dom]
        ridge = pk["tf_sustained"] * 1e3 / pk["hbm"]
        ai = work[dom]["flops"] / work[dom]["bytes"]
        if ai > ridge:
            # a kernel timed alone (a graph of four launches): the burst figure is its denominator
            bound, ach, peak, unit = "tensor", work[dom]["flops"] / per_launch_ms / 1e9, pk["tf_burst"], "TFLOP/s"
        else:
            bound, ach, peak, unit = "hbm", work[dom]["bytes"] / per_launch_ms / 1e6, pk["hbm"], "GB/s"
        stages = {k: {"ms_per_launch": stage_ms[k], "GBps": work[k]["bytes"] / stage_ms[k] / 1e6,
                      "TFLOPs": work[k]["flops"] / stage_ms[k] / 1e9,
                      "frac_of_hbm_peak": work[k]["bytes"] / stage_ms[k] / 1e6 / pk["hbm"]} for k in stage_ms}
        cpu = None
        if world == 1 and not args.no_cpu:
            torch.set_num_threads(max(1, os.cpu_count() or 1))
            cpu_v, cpu_per, cores, cpu_done, kind = cpu_model_throughput(32, 8, 1, budget_s=20.0)
            cpu = {"value": cpu_v, "unit": UNIT, "cores": cores, "kind": kind,
                   "sample": f"{cpu_done} forwards of 32 images (of the 256-image batch), fp32, torch CPU, "
                             + ("the reference's own vit.ViT" if kind == "reference" else "oracle port")}
        n_batches = args.steps * inner
        h2d = B * 3 * 224 * 224 * 2
        h2d_u8 = B * 3 * 224 * 224
        d2h = world * B * classes * 2            # per batch: the gathered logits of every rank
        line = {
            "metric": METRIC, "value": total * n_batches / (ms / 1e3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_record(world, inner, LANES),
            "ms_per_batch": ms / n_batches, "host_numa_bound": bool(numa_bound),
            "per_rank_ms_per_batch": {"device_resident": [r[0] / n_batches for r in per_rank],
                                      "e2e": [r[3] / n_batches for r in per_rank]},
            "e2e": {"value": total * n_batches / (ms_e2e_u8 / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d_u8 * inner,
                    "d2h_bytes_per_step": d2h * inner, "ms_per_step": ms_e2e_u8 / args.steps,
                    "host_images": "uint8, pinned (what an image decoder produces); ToTensor + Normalize run inside "
                                   "the patch unfold kernel, in the timed region",
                    "h2d_GBps_per_rank": h2d_u8 * n_batches / (ms_e2e_u8 / 1e3) / 1e9},
            "e2e_bf16_images": {"value": total * n_batches / (ms_e2e / 1e3), "unit": UNIT,
                                "h2d_bytes_per_step": h2d * inner, "d2h_bytes_per_step": d2h * inner,
                                "ms_per_step": ms_e2e / args.steps,
                                "h2d_GBps_per_rank": h2d * n_batches / (ms_e2e / 1e3) / 1e9,
                                "note": "host images already normalised and rounded to bfloat16 (twice the bytes; "
                                        "float32 host images would double them again); an extra record"},
            "gpu_launches": int(per_forward * n_batches),
            "roofline": {"bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(dom), "kernel": dom, "peak_source": pk["source"],
                         "ms_per_launch": per_launch_ms, "stages": stages},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        if world > 1:
            line["strong"] = {"global_batch": BATCH_PER_GPU, "batch_per_gpu": BATCH_PER_GPU // world,
                              "images_per_s": BATCH_PER_GPU / (ms_strong / 1e3), "ms_per_batch": ms_strong,
                              "note": "the baseline's 256-image batch split over the ranks, device-resident, "
                                      "max over ranks; `value` stays the weak-scaling figure"}

        if world == 1 and not args.no_extras:
            with torch.no_grad():
                del fl                                   # the graphs and their pools
                torch.cuda.empty_cache()
                line["configs"] = other_configs(dev)
                line["layer_sweep"] = layer_sweep(dev, [4096, 16384])
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--inner-iters", type=int, default=0,
                    help="batches per step (default: chosen so that the timed region lasts about a second)")
    ap.add_argument("--lanes", type=int, default=2,
                    help="batches in flight per GPU (CUDA streams with a graph set each); 1 = one after another")
    ap.add_argument("--gather-every", type=int, default=0,
                    help="batches per logits all-gather at N > 1 (default: one collective per step)")
    ap.add_argument("--no-extras", action="store_true", help="skip the cfg-3 / cfg-4 models and the layer sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--stage", choices=["qkv_proj", "sim_topk", "gather_conv", "out_proj", "out_proj_skip", "mlp0",
                                        "mlp3", "layernorm", "attention", "conv1d_attention", "mlp_fused",
                                        "mlp0_prenorm", "qkv_prenorm", "mlp3_moments"],
                    help="run only this stage of one layer (profiling aid)")
    ap.add_argument("--forward-of", choices=["cfg-2", "cfg-3", "cfg-4"],
                    help="one eager forward of that configuration's whole model (for launch lists)")
    ap.add_argument("--layer-sweep", action="store_true",
                    help="standalone layer on long sequences (8 x N x 768), per-stage time and roofline")
    ap.add_argument("--sweep-n", type=int, nargs="+", default=[1024, 4096, 16384])
    ap.add_argument("--stage-batch", type=int, default=BATCH_PER_GPU)
    ap.add_argument("--stage-iters", type=int, default=3)
    args = ap.parse_args()
    if args.forward_of:
        return run_forward_of(args)
    if args.stage:
        with torch.no_grad():
            return run_single_stage(args)
    if args.layer_sweep:
        return run_layer_sweep(args)
    args.warmup = max(args.warmup, 3)
    if args.inner_iters <= 0:
        args.inner_iters = inner_iters_for(args.steps)
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
