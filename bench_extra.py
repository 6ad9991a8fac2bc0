"""Extra benchmark workloads, reached through `python bench.py --workload varlen|decode`.

varlen (BASELINE config 3): packed KDA forward+backward, 65,536 tokens, H=16, Dk=Dv=128, seeded document
lengths ~ U[256, 8192], per-sequence initial states ~ N(0, 0.02), bf16 I/O.  With N GPUs the heads are
sharded (H/N per GPU, every GPU sees all sequences), no collective.
decode (BASELINE config 4): recurrent decode, batch 256, H=16, Dk=Dv=128, fp32 state ~ N(0, 0.02), one token
per step; the state (256 MiB) is read and rewritten every step.  With N GPUs the batch is sharded.
pointwise: the HBM-bound kernels either side of the KDA operator at a size that cannot sit in L2: short convolution
(W=4, SiLU) and gated RMSNorm, forward and backward, on 65,536 tokens x 2,048 channels (256 MiB bf16 per tensor).
Each kernel is timed alone with CUDA events; the figure is algorithmic bytes / time against the measured HBM peak.
Each prints one JSON line on rank 0 with the metric, the algorithmic roofline figure and the per-kernel times.
"""

from __future__ import annotations

import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
FLOP_PER_TOKEN_HEAD = 423040.0      # chunked KDA fwd+bwd, C=64, K=V=128 (triangular products at triangular cost)


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def _lengths(total, seed):
    gen = torch.Generator().manual_seed(seed)
    out, acc = [], 0
    while acc < total:
        n = int(torch.randint(256, 8193, (1,), generator=gen).item())
        n = min(n, total - acc)
        out.append(n)
        acc += n
    return out


def run_varlen(args, rank, world, local, dist):
    import experiment_swa_kda_b200 as m
    from experiment_swa_kda_b200 import _lib
    from bench import kda_kernel_flops
    dev = torch.device(f"cuda:{local}")
    total, H, D = args.tokens, 16, 128
    Hl = H // world                                     # heads of this rank
    lens = _lengths(total, 0)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)      # seeded, drawn on the device (same distributions)
    rn = lambda *sh: torch.randn(*sh, generator=gen, device=dev)
    unit = lambda t: t / t.norm(dim=-1, keepdim=True)
    bf = torch.bfloat16
    x = {
        "q": unit(rn(1, total, Hl, D)).to(bf), "k": unit(rn(1, total, Hl, D)).to(bf), "v": rn(1, total, Hl, D).to(bf),
        "g": (-torch.nn.functional.softplus(rn(1, total, Hl, D)) * 0.1).clamp(-5, 0).to(bf),
        "beta": torch.sigmoid(rn(1, total, Hl)).to(bf),
    }
    x = {n: t.requires_grad_(True) for n, t in x.items()}
    h0 = (rn(len(lens), Hl, D, D) * 0.02).requires_grad_(True)
    probe = rn(1, total, Hl, D).to(bf)

    def step():
        o, fs = m.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=h0, output_final_state=True, cu_seqlens=cu)
        return torch.autograd.grad(o, list(x.values()) + [h0], probe)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    l0 = _lib.launch_count()
    for a, b in ev:      # inputs (5 x 32 MiB per head-shard at N=1: 1.3 GB with panels) are far larger than L2
        a.record()
        step()
        b.record()
    barrier()
    launches = _lib.launch_count() - l0
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in ev)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    _lib.profile(True)
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize(dev)
    rep = _lib.profile_report()
    _lib.profile(False)
    if rank != 0:
        return None
    peaks, src = _peaks()
    nch = sum((n + 63) // 64 for n in lens) * Hl
    flops = kda_kernel_flops(D, D)
    tot = sum(v[1] for v in rep.values()) or 1.0
    kern = {}
    for name, (n, tms) in rep.items():
        row = {"launches_per_step": n / args.steps, "avg_us": tms / n * 1e3, "share": tms / tot}
        if name in flops:
            row["tflops"] = flops[name] * nch / (tms / n * 1e-3) / 1e12
            row["frac_of_bf16_peak"] = row["tflops"] / peaks["bf16_tflops"]
        kern[name] = row
    top = max(rep, key=lambda k: rep[k][1])
    line = {
        "metric": "kda_varlen_fwd_bwd_token_heads_per_s", "value": total * H / (ms * 1e-3), "unit": "token-heads/s",
        "tokens_per_s": total / (ms * 1e-3) if world == 1 else total / (ms * 1e-3), "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"config3 packed KDA fwd+bwd: {total} tokens, {len(lens)} sequences U[256,8192], H16 D128 chunk64, "
                               f"heads sharded {Hl}/GPU, initial states N(0,0.02)", "l2": "inputs larger than L2"},
        "tflops_algorithmic": FLOP_PER_TOKEN_HEAD * total * H / (ms * 1e-3) / 1e12,
        "gpu_launches": int(launches),
        "roofline": {"kernel": top, "bound": "tensor", "achieved": kern[top].get("tflops"), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": kern[top].get("frac_of_bf16_peak"), "traffic": None, "peak_source": src},
        "kernels": kern,
    }
    return line


def run_decode(args, rank, world, local, dist):
    from experiment_swa_kda_b200 import _lib
    lib = _lib.load()
    dev = torch.device(f"cuda:{local}")
    B, H, D = 256 // world, 16, 128
    n_steps = 1024
    gen = torch.Generator().manual_seed(7 + rank)
    bf = torch.bfloat16
    unit = lambda t: t / t.norm(dim=-1, keepdim=True)
    NI = 64           # distinct per-step inputs, cycled (1 MiB each at N=1; the 256 MiB state dominates the traffic)
    rn = lambda *sh: torch.randn(*sh, generator=gen)
    q = unit(rn(NI, B, H, D)).to(bf).to(dev)
    k = unit(rn(NI, B, H, D)).to(bf).to(dev)
    v = rn(NI, B, H, D).to(bf).to(dev)
    g = (-torch.nn.functional.softplus(rn(NI, B, H, D)) * 0.1).clamp(-5, 0).to(bf).to(dev)
    beta = torch.sigmoid(rn(NI, B, H)).to(bf).to(dev)
    state = (rn(B, H, D, D) * 0.02).to(dev)
    o = torch.empty(NI, B, H, D, dtype=bf, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    p = lambda t: t.data_ptr()

    def steps(stream):
        # one library call per NI steps: the per-token launches are issued from C, the state is updated in place
        rc = lib.kda_decode_steps(NI, B, H, D, D, 1, 1, 1, D ** -0.5, p(q), p(k), p(v), p(g), p(beta), p(state), p(o), stream)
        if rc:
            raise RuntimeError(f"kda_decode_steps failed: {rc}")

    graph = None
    if not getattr(args, "no_graph", False):
        # the NI-step call captured once and replayed, as a serving loop with fixed buffers would do: the launches of
        # a replayed graph follow each other more closely than launches issued one by one
        steps(st)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            steps(torch.cuda.current_stream(dev).cuda_stream)

    def run(n):
        for _ in range(n // NI):
            if graph is not None:
                graph.replay()
            else:
                steps(st)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    run(64)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    run(n_steps)
    b.record()
    barrier()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / n_steps
    if rank != 0:
        return None
    peaks, src = _peaks()
    Bt = B * world
    bytes_step = 2 * Bt * H * D * D * 4 + Bt * H * (3 * D + D) * 2 + Bt * H * 2 + Bt * H * D * 2
    gbs = bytes_step / (ms * 1e-3) / 1e9
    line = {
        "metric": "kda_decode_state_GBps", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": n_steps, "warmup": 64,
        "us_per_step": ms * 1e3, "tokens_per_s": Bt / (ms * 1e-3), "higher_is_better": True, "scaling": "strong",
        "dtype": "f32 state, bf16 activations", "data": "synthetic",
        "config": {"workload": f"config4 recurrent decode: batch {Bt} ({B}/GPU), H16, Dk=Dv=128, fp32 state read+written every step, "
                               f"{n_steps} steps in one timed region", "launch": "kda_decode_steps: 64 steps per library call, one kernel launch per step, state in place; " + ("the call captured in a CUDA graph and replayed" if graph is not None else "eager"), "l2": "state (256 MiB at N=1) larger than L2; at N=8 the 32 MiB "
                               "per-GPU state can sit in L2, so the figure is effective bandwidth"},
        "bytes_per_step": bytes_step,
        "roofline": {"kernel": "decode_kernel", "bound": "hbm", "achieved": gbs / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / world / peaks["hbm_gbs"], "traffic": None, "peak_source": src},
    }
    return line


def run_pointwise(args, rank, world, local, dist):
    from experiment_swa_kda_b200 import ops
    dev = torch.device(f"cuda:{local}")
    T, C, D, W = 65536, 2048, 128, 4
    bf = torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(11 + rank)
    rnd = lambda *sh: torch.randn(*sh, generator=gen, device=dev, dtype=torch.float32).to(bf)
    x, dy = rnd(1, T, C), rnd(1, T, C)
    w = ((torch.rand(C, W, generator=gen, device=dev) * 2 - 1) * (3 ** 0.5) * C ** -0.5)
    xr, gate, dyr = x.view(T * C // D, D), rnd(T * C // D, D), dy.view(T * C // D, D)
    nw = torch.ones(D, device=dev)
    _, inv = ops.rmsnorm_gate_fwd(xr, gate, nw, 1e-6)
    n = T * C * 2                                       # bytes of one bf16 tensor
    cases = {
        "conv_fwd": (lambda: ops.conv_fwd(x, w, None, False, True), 2 * n),
        "conv_bwd": (lambda: ops.conv_bwd(x, w, None, dy, None, True), 3 * n),
        "rmsnorm_gate_fwd": (lambda: ops.rmsnorm_gate_fwd(xr, gate, nw, 1e-6), 3 * n),
        "rmsnorm_gate_bwd": (lambda: ops.rmsnorm_gate_bwd(xr, gate, nw, inv, dyr), 5 * n),
    }
    peaks, src = _peaks()
    out = {}
    for name, (fn, nbytes) in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(max(args.steps, 5))]
        for a, b in evs:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize(dev)
        ts = sorted(a.elapsed_time(b) for a, b in evs)
        ms = ts[len(ts) // 2]
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"us": ms * 1e3, "algorithmic_bytes": nbytes, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]}
    if rank != 0:
        return None
    worst = min(out, key=lambda k: out[k]["frac_of_hbm_peak"])
    line = {
        "metric": "pointwise_hbm_GBps_min", "value": out[worst]["gbs"], "unit": "GB/s", "n_gpus": world, "steps": max(args.steps, 5),
        "warmup": 3, "higher_is_better": True, "scaling": "weak", "dtype": "bf16 I/O, f32 math", "data": "synthetic",
        "config": {"workload": f"short convolution (W=4, SiLU) and gated RMSNorm fwd/bwd on {T} tokens x {C} channels "
                               f"(256 MiB per tensor, larger than L2), each kernel timed alone, median",
                   "timing": "includes the weight-gradient partial reduction launch for the two backward calls"},
        "kernels": out,
        "roofline": {"kernel": worst, "bound": "hbm", "achieved": out[worst]["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": out[worst]["frac_of_hbm_peak"], "traffic": None, "peak_source": src},
    }
    return line


def run_prefill(args, rank, world, local, dist):
    """No-grad prefill of one layer's operator chain at the config-1 shape, two ways: the three convolutions as their own
    launch followed by the forward-only chunk forward, and the convolutions folded into the intra-chunk kernel
    (kda_chunk_fwd_conv: q, k, v never written).  Same inputs, identical outputs; CUDA-graph replay, L2 flushed between
    steps, median."""
    from experiment_swa_kda_b200 import ops, _lib
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import kda_oracle as O
    dev = torch.device(f"cuda:{local}")
    B, T, H, D = 2, 4096, 3, 128
    d = O.make_inputs(B, T, H, D, D, seed=3)
    g, beta = d["g"].bfloat16().to(dev), d["beta"].bfloat16().to(dev)
    gen = torch.Generator().manual_seed(5)
    xs = [torch.randn(B, T, H * D, generator=gen).bfloat16().to(dev) for _ in range(3)]
    ws = [((torch.rand(H * D, 4, generator=gen) * 2 - 1) * 0.3).to(dev) for _ in range(3)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sh4 = (B, T, H, D)

    def unfused():
        with torch.no_grad():
            q, k, v = ops.ConvMultiFunction.apply(True, 3, *xs, *ws)
        return ops.chunk_kda_fwd(q.view(sh4), k.view(sh4), v.view(sh4), g, beta, None, None, D ** -0.5, True, True, _lib.LANE_TC, forward_only=True)[:2]

    def fused():
        return ops.chunk_kda_conv_fwd(xs[0].view(sh4), xs[1].view(sh4), xs[2].view(sh4), *ws, g, beta, None, None, D ** -0.5, True, True)

    res, outs = {}, {}
    for name, fn in (("convolutions_then_forward", unfused), ("convolutions_in_forward_kernel", fused)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        l0 = _lib.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs[name] = fn()
        launches = _lib.launch_count() - l0
        times = []
        for _ in range(max(args.steps, 10)):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize(dev)
            times.append(a.elapsed_time(b) * 1e3)
        times.sort()
        res[name] = {"us": times[len(times) // 2], "launches": launches}
    same = all(torch.equal(a, b) for a, b in zip(outs["convolutions_then_forward"], outs["convolutions_in_forward_kernel"]))
    if rank != 0:
        return None
    return {"metric": "kda_prefill_us", "value": res["convolutions_in_forward_kernel"]["us"], "unit": "us", "n_gpus": world,
            "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "no-grad prefill, conv4+SiLU(q,k,v) -> chunked KDA forward with final state, B2 T4096 H3 D128"},
            "variants": res, "outputs_identical": bool(same)}


def run(args, rank, world, local):
    import torch.distributed as dist
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = {"varlen": run_varlen, "decode": run_decode, "pointwise": run_pointwise, "prefill": run_prefill}[args.workload](args, rank, world, local, dist)
    if line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sharded_summary(args, rank, world, local, dist):
    """BASELINE configs 3 (packed, heads sharded) and 4 (decode, batch sharded) at this world size, condensed for the
    main benchmark line: strong scaling, no data-path collective, max-over-ranks device time."""
    import copy
    a = copy.copy(args)
    a.steps, a.warmup = min(args.steps, 10), 3
    v = run_varlen(a, rank, world, local, dist)
    torch.cuda.empty_cache()
    d = run_decode(a, rank, world, local, dist)
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    intra = {k: round(r["avg_us"], 1) for k, r in v["kernels"].items()}
    return {
        "varlen": {"workload": v["config"]["workload"], "ms_per_step": v["ms_per_step"], "tokens_per_s": v["tokens_per_s"],
                   "token_heads_per_s": v["value"], "tflops_algorithmic": v["tflops_algorithmic"],
                   "frac_of_bf16_peak": v["tflops_algorithmic"] / world / _peaks()[0]["bf16_tflops"], "kernel_us": intra,
                   "scaling": "strong (16 heads / N per GPU)"},
        "decode": {"workload": d["config"]["workload"], "us_per_step": d["us_per_step"], "gbs_aggregate": d["value"],
                   "gbs_per_gpu": d["value"] / world, "frac_of_hbm_peak_per_gpu": d["roofline"]["frac"],
                   "launch": d["config"].get("launch"), "scaling": "strong (256 rows / N per GPU)",
                   "note": d["config"]["l2"]},
    }
