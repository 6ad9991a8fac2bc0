"""Benchmark of the KDA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload chain|varlen|decode]

A step is one pass of the hot path over one batch of seeded synthetic input.  Default
workload ("chain"): B=2, T=4096, H=3, Dk=Dv=128, bf16 I/O with float32 state/accumulation:
short causal conv (width 4, SiLU) on q/k/v -> chunked KDA forward+backward -> gated RMSNorm
(eps 1e-6), forward and backward through the whole chain.  With N > 1 (launched by
torch.distributed.run, one rank per GPU) every rank runs the same per-GPU batch (weak
scaling, no data-path collective); the time is the maximum over ranks.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "kda_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"

CHAIN = dict(B=2, T=4096, H=3, D=128, W=4, eps=1e-6)


# ----------------------------------------------------------------------------------------------
# algorithmic work (multiply-adds at triangular cost, no recompute), per 64-token chunk and head
# ----------------------------------------------------------------------------------------------
def kda_kernel_flops(K, V, C=64):
    tri, stri = C * (C + 1) // 2, C * (C - 1) // 2
    fwd = {
        "build_am_kernel": tri * K + stri * K + C ** 3 / 6,
        "uw_kernel": tri * (V + K),
        "scan_fwd_kernel": 2 * C * K * V,
        "out_kernel": C * K * V + tri * V,
    }
    fwd_total = sum(fwd.values())
    bwd = {"scan_bwd_kernel": 3 * C * K * V + tri * V, "pullback_kernel": 2 * (tri + stri) * K}
    bwd["bwd_local_kernel"] = 2 * fwd_total - sum(bwd.values())
    tcl = {   # tensor-core lane kernels: the multiply-adds each one actually performs (different kernel boundaries and
        # a regrouped recurrence, so the parts do not add up to the reference-algorithm total below)
        "tc_intra_fwd_kernel": fwd["build_am_kernel"] + fwd["uw_kernel"] + C * K * K + C * C * K,   # + the chunk transition
        "tc_affine_scan_fwd_kernel": K * K * V + C * K * V,
        "tc_chunk_out_kernel": 2 * C * K * V + C * C * V,
        "tc_affine_scan_bwd_kernel": K * K * V + C * K * V,
        "tc_chunk_dz_kernel": C * C * V + C * K * V,
        "tc_intra_bwd_kernel": bwd["bwd_local_kernel"] + bwd["pullback_kernel"],
    }
    out = {k: 2.0 * v for k, v in {**fwd, **bwd, **tcl}.items()}     # FLOP = 2 * MAC
    out["_fwd_bwd_total"] = 2.0 * 3 * fwd_total
    return out


def chain_kernel_bytes(cfg):
    B, T, H, D = cfg["B"], cfg["T"], cfg["H"], cfg["D"]
    n = B * T * H * D * 2      # one bf16 tensor
    return {"conv_fwd_kernel": 2 * n, "conv_bwd_kernel": 3 * n, "rmsnorm_fwd_kernel": 3 * n, "rmsnorm_bwd_kernel": 5 * n}


# ----------------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index):
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.05)

    def start(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=1.0)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------------------------
# the chain workload
# ----------------------------------------------------------------------------------------------
class Chain:
    """conv(q,k,v) -> chunked KDA -> gated RMSNorm, forward and backward, via the public API."""

    def __init__(self, cfg, dev, seed):
        import experiment_swa_kda_b200 as m
        self.m, self.cfg, self.dev = m, cfg, dev
        B, T, H, D, W = cfg["B"], cfg["T"], cfg["H"], cfg["D"], cfg["W"]
        C = H * D
        gen = torch.Generator().manual_seed(seed)
        bf = torch.bfloat16
        self.host = {
            "xq": torch.randn(B, T, C, generator=gen).to(bf), "xk": torch.randn(B, T, C, generator=gen).to(bf),
            "xv": torch.randn(B, T, C, generator=gen).to(bf),
            "g": (-torch.nn.functional.softplus(torch.randn(B, T, H, D, generator=gen)) * 0.1).clamp(-5, 0).to(bf),
            "beta": torch.sigmoid(torch.randn(B, T, H, generator=gen)).to(bf),
            "gate": torch.randn(B, T, H, D, generator=gen).to(bf),
            "probe": torch.randn(B, T, H, D, generator=gen).to(bf),
        }
        self.host = {n: t.pin_memory() for n, t in self.host.items()}
        self.convs = [m.ShortConvolution(C, W).to(dev) for _ in range(3)]
        bound = (3 ** 0.5) * C ** -0.5
        for i, c in enumerate(self.convs):
            with torch.no_grad():
                c.weight.copy_((torch.rand(C, 1, W, generator=gen) * 2 - 1) * bound)
        self.norm = m.RMSNormGated(D, eps=cfg["eps"]).to(dev)
        self.x = None
        self.leaf_names = ("xq", "xk", "xv", "g", "beta", "gate")
        self.host_out = None

    def tokens(self):
        return self.cfg["B"] * self.cfg["T"]

    def upload(self):
        self.x = {n: t.to(self.dev, non_blocking=True) for n, t in self.host.items()}
        for n in self.leaf_names:
            self.x[n].requires_grad_(True)

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host.values())

    def step(self):
        x, cfg = self.x, self.cfg
        sh = (cfg["B"], cfg["T"], cfg["H"], cfg["D"])
        q, k, v = (t.view(sh) for t in self.m.short_convolutions(self.convs, (x["xq"], x["xk"], x["xv"])))
        y, _ = self.m.chunk_kda_norm(q, k, v, x["g"], x["beta"], x["gate"], self.norm.weight, eps=cfg["eps"])
        leaves = [x[n] for n in self.leaf_names] + [c.weight for c in self.convs] + [self.norm.weight]
        grads = torch.autograd.grad(y, leaves, x["probe"])
        return y, grads

    def download(self, y, grads):
        outs = [y.detach()] + [g for g in grads]
        if self.host_out is None:
            self.host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
        for h, t in zip(self.host_out, outs):
            h.copy_(t, non_blocking=True)
        return sum(h.numel() * h.element_size() for h in self.host_out)


class OpsChain:
    """The same chain driven the way the reference mixer drives it: autograd Functions that save only the operator inputs
    and the forward output and call `torch.ops.nanochat_kda.*` positionally (reference nanochat/mixers/kda.py:383-466):
    causal_convolution_forward x3 -> chunk_forward (raw gate and beta logits, activations fused) -> rmsnorm_gate_forward,
    and the three backwards."""

    def __init__(self, chain):
        from experiment_swa_kda_b200 import nanochat_ops
        nanochat_ops.register()
        ops = torch.ops.nanochat_kda
        self.c = chain
        cfg, dev = chain.cfg, chain.dev
        H, D = cfg["H"], cfg["D"]
        self.A_log = torch.zeros(H, device=dev, requires_grad=True)
        self.dt_bias = torch.zeros(H * D, device=dev, requires_grad=True)
        self.w = [c.weight.detach().squeeze(1).to(torch.bfloat16).requires_grad_(True) for c in chain.convs]
        self.nw = chain.norm.weight.detach().clone().requires_grad_(True)
        self.scale = D ** -0.5

        class Conv(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x, w):
                y, _ = ops.causal_convolution_forward(x, w, None, False)
                ctx.save_for_backward(x, w, y)
                return y

            @staticmethod
            def backward(ctx, dy):
                x, w, y = ctx.saved_tensors
                dx, dw, _ = ops.causal_convolution_backward(x, w, None, y, None, dy, None)
                return dx, dw

        class KDA(torch.autograd.Function):
            @staticmethod
            def forward(ctx, q, k, v, raw, bl, A, b, scale):
                o, _ = ops.chunk_forward(q, k, v, raw, bl, A, b, None, False, -5.0, scale)
                ctx.scale = scale
                ctx.save_for_backward(q, k, v, raw, bl, A, b, o)
                return o

            @staticmethod
            def backward(ctx, do):
                q, k, v, raw, bl, A, b, o = ctx.saved_tensors
                g = ops.chunk_backward(q, k, v, raw, bl, A, b, None, o, None, do, None, -5.0, ctx.scale)
                return (*g[:7], None)

        class Norm(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x, gate, w, eps):
                y, inv = ops.rmsnorm_gate_forward(x, gate, w, eps)
                ctx.eps = eps
                ctx.save_for_backward(x, gate, w, inv)
                return y

            @staticmethod
            def backward(ctx, dy):
                x, gate, w, inv = ctx.saved_tensors
                return (*ops.rmsnorm_gate_backward(x, gate, w, inv, dy, ctx.eps), None)

        self.Conv, self.KDA, self.Norm = Conv, KDA, Norm
        # raw gate / beta logits that activate to the chain's g and beta (A_log = 0, dt_bias = 0, lower bound -5)
        with torch.no_grad():
            p = (chain.x["g"].float() / -5.0).clamp(1e-7, 1 - 1e-7)
            self.raw = (torch.log(p) - torch.log1p(-p)).to(torch.bfloat16).requires_grad_(True)
            b = chain.x["beta"].float().clamp(1e-6, 1 - 1e-6)
            self.bl = (torch.log(b) - torch.log1p(-b)).to(torch.bfloat16).requires_grad_(True)

    def step(self):
        c, x, cfg = self.c, self.c.x, self.c.cfg
        sh = (cfg["B"], cfg["T"], cfg["H"], cfg["D"])
        q, k, v = (self.Conv.apply(x[n], w).view(sh) for n, w in zip(("xq", "xk", "xv"), self.w))
        o = self.KDA.apply(q, k, v, self.raw, self.bl, self.A_log, self.dt_bias, self.scale)
        y = self.Norm.apply(o, x["gate"], self.nw, cfg["eps"])
        leaves = [x["xq"], x["xk"], x["xv"], self.raw, self.bl, x["gate"], *self.w, self.nw, self.A_log, self.dt_bias]
        return y, torch.autograd.grad(y, leaves, x["probe"])


def oracle_chain_step(cfg, T, seed, threads):
    """The CPU oracle on the same chain, T tokens per sequence (cost is linear in T)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import kda_oracle as O
    torch.set_num_threads(threads)
    B, H, D, W = cfg["B"], cfg["H"], cfg["D"], cfg["W"]
    C = H * D
    gen = torch.Generator().manual_seed(seed)
    xs = [torch.randn(B, T, C, generator=gen).requires_grad_(True) for _ in range(3)]
    ws = [((torch.rand(C, W, generator=gen) * 2 - 1) * (3 ** 0.5) * C ** -0.5).requires_grad_(True) for _ in range(3)]
    g = (-torch.nn.functional.softplus(torch.randn(B, T, H, D, generator=gen)) * 0.1).clamp(-5, 0).requires_grad_(True)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen)).requires_grad_(True)
    gate = torch.randn(B, T, H, D, generator=gen).requires_grad_(True)
    nw = torch.ones(D, requires_grad=True)
    probe = torch.randn(B, T, H, D, generator=gen)
    t0 = time.perf_counter()
    q, k, v = (O.causal_conv(x, w)[0].view(B, T, H, D) for x, w in zip(xs, ws))
    o, _ = O.kda_recurrence(q, k, v, g, beta)
    y = O.rmsnorm_gated(o, gate, nw, cfg["eps"])
    torch.autograd.grad(y, xs + ws + [g, beta, gate, nw], probe)
    return time.perf_counter() - t0


# ----------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    T = 1024      # tokens per sequence of the sample: the token loop's autograd tape grows with T (about 2 GB here)
    for _ in range(args.warmup):
        oracle_chain_step(CHAIN, 64, 0, threads)
    times = [oracle_chain_step(CHAIN, T, 1 + i, threads) for i in range(args.steps)]
    dt = sum(times) / len(times)
    val = CHAIN["B"] * T / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config1 chain conv4+SiLU -> KDA fwd+bwd -> gated RMSNorm, B2 H3 D128", "chunk": 64,
                   "sample": f"T={T} tokens per sequence per step (cost linear in T; the GPU arm runs T=4096)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"oracle token loop + autograd, B2 T{T} H3 D128, {args.steps} steps"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--profile-warm", action="store_true", help="per-kernel pass without the L2 flush between steps (what a kernel costs inside the replayed graph, where its inputs were just written)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the config-3 / config-4 sharded workloads attached to the line")
    ap.add_argument("--tokens", type=int, default=8 * 8192, help="packed tokens of the varlen workload")
    ap.add_argument("--workload", default="chain", choices=["chain", "varlen", "decode", "pointwise", "train", "prefill"],
                    help="chain = config 1 (default, the driver's line); varlen = config 3; decode = config 4; pointwise = conv / gated RMSNorm at 256 MiB tensors; "
                         "train = config 2 (the reference's GPT + MuonAdamW step on these kernels); prefill = no-grad forward with the "
                         "convolutions as their own launch vs inside the intra-chunk kernel")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "train":
        import bench_train
        bench_train.run(args, rank, world, local)
        return
    if args.workload != "chain":
        import bench_extra
        bench_extra.run(args, rank, world, local)
        return

    import torch.distributed as dist
    from experiment_swa_kda_b200 import _lib
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    chain = Chain(CHAIN, dev, seed=1234 + rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # larger than the 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident arm -----------------------------------------------------------------
    # The step (every kernel of the forward and backward chain, launched through the public API) is captured
    # once into a CUDA graph and replayed: at this size the chain is ~30 short kernels and eager launching
    # leaves the GPU idle between them.
    chain.upload()
    for _ in range(max(args.warmup, 3)):
        chain.step()
    barrier()
    graph = None
    l0 = _lib.launch_count()
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs = chain.step()
        run_step = graph.replay
    else:
        outs = None
        run_step = chain.step
    launches_per_step = _lib.launch_count() - l0
    for _ in range(3):
        run_step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    l0 = _lib.launch_count()
    barrier()
    for a, b in ev:
        flush.zero_()
        a.record()
        run_step()
        b.record()
    barrier()
    launches = (_lib.launch_count() - l0) if graph is None else launches_per_step * args.steps
    clocks = sampler.stop()
    ms = sum(a.elapsed_time(b) for a, b in ev)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = chain.tokens() * world / (ms_step * 1e-3)

    # ---- end-to-end arm: pinned host inputs -> device -> chain -> pinned host results ----------
    # Every step copies its own inputs from pinned host memory and reads its own results back to pinned host memory.
    # With the graph, the copies run on streams of their own and are double-buffered, so the upload of step i+1 and the
    # download of step i-1 overlap the kernels of step i (PCIe is full duplex); the timed region runs from the first
    # upload to the last download, pipeline fill and drain included.
    def e2e_serial(steps):
        ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        nbytes = 0
        for a, b in ev2:
            flush.zero_()
            a.record()
            chain.upload()
            nbytes = chain.download(*chain.step())
            b.record()
        barrier()
        return sum(a.elapsed_time(b) for a, b in ev2), nbytes

    def e2e_pipelined(steps):
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        flat = [outs[0]] + list(outs[1])

        def carve(buf, like):          # 256-byte aligned views of one flat byte buffer, shaped like the tensors
            views, off = [], 0
            for t in like:
                n = t.numel() * t.element_size()
                views.append(buf[off:off + n].view(t.dtype).view(t.shape))
                off += (n + 255) // 256 * 256
            return views

        size = lambda like: sum((t.numel() * t.element_size() + 255) // 256 * 256 for t in like)
        names = list(chain.host)
        ins = [chain.host[n] for n in names]
        # one pinned buffer and one copy per direction and step: the step's inputs sit back to back in pinned host
        # memory, the results land back to back in another pinned buffer
        h_in = torch.empty(size(ins), dtype=torch.uint8).pin_memory()
        for v, t in zip(carve(h_in, ins), ins):
            v.copy_(t)
        d_in = [torch.empty(size(ins), dtype=torch.uint8, device=dev) for _ in range(2)]
        d_in_views = [carve(b, ins) for b in d_in]
        d_out = [torch.empty(size(flat), dtype=torch.uint8, device=dev) for _ in range(2)]
        d_out_views = [carve(b, flat) for b in d_out]
        h_out = [torch.empty(size(flat), dtype=torch.uint8).pin_memory() for _ in range(2)]
        ev = {k: [torch.cuda.Event() for _ in range(2)] for k in ("in_ready", "in_free", "out_ready", "out_free")}
        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        t_begin.record(s_in)
        with torch.no_grad():
            for i in range(steps):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev["in_free"][b])
                    d_in[b].copy_(h_in, non_blocking=True)
                    ev["in_ready"][b].record(s_in)
                main.wait_event(ev["in_ready"][b])
                flush.zero_()
                for n, v in zip(names, d_in_views[b]):
                    chain.x[n].copy_(v)                              # graph inputs live at fixed addresses
                ev["in_free"][b].record(main)
                graph.replay()
                if i >= 2:
                    main.wait_event(ev["out_free"][b])
                for dst, src in zip(d_out_views[b], flat):
                    dst.copy_(src)
                ev["out_ready"][b].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev["out_ready"][b])
                    h_out[b].copy_(d_out[b], non_blocking=True)
                    ev["out_free"][b].record(s_out)
        t_end.record(s_out)
        s_out.synchronize()
        barrier()
        return t_begin.elapsed_time(t_end), sum(t.numel() * t.element_size() for t in flat)

    def copy_only(steps):
        """The end-to-end arm's copies alone (same pinned buffers and sizes, both directions at once, no kernels): the
        host-path ceiling of the end-to-end figure."""
        flat = [outs[0]] + list(outs[1]) if outs is not None else list(chain.step()[1])
        n_in = chain.h2d_bytes()
        n_out = sum(t.numel() * t.element_size() for t in flat)
        h_in, h_out = torch.empty(n_in, dtype=torch.uint8).pin_memory(), torch.empty(n_out, dtype=torch.uint8).pin_memory()
        d_in, d_out = torch.empty(n_in, dtype=torch.uint8, device=dev), torch.empty(n_out, dtype=torch.uint8, device=dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        barrier()
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        s_in.wait_stream(torch.cuda.current_stream(dev))
        s_out.wait_stream(torch.cuda.current_stream(dev))
        a.record(s_in)
        s_out.wait_event(a)
        for _ in range(steps):
            with torch.cuda.stream(s_in):
                d_in.copy_(h_in, non_blocking=True)
            with torch.cuda.stream(s_out):
                h_out.copy_(d_out, non_blocking=True)
        b.record(s_in)
        c.record(s_out)
        s_in.synchronize()
        s_out.synchronize()
        barrier()
        return max(a.elapsed_time(b), a.elapsed_time(c))

    e2e_run = e2e_serial if graph is None else e2e_pipelined
    e2e_run(3)
    e2e_ms, d2h = e2e_run(args.steps)
    copy_only(3)
    t3 = torch.tensor([copy_only(args.steps)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t3, op=dist.ReduceOp.MAX)
    copy_ms_step = float(t3.item()) / args.steps

    # ---- the raw operator surface (torch.ops.nanochat_kda.*), driven like the reference mixer, same timing protocol ----
    ops_ms_step, ops_launches, ops_error, ops_kernels = None, None, None, None
    try:
        oc = OpsChain(chain)
        for _ in range(3):
            oc.step()
        barrier()
        l1 = _lib.launch_count()
        if not args.no_graph:
            og = torch.cuda.CUDAGraph()
            with torch.cuda.graph(og):
                oc.step()
            run_ops = og.replay
        else:
            run_ops = oc.step
        ops_launches = _lib.launch_count() - l1
        for _ in range(3):
            run_ops()
        barrier()
        ev3 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in ev3:
            flush.zero_()
            a.record()
            run_ops()
            b.record()
        barrier()
        t4 = torch.tensor([sum(a.elapsed_time(b) for a, b in ev3)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t4, op=dist.ReduceOp.MAX)
        ops_ms_step = float(t4.item()) / args.steps
        # where the operator surface spends its launches (eager, the library's launch accounting as below)
        torch.cuda.synchronize(dev)
        _lib.profile(True)
        for _ in range(args.steps):
            flush.zero_()
            oc.step()
        torch.cuda.synchronize(dev)
        ops_kernels = {k: [n / args.steps, round(tot / n * 1e3, 2)] for k, (n, tot) in _lib.profile_report().items()}
        _lib.profile(False)
        del oc
    except Exception as exc:      # the operator library is optional for the headline number; say why it is missing
        ops_ms_step = None
        ops_error = f"{type(exc).__name__}: {exc}"
    t2 = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_value = chain.tokens() * world / (float(t2.item()) / args.steps * 1e-3)
    e2e_mode = ("serial: upload, kernels, download on one stream" if graph is None else
                "double-buffered: upload of step i+1 and download of step i-1 overlap the kernels of step i")

    # ---- per-kernel device time (separate pass so the events do not perturb the numbers above) --
    chain.upload()
    torch.cuda.synchronize(dev)
    _lib.profile(True)
    for _ in range(args.steps):
        if not args.profile_warm:
            flush.zero_()
        chain.step()
    torch.cuda.synchronize(dev)
    rep = _lib.profile_report()
    _lib.profile(False)

    sharded = None
    if not args.no_sharded:
        import bench_extra
        torch.cuda.empty_cache()
        sharded = bench_extra.sharded_summary(args, rank, world, local, dist)

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm_peak = peaks.get("hbm_gbs", 6650.0)
        tf_peak = peaks.get("bf16_tflops", 1590.0)
        src = "measured" if peaks else "fallback"
        nch = CHAIN["B"] * (CHAIN["T"] // 64) * CHAIN["H"]
        flops = kda_kernel_flops(CHAIN["D"], CHAIN["D"])
        nbytes = chain_kernel_bytes(CHAIN)
        kern = {}
        total_ms = sum(v[1] for v in rep.values()) or 1.0
        for name, (n, tot) in rep.items():
            avg_ms = tot / n
            row = {"launches_per_step": n / args.steps, "avg_us": avg_ms * 1e3, "share": tot / total_ms}
            if name in flops:
                row["tflops"] = flops[name] * nch / (avg_ms * 1e-3) / 1e12
            if name in nbytes:
                row["gbs"] = nbytes[name] / (avg_ms * 1e-3) / 1e9
            kern[name] = row
        top = max(rep, key=lambda k: rep[k][1]) if rep else None      # per kernel name; the two scans are separate instantiations
        traffic = None
        try:
            traffic = json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json"))).get(top)
        except Exception:
            pass
        if top in flops:
            roof = {"kernel": top, "bound": "tensor", "achieved": kern[top]["tflops"], "peak": tf_peak, "unit": "TFLOP/s",
                    "frac": kern[top]["tflops"] / tf_peak, "traffic": traffic, "peak_source": src}
        elif top in nbytes:
            roof = {"kernel": top, "bound": "hbm", "achieved": kern[top]["gbs"], "peak": hbm_peak, "unit": "GB/s",
                    "frac": kern[top]["gbs"] / hbm_peak, "traffic": traffic, "peak_source": src}
        else:
            roof = {"kernel": top, "bound": "hbm", "achieved": None, "peak": hbm_peak, "unit": "GB/s", "frac": None,
                    "traffic": traffic, "peak_source": src}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "config1 chain: conv4+SiLU(q,k,v) -> chunked KDA fwd+bwd -> gated RMSNorm fwd+bwd; "
                                   "B2 T4096 H3 Dk=Dv=128 chunk64, bf16 I/O, fp32 state/accumulation",
                       "tokens_per_step_per_gpu": chain.tokens(), "l2": "flushed between steps (256 MiB write)",
                       "lane": "tcgen05 (intra-chunk products, chunk transitions and affine state scans)",
                       "launch": "eager" if args.no_graph else "CUDA graph replay of the captured step", "sharding": "replicated per-GPU batches, no collective"},
            "tflops_algorithmic": flops["_fwd_bwd_total"] * nch * world / (ms_step * 1e-3) / 1e12,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": chain.h2d_bytes(), "d2h_bytes_per_step": d2h,
                    "ms_per_step": float(t2.item()) / args.steps, "copies": e2e_mode,
                    "copy_only_ms_per_step": copy_ms_step,
                    "copy_only_note": "the same bytes per step in both directions at once from/to pinned host memory with no "
                                      "kernel in between: the host-path floor of ms_per_step"},
            "ops_path": ({"ms_per_step": ops_ms_step, "tokens_per_s": chain.tokens() * world / (ops_ms_step * 1e-3),
                          "launches_per_step": ops_launches, "ratio_to_value_arm": ops_ms_step / ms_step,
                          "what": "the same chain through torch.ops.nanochat_kda.* (raw gate / beta logits, activations fused, "
                                  "forward sidecar instead of a recompute), driven by reference-style autograd Functions",
                          "kernels": ops_kernels}
                         if ops_ms_step else {"unavailable": ops_error}),
            "sharded": sharded,
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "kernels": kern,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            oracle_chain_step(CHAIN, 64, 0, threads)
            Ts, nrep = 1024, 12      # about 10 s of CPU work
            dts = [oracle_chain_step(CHAIN, Ts, 1 + i, threads) for i in range(nrep)]
            dt = sum(dts) / nrep
            line["cpu_baseline"] = {"value": CHAIN["B"] * Ts / dt, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"oracle token loop + autograd on the same chain, B2 T{Ts} H3 D128, {nrep} steps "
                                              f"({sum(dts):.1f} s); cost is linear in T, the GPU arm runs T=4096"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
