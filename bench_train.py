"""BASELINE config 2: the reference's nanochat-KDA training step on the B200 kernels, data-parallel over NCCL.

    python bench.py --workload train [--gpus N]        (torchrun for N > 1, one rank per GPU)

The caller is the reference's own, unmodified Python - `nanochat.gpt.GPT` (6 KDA layers, d_model 384 = 3 x 128, MLP 4x,
vocab 65536), `GPT.setup_optimizer()` -> `MuonAdamW` (Muon for matrices, AdamW for embeddings / scalars; in a process
group its step reduce-scatters gradients and all-gathers parameters over NCCL, reference nanochat/optim.py:428-459) and
the micro-step loop of scripts/base_train.py:575-619 - installed from the reference tree into the git-ignored
baseline/_ref.  Its `project_cuda` KDA backend is pointed at this library by experiment_swa_kda_b200.nanochat_plugin;
nanochat/mixers/kda.py routes to `torch.ops.nanochat_kda.*` unchanged.  Eager bf16, B2 x T4096 per GPU, 4 micro-steps per
update (32,768 tokens per GPU per update: weak scaling, total batch = 32,768 x N), seed 42, tokens uniform over the
vocabulary.  Protocol of the reference's benchmark (docs/BENCHMARK.md:21-23): 7 updates, the first two are warm-up, the
figure is total tokens / median update time of the other five; timed with CUDA events between barriers, max over ranks.
"""

from __future__ import annotations

import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(ROOT, "baseline", "_ref")
GB10_TOKENS_PER_S = 44942.0      # the reference's published figure for this workload on one GB10 (docs/BENCHMARK.md:58-63)


def build(device, T, kda_backend, seed=42, n_layer=6, vocab=65536):
    from nanochat.gpt import GPT, GPTConfig
    cfg = GPTConfig(sequence_len=T, vocab_size=vocab, n_layer=n_layer, n_head=3, n_kv_head=3, n_embd=384, window_pattern="K",
                    force_final_full=False, kda_backend=kda_backend)
    torch.manual_seed(seed)
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device=device)
    model.init_weights()
    return model, model.setup_optimizer()


def update(model, opt, batches):
    """One optimizer update: gradient accumulation over the micro-batches, then the reference optimizer's step."""
    n = len(batches)
    loss = None
    for x, y in batches:
        loss = model(x, y)
        (loss / n).backward()
    opt.step()
    model.zero_grad(set_to_none=True)
    return loss.detach()


class GraphedMicroStep:
    """One micro-step (forward, loss / n, backward into the parameters' existing .grad tensors) captured once in a CUDA
    graph and replayed per micro-batch with the tokens copied into fixed buffers; the optimizer step stays eager (the
    reference's own, with its NCCL collectives).  This is the first item the reference's plan lists for this caller once
    the KDA calls are fast: at B200 speed the eager micro-step is bound by launching the model's ~1,000 small kernels."""

    def __init__(self, model, batch, n):
        x, y = batch
        self.model, self.n = model, n
        self.x, self.y = x.clone(), y.clone()
        # gradients must exist before the capture so that the captured backward accumulates in place
        for _ in range(2):
            (model(self.x, self.y) / n).backward()
        torch.cuda.synchronize()
        model.zero_grad(set_to_none=False)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = model(self.x, self.y)
            (self.loss / n).backward()
        model.zero_grad(set_to_none=False)

    def update(self, opt, batches):
        for x, y in batches:
            self.x.copy_(x)
            self.y.copy_(y)
            self.graph.replay()
        opt.step()
        self.model.zero_grad(set_to_none=False)
        return self.loss.detach().clone()


def import_reference():
    if not os.path.isdir(os.path.join(REF, "nanochat")):
        return "baseline/_ref holds no installed reference (python -m pip install --no-deps --target baseline/_ref <reference tree>)"
    if REF not in sys.path:
        sys.path.insert(0, REF)
    os.environ.setdefault("TORCH_COMPILE_DISABLE", "1")      # eager, as the workload is defined; no inductor in the timed path
    try:
        from experiment_swa_kda_b200 import nanochat_plugin
        nanochat_plugin.install()
        from nanochat.mixers.kda import prepare_kda_backend
        prepare_kda_backend("project_cuda")
    except Exception as exc:      # noqa: BLE001 - reported in the JSON line
        return f"{type(exc).__name__}: {exc}"
    return None


def run(args, rank, world, local):
    import torch.distributed as dist
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    why = import_reference()
    if why is not None:
        if rank == 0:
            print(json.dumps({"metric": "nanochat_kda_train_tokens_per_s", "unavailable": why, "n_gpus": world}), flush=True)
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from experiment_swa_kda_b200 import _lib
    B, T, accum, vocab = 2, 4096, 4, 65536
    model, opt = build(dev, T, "project_cuda")
    gen = torch.Generator(device=dev).manual_seed(42 + rank)
    n_updates, n_warm = 7, 2
    data = [[(torch.randint(0, vocab, (B, T), generator=gen, device=dev), torch.randint(0, vocab, (B, T), generator=gen, device=dev))
             for _ in range(accum)] for _ in range(n_updates)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    graphed, graph_note = None, "eager micro-steps"
    if not getattr(args, "no_graph", False):
        try:
            graphed = GraphedMicroStep(model, data[0][0], accum)
            graph_note = "micro-step (forward + backward) captured in a CUDA graph and replayed; optimizer step eager"
        except Exception as exc:      # noqa: BLE001 - the eager path is the fallback, and the line says which one ran
            graphed, graph_note = None, f"eager micro-steps (graph capture failed: {type(exc).__name__}: {exc})"[:300]
            torch.cuda.synchronize(dev)
            model.zero_grad(set_to_none=True)
    times, losses = [], []
    l0 = _lib.launch_count()
    torch.cuda.reset_peak_memory_stats(dev)
    for u in range(n_updates):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        loss = graphed.update(opt, data[u]) if graphed is not None else update(model, opt, data[u])
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
        losses.append(float(loss.item()))
    launches = _lib.launch_count() - l0
    peak = torch.cuda.max_memory_allocated(dev)
    if rank == 0:
        med = statistics.median(times[n_warm:])
        total = B * T * accum * world
        line = {
            "metric": "nanochat_kda_train_tokens_per_s", "value": total / (med * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": n_updates - n_warm, "warmup": n_warm, "ms_per_step": med, "higher_is_better": True, "scaling": "weak",
            # the reference's published figure for this exact workload (one GB10, docs/BENCHMARK.md:58-63); whole-job value over it
            "vs_baseline": total / (med * 1e-3) / GB10_TOKENS_PER_S, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config2 nanochat-KDA training step: reference GPT (6 KDA layers, d_model 384 = 3x128, MLP 4x, vocab "
                                   "65536) + MuonAdamW, B2 T4096 per GPU, grad-accum 4, seed 42, uniform tokens, bf16; KDA layers "
                                   "on libkda_b200 through torch.ops.nanochat_kda.*",
                       "launch": graph_note,
                       "tokens_per_update": total, "parallelism": f"dp{world}" + (" (NCCL reduce-scatter / all-gather in MuonAdamW.step)" if world > 1 else ""),
                       "optimizer_kernels": "eager (TORCH_COMPILE_DISABLE=1)" if os.environ.get("TORCH_COMPILE_DISABLE") == "1" else "torch.compile",
                       "protocol": "7 updates, 2 warm-up, median of 5"},
            "update_ms": times, "loss": losses, "kda_kernel_launches": int(launches), "peak_memory_mib": peak / 2 ** 20,
            "context": {"reference_gb10_tokens_per_s": GB10_TOKENS_PER_S, "ratio_to_gb10": total / world / (med * 1e-3) / GB10_TOKENS_PER_S,
                        "note": "the reference's published figure is one GB10 (sm_121); per-GPU ratio, different hardware"},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
