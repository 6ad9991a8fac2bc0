"""The reference's own GPT + MuonAdamW training step with its `project_cuda` KDA backend resolved to this library
(experiment_swa_kda_b200.nanochat_plugin), against the same step on the reference's eager `reference` backend (run on the
host: on a CUDA device that backend's convolution wants the FLA Triton package, which is not part of this tier).

The reference Python comes from the git-ignored baseline/_ref install; nothing of it is modified.  BASELINE config 2's
model (6 KDA layers, d_model 384 = 3 x 128, vocab 65536) at a reduced sequence length, same seed, same synthetic tokens:
the loss sequence over the first updates must agree (bf16 on both sides; the KDA layers are the only difference).
"""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanochat")), reason="no installed reference under baseline/_ref")
def test_loss_sequence_matches_the_reference_backend_at_reduced_length():
    sys.path.insert(0, ROOT)
    import bench_train
    assert bench_train.import_reference() is None
    from experiment_swa_kda_b200 import _lib
    dev = torch.device("cuda:0")
    T, B, accum, updates = 256, 2, 2, 3
    gen = torch.Generator().manual_seed(42)
    data = [[(torch.randint(0, 65536, (B, T), generator=gen), torch.randint(0, 65536, (B, T), generator=gen))
             for _ in range(accum)] for _ in range(updates)]
    losses = {}
    for backend, where in (("project_cuda", dev), ("reference", torch.device("cpu"))):
        model, opt = bench_train.build(where, T, backend)
        n0 = _lib.launch_count()
        losses[backend] = [float(bench_train.update(model, opt, [(x.to(where), y.to(where)) for x, y in batch]).item()) for batch in data]
        launched = _lib.launch_count() - n0
        assert (launched > 0) == (backend == "project_cuda")      # the project backend really ran this library's kernels
        del model, opt
        torch.cuda.empty_cache()
    for a, b in zip(losses["project_cuda"], losses["reference"]):
        assert abs(a - b) <= 1e-2 * abs(b), losses
    assert losses["reference"][-1] < losses["reference"][0]      # and the step does train


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanochat")), reason="no installed reference under baseline/_ref")
def test_graph_replayed_micro_steps_train_exactly_like_eager_ones():
    """bench_train.GraphedMicroStep (forward + backward captured once, replayed per micro-batch, gradients accumulated
    in place, optimizer step eager) gives the same loss sequence as the eager update, bit for bit: the operator library
    is capturable (no host synchronisation, the forward's sidecar found again at capture time)."""
    sys.path.insert(0, ROOT)
    import bench_train
    assert bench_train.import_reference() is None
    dev = torch.device("cuda:0")
    T, B, accum, updates = 256, 2, 2, 3
    gen = torch.Generator().manual_seed(7)
    data = [[(torch.randint(0, 65536, (B, T), generator=gen).to(dev), torch.randint(0, 65536, (B, T), generator=gen).to(dev))
             for _ in range(accum)] for _ in range(updates)]
    losses = []
    for graphed in (False, True):
        model, opt = bench_train.build(dev, T, "project_cuda")
        if graphed:
            step = bench_train.GraphedMicroStep(model, data[0][0], accum)
            losses.append([float(step.update(opt, batch).item()) for batch in data])
        else:
            losses.append([float(bench_train.update(model, opt, batch).item()) for batch in data])
        del model, opt
        torch.cuda.empty_cache()
    assert losses[0] == losses[1], losses
