"""Expert parallelism over 2 and 4 CPU ranks equals the unsharded mixture-of-experts layer."""
import json
import os
import subprocess
import sys

import pytest

WORKER = os.path.join(os.path.dirname(__file__), "workers", "ep_worker.py")


@pytest.mark.parametrize("world,port", [(2, 29641), (4, 29642)])
def test_expert_parallel_matches_single_process(world, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["out_err"] < 1e-5 and r["dx_err"] < 1e-4 and r["dw_err"] < 1e-4, r


def test_expert_parallel_with_gathered_weights_matches_single_process():
    """``dispatch='global'``: the experts' weights are all-gathered and every rank runs its own tokens; the weight gradients
    return to their owners by a reduce-scatter."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29655", WORKER, "global"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["out_err"] < 1e-5 and r["dx_err"] < 1e-4 and r["dw_err"] < 1e-4, r


def _run_moe(world, port):
    worker = os.path.join(os.path.dirname(__file__), "workers", "moe_fsdp_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), worker]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    return json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])


def test_moe_lm_trains_under_fsdp_with_expert_parallel_units():
    """Experts split over 2 ranks as rank-local units of the FSDP engine (no reduction, local AdamW), the rest sharded:
    the same losses and final weights as one process holding every expert."""
    one, two = _run_moe(1, 29651), _run_moe(2, 29652)
    assert two["local_units"] == 2 and two["losses"][-1] < two["losses"][0]
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (one, two)
    assert abs(one["digest"] - two["digest"]) < 1e-3 * one["digest"], (one["digest"], two["digest"])
    assert two["experts"] == one["experts"]              # the export concatenates every rank's experts


@pytest.mark.gpu
@pytest.mark.multigpu
def test_expert_parallel_two_gpus_peer_memory_exchange():
    """Dispatch by peer stores into the owners' expert-sorted buffers and combine by peer loads (one kernel each), against
    the NCCL all-to-all form of the same layer; three calls in a row so that buffers and flags are reused."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = os.path.join(os.path.dirname(__file__), "workers", "ep_gpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29661", worker]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert max(r["errs"]) < 5e-2, r


def test_expert_product_written_into_a_given_buffer_keeps_autograd_intact():
    """The last expert product may write straight into a caller's buffer (the one peers pull from): same values and gradients as the
    allocating form, call after call, and the buffer itself never joins the autograd graph."""
    import torch
    from dew_b200.ops import grouped as G
    from dew_b200.ops import mx
    torch.manual_seed(0)
    E, N, K = 2, 128, 128
    lay = G.group_layout(torch.randint(0, E, (200,)), E)
    x = torch.zeros(lay.rows, K).bfloat16()
    x[lay.positions] = torch.randn(200, K).bfloat16()
    x.requires_grad_()
    w = torch.randn(E, N, K).bfloat16().requires_grad_()
    base = torch.zeros(lay.rows * N, dtype=torch.bfloat16)
    grads = []
    for _ in range(2):
        x.grad = w.grad = None
        out = torch.empty(0, dtype=torch.bfloat16).set_(base.untyped_storage(), 0, (lay.rows, N), (N, 1))
        y = mx.mx_grouped_linear(x, w, lay, out, False)
        assert y.data_ptr() == base.data_ptr() and y.grad_fn is not None
        (y.float() * 2).sum().backward()
        grads.append((x.grad.clone(), w.grad.clone()))
        assert base.grad_fn is None and not base.requires_grad
    x.grad = w.grad = None
    y2 = mx.mx_grouped_linear(x, w, lay)
    (y2.float() * 2).sum().backward()
    assert torch.equal(y2, y.detach()) and torch.equal(x.grad, grads[1][0]) and torch.equal(w.grad, grads[1][1])
    assert torch.equal(grads[0][0], grads[1][0])
