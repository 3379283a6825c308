"""Worker: sequence-parallel conv / banded attention / recurrent scan and the vocabulary- and feature-parallel reductions
against the unsplit computation, over CPU ranks."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200.ops import functional as Fn  # noqa: E402
from dew_b200.ops import scan  # noqa: E402
from dew_b200.parallel import sp_ops as S  # noqa: E402


def main():
    backend = sys.argv[1] if len(sys.argv) > 1 else "gloo"
    if backend == "nccl":
        # GPU ranks: every exchange below is one kernel over peer memory (parallel.peer_link)
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        from dew_b200.parallel.peer_link import PeerLink
        link = PeerLink(None, max_bytes=1 << 20, device=dev, wait_limit_s=10.0)
        S.use_peer_link(link)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    rank, N = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    res = {}
    _randn, _rand, _randint = torch.randn, torch.rand, torch.randint

    class _T:                                   # the same draws on every backend: made on the CPU, moved to the device
        @staticmethod
        def randn(*a, **k):
            return _randn(*a, **k).to(dev)

        @staticmethod
        def rand(*a, **k):
            return _rand(*a, **k).to(dev)

        @staticmethod
        def randint(*a, **k):
            return _randint(*a, **k).to(dev)
    B, T, C, K = 2, 12 * N, 6, 4
    sl = slice(rank * T // N, (rank + 1) * T // N)
    # ---- short conv with halo
    x = _T.randn(B, T, C, generator=g)
    w, b = _T.randn(C, K, generator=g), _T.randn(C, generator=g)
    xf = x.clone().requires_grad_()
    ref = scan.short_conv_reference(xf, w, b, True)
    ref.pow(2).sum().backward()
    xl = x[:, sl].clone().requires_grad_()
    out = S.sequence_parallel_short_conv(xl, w, b, True)
    out.pow(2).sum().backward()
    res["conv_out"] = float((out - ref[:, sl]).abs().max())
    res["conv_dx"] = float((xl.grad - xf.grad[:, sl]).abs().max())
    # ---- banded attention with halo
    H, Hkv, D, W = 4, 2, 8, 5
    q, k, v = (_T.randn(B, T, h, D, generator=g) for h in (H, Hkv, Hkv))
    full = [t.clone().requires_grad_() for t in (q, k, v)]
    ref = Fn.attention_reference(*full, causal=True, window=W)
    ref.pow(2).sum().backward()
    loc = [t[:, sl].clone().requires_grad_() for t in (q, k, v)]
    out = S.banded_attention(*loc, W)
    out.pow(2).sum().backward()
    res["band_out"] = float((out - ref[:, sl]).abs().max())
    res["band_dk"] = float((loc[1].grad - full[1].grad[:, sl]).abs().max())
    # ---- gated delta rule across ranks
    Hh, Dk, Dv = 2, 8, 6
    f = torch.float64
    qq = torch.nn.functional.normalize(_T.randn(B, T, Hh, Dk, dtype=f, generator=g), dim=-1)
    kk = torch.nn.functional.normalize(_T.randn(B, T, Hh, Dk, dtype=f, generator=g), dim=-1)
    vv = _T.randn(B, T, Hh, Dv, dtype=f, generator=g)
    gg = -_T.rand(B, T, Hh, dtype=f, generator=g) * 0.2
    bb = _T.rand(B, T, Hh, dtype=f, generator=g)
    fulls = [t.clone().requires_grad_() for t in (qq, kk, vv, gg, bb)]
    ro, rs = scan.gated_delta_rule_recurrent(*fulls)
    (ro.pow(2).sum() + rs.pow(2).sum()).backward()
    locs = [t[:, sl].clone().requires_grad_() for t in (qq, kk, vv, gg, bb)]
    out, fin = S.sequence_parallel_scan(lambda s0: scan.gated_delta_rule_chunked(*locs, initial_state=s0), torch.zeros(B, Hh, Dk, Dv, dtype=f, device=dev))
    loss = out.pow(2).sum() + (fin.pow(2).sum() if rank == N - 1 else 0 * fin.sum())
    loss.backward()
    res["scan_out"] = float((out - ro[:, sl]).abs().max())
    res["scan_dv"] = float((locs[2].grad - fulls[2].grad[:, sl]).abs().max())
    res["scan_dk"] = float((locs[1].grad - fulls[1].grad[:, sl]).abs().max())
    if rank == N - 1:
        res["scan_state"] = float((fin - rs).abs().max())
    # ---- vocabulary-parallel cross-entropy and feature-sharded RMSNorm
    Tt, d, V = 10, 8, 6 * N
    h = _T.randn(Tt, d, generator=g)
    Wf = _T.randn(V, d, generator=g)
    tg = _T.randint(0, V, (Tt,), generator=g)
    tg[3] = -100
    hf, wf = h.clone().requires_grad_(), Wf.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(hf @ wf.t(), tg, ignore_index=-100, reduction="sum")
    ref.backward()
    hl, wl = h.clone().requires_grad_(), Wf[rank * V // N:(rank + 1) * V // N].clone().requires_grad_()
    loss, mass = S.vocab_parallel_cross_entropy(hl, wl, tg)
    loss.backward()
    dh = hl.grad.clone()
    dist.all_reduce(dh)                              # every rank contributes its shard's part of d hidden
    res["vce_loss"] = abs(float(loss) - float(ref))
    res["vce_mass"] = abs(int(mass) - 9)
    res["vce_dh"] = float((dh - hf.grad).abs().max())
    res["vce_dw"] = float((wl.grad - wf.grad[rank * V // N:(rank + 1) * V // N]).abs().max())
    xx, ww = _T.randn(3, 4 * N, generator=g), _T.randn(4 * N, generator=g)
    ref = Fn.rms_norm_reference(xx, ww, 1e-6)
    cs = slice(rank * 4, (rank + 1) * 4)
    res["norm"] = float((S.sharded_rms_norm(xx[:, cs], ww[cs], 4 * N) - ref[:, cs]).abs().max())
    if backend == "nccl":
        from dew_b200.ops import library as L
        torch.cuda.synchronize()
        L.check_status()
        res["launches"] = -float(L.LAUNCHES)                # (negative: passes the "below tolerance" check, read by the test)
    gathered = [None] * N
    dist.all_gather_object(gathered, res)
    if rank == 0:
        keys = set().union(*[set(r) for r in gathered])
        print("RESULT " + json.dumps({k: max(r[k] for r in gathered if k in r) for k in keys}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
