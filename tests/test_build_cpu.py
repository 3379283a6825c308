"""The resource gate: every kernel of the library compiles for sm_100a and none spills more than a few words (a kernel
that starts to spill is caught here, before any GPU run)."""
import shutil

import pytest

from dew_b200.ops import build as B

SPILL_BUDGET = 64          # bytes of spill stores per kernel


@pytest.mark.skipif(shutil.which("nvcc") is None and not __import__("os").path.exists("/usr/local/cuda/bin/nvcc"), reason="needs nvcc")
def test_every_kernel_builds_within_its_register_budget():
    B.build(verbose=False)
    res = B.kernel_resources()
    assert len(res) > 100                                    # the logs were parsed
    over = {k: v for k, v in res.items() if v["spill_stores"] > SPILL_BUDGET}
    assert not over, over
    assert all(0 < v["registers"] <= 255 for v in res.values())
    # the tensor-core kernels exist under their names
    names = " ".join(k[1] for k in res)
    for needle in ("flash_fwd_kernel", "flash_dq_kernel", "flash_dkv_kernel", "gemm_pair_kernel", "gdn_scan_fwd_kernel", "moe_push_kernel",
                   "paged_decode_tma_kernel", "rs_adamw_ag_kernel"):
        assert needle in names, needle
