"""The cost model: single-operation rooflines behave, and whole-step predictions land near the steps measured on B200s."""
import pytest

from dew_b200.ops.step_cost import PRESETS, Machine, Transformer, attention_ms, collective_ms, decode_step, gemm_ms, main, rowwise_ms, transformer_step

M = Machine()          # nominal constants: the test does not depend on a measurement file being present


def test_single_operation_rooflines():
    big = gemm_ms(16384, 4096, 4096, M)
    assert 2 * 16384 * 4096 * 4096 / (big * 1e-3) / 1e12 < M.bf16_tflops            # never above the peak
    assert gemm_ms(16384, 8192, 4096, M) == pytest.approx(2 * big, rel=0.1)
    skinny = gemm_ms(128, 4096, 4096, M)                                             # bandwidth-bound: reading the weight dominates
    assert skinny == pytest.approx(4096 * 4096 * 2 / (M.hbm_gbs * 1e9 * 0.85) * 1e3 + 0.002, rel=0.1)           # plus a launch
    # a product with one tile more than a whole wave costs about a wave more
    assert gemm_ms(256 * 38, 512, 4096, M) > 1.8 * gemm_ms(256 * 37, 512, 4096, M) - 0.01
    assert attention_ms(2, 4096, 32, 8, 128, M, backward=True) > 2 * attention_ms(2, 4096, 32, 8, 128, M)
    assert attention_ms(1, 16384, 32, 8, 128, M, window=2048) < 0.3 * attention_ms(1, 16384, 32, 8, 128, M)
    assert rowwise_ms(6.553e9, M) == pytest.approx(1 / 0.85, rel=0.01)                        # 6.553 GB at 6553 GB/s: a millisecond over the efficiency
    assert collective_ms("all_reduce", 1 << 30, 1, M) == 0.0
    ar8 = collective_ms("all_reduce", 1 << 30, 8, M)
    assert (1 << 30) * 2 * 7 / 8 / (ar8 * 1e-3) / 1e9 == pytest.approx(M.nvlink_bus_gbs, rel=0.02)       # the bus bandwidth it was built from
    assert collective_ms("all_gather", 1 << 30, 8, M) < ar8 and collective_ms("all_reduce", 4096, 8, M) == pytest.approx(0.012, rel=0.05)
    with pytest.raises(ValueError):
        collective_ms("broadcast", 1, 2, M)


def test_step_predictions_against_measured_steps():
    dense = PRESETS["dense8b"]
    assert dense.params == pytest.approx(8.03e9, rel=0.01)
    one = transformer_step(dense, sequences=32, seq_len=4096, world=1, machine=M)
    eight = transformer_step(dense, sequences=32, seq_len=4096, world=8, machine=M)
    # measured on B200s: 21.3 K tok/s on one GPU (6.18 s a step), 168.4 K on eight, 87.7 GB a GPU at eight
    assert one["tokens_per_s"] == pytest.approx(21300, rel=0.10) and eight["tokens_per_s"] == pytest.approx(168400, rel=0.10)
    assert eight["memory_gb"] == pytest.approx(87.7, rel=0.10) and eight["fits"]
    assert one["by_family"]["gemm"] / one["ms"] == pytest.approx(0.77, abs=0.06)                            # the measured share of the products
    assert 0.40 < one["mfu_datasheet"] < 0.55
    sharded = transformer_step(dense, sequences=32, seq_len=4096, world=8, machine=M, sharded_state=True)
    assert sharded["memory_gb"] < 0.55 * eight["memory_gb"] and sharded["ms"] > eight["ms"]
    tp = transformer_step(dense, sequences=32, seq_len=4096, world=8, tensor=2, machine=M)
    assert tp["by_family"]["tensor_parallel"] > 0 and tp["tokens_per_s"] < eight["tokens_per_s"]
    remat = transformer_step(dense, sequences=32, seq_len=4096, world=8, machine=M, remat=True)
    assert remat["ms"] > 1.2 * eight["ms"] and remat["activation_gb"] < 0.5 * eight["activation_gb"]
    wide = Transformer(features=6656, layers=60, heads=52, kv_heads=8, mlp=17920)                          # about 29 B parameters
    assert 28e9 < wide.params < 32e9
    big = transformer_step(wide, sequences=8, seq_len=4096, world=8, machine=M)
    assert not big["fits"] and transformer_step(wide, sequences=8, seq_len=4096, microbatch=1, world=8, machine=M, sharded_state=True)["fits"]
    assert not transformer_step(PRESETS["llama70b"], sequences=8, seq_len=4096, microbatch=1, world=8, machine=M, sharded_state=True)["fits"]
    # the expert-parallel step (measured 256 K tok/s at eight GPUs): the model leaves out latency-bound small kernels and lands high
    moe = transformer_step(PRESETS["moe"], sequences=16, seq_len=4096, world=8, expert=8, machine=M, mx_experts=True)
    assert 256000 < moe["tokens_per_s"] < 1.4 * 256000 and moe["by_family"]["exchange"] > 0.2 * moe["ms"]
    # serving: 128 rows at tensor parallel 8 measured 3.04 ms a step; one GPU 16.2 K tok/s
    tp8 = decode_step(dense, rows=128, context=1024, tensor=8, machine=M)
    assert tp8["ms"] == pytest.approx(3.04, rel=0.15) and tp8["by_family"]["all_reduce"] > 0.4 * tp8["ms"]
    one_gpu = decode_step(dense, rows=128, context=1024, tensor=1, machine=M)
    assert one_gpu["tokens_per_s"] == pytest.approx(16200, rel=0.25)
    out = main(["--model", "qwen3_0p6b", "--gpus", "1", "--sequences", "8", "--seq-len", "1024", "--microbatch", "8"])
    assert out["fits"] and out["ms"] > 0
