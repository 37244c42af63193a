"""Pure parts of the receipt: the roofline arithmetic and the strategy check on kernel manifests."""

from __future__ import annotations

import math

import pytest

from tpu_cake_b200 import receipt


def test_roofline_metrics_follow_the_reference_formulae():
    model_input = {
        "hardware": {"compute_peak_ops_s": 1.0e15, "memory_bandwidth_bytes_s": 5.0e12, "effective_compute_fraction": 0.9,
                     "effective_memory_fraction": 0.8},
        "workload": {"operations": 2.0e12, "bytes_read": 3.0e8, "bytes_written": 1.0e8, "measured_time_s": 4.0e-3},
    }
    m = receipt.roofline_metrics(model_input)
    assert m["total_bytes"] == 4.0e8 and m["arithmetic_intensity_ops_per_byte"] == 5000.0
    assert math.isclose(m["compute_time_s"], 2.0e12 / 9.0e14) and math.isclose(m["memory_time_s"], 4.0e8 / 4.0e12)
    assert m["lower_bound_time_s"] == max(m["compute_time_s"], m["memory_time_s"])
    assert math.isclose(m["measured_throughput_ops_s"], 5.0e14)
    assert math.isclose(m["attainable_throughput_ops_s"], min(9.0e14, 4.0e12 * 5000.0))
    assert math.isclose(m["peak_efficiency"], 5.0e14 / 9.0e14)
    assert math.isclose(m["headroom_to_attainable"] * m["attainable_efficiency"], 1.0)


def test_kernel_manifest_must_match_the_declared_strategy():
    p2p = "p2p_fused_epilogue_bf16_transport"
    assert receipt.expected_kernels(p2p, 8, 256) == (["cake_matmul_rs_sm100<256>", "cake_reduce_slots_sm100"], ("ncclDevKernel_ReduceScatter",))
    assert receipt.expected_kernels("nccl_reduce_scatter", 8, 128)[0] == ["cake_matmul_rs_sm100<128>"]
    assert receipt.expected_kernels(p2p, 1, 256)[0] == ["cake_matmul_rs_sm100<256>"]
    receipt._validate_strategy({"kernels": ["cake_matmul_rs_sm100<256>", "cake_reduce_slots_sm100"]}, p2p, 8, 256)
    with pytest.raises(ValueError, match="KERNEL_MANIFEST_DOES_NOT_MATCH_STRATEGY"):
        receipt._validate_strategy({"kernels": ["cake_matmul_rs_sm100<256>"]}, p2p, 8, 256)
    with pytest.raises(ValueError, match="KERNEL_MANIFEST_DOES_NOT_MATCH_STRATEGY"):
        receipt._validate_strategy({"kernels": ["cake_matmul_rs_sm100<256>", "cake_reduce_slots_sm100"]}, "nccl_reduce_scatter", 8, 256)
