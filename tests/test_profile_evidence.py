"""The ncu reader's acceptance rules (the reference's XProf rules on GPU captures)."""

from __future__ import annotations

from tpu_cake_b200.profile_evidence import ProfileExpectation, assess_capture, assess_evidence, read_ncu_csv

HEADER = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'


def row(launch, kernel, device, metric, unit, value):
    return f'"{launch}","1","python","h","{kernel}","1","7","(192, 1, 1)","(148, 1, 1)","{device}","10.0","s","{metric}","{unit}","{value}"\n'


def capture(rows):
    return read_ncu_csv("==PROF== Connected\n" + HEADER + "".join(rows))


GEMM = "void cake::cake_matmul_rs_sm100<256, 0>(CUtensorMap_st, CUtensorMap_st, cake::OwnerMaps, cake::MatmulParams)"
GOOD = [
    row(0, GEMM, 0, "gpu__time_duration.sum", "us", "1,476.2"),
    row(0, GEMM, 0, "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "%", "87.0"),
    row(0, GEMM, 0, "dram__bytes_read.sum", "Gbyte", "2.9"),
    row(1, "void cake::cake_reduce_slots_sm100<__nv_bfloat16, __nv_bfloat16>(...)", 0, "gpu__time_duration.sum", "us", "40"),
]
EXPECT = ProfileExpectation(name="matmul-p2p", required_timed_hlo_markers=("cake_matmul_rs_sm100", "cake_reduce_slots_sm100"),
                            forbidden_timed_hlo_fragments=("ncclDevKernel_ReduceScatter",), require_hbm_read_counters=True)


def test_good_capture_is_accepted_and_timed():
    assessment = assess_evidence(capture(GOOD), EXPECT)
    assert assessment.accepted and assessment.findings == ()
    assert assessment.marker_launches == {"cake_matmul_rs_sm100": 1, "cake_reduce_slots_sm100": 1}
    assert abs(assessment.marker_time_ns["cake_matmul_rs_sm100"] - 1_476_200.0) < 1.0


def test_rejections_mirror_the_reference_rules():
    def codes(rows, expectation=EXPECT):
        return {f.code for f in assess_evidence(capture(rows), expectation).findings}

    assert "REQUIRED_TIMED_MARKER_MISSING" in codes(GOOD[:3])
    assert "NO_TENSOR_CORE_ACTIVITY" in codes([GOOD[0], GOOD[2], GOOD[3]])
    assert "MISSING_HBM_READ_COUNTERS" in codes([GOOD[0], GOOD[1], GOOD[3]])
    assert "FORBIDDEN_TIMED_FRAGMENT_PRESENT" in codes(GOOD + [row(2, "ncclDevKernel_ReduceScatter_Sum_f32_RING_LL(...)", 0, "gpu__time_duration.sum", "us", "300")])
    eight = ProfileExpectation(name="eight", minimum_tpu_device_planes=8, require_tensor_core_activity=False)
    assert "INSUFFICIENT_GPU_DEVICES" in codes(GOOD, eight)
    pinned = ProfileExpectation(name="count", required_timed_hlo_markers=("cake_matmul_rs_sm100",), expected_marker_launches=3)
    assert "MARKER_LAUNCH_COUNT_MISMATCH" in codes(GOOD, pinned)
    empty = assess_evidence(capture([]), ProfileExpectation(name="empty", require_tensor_core_activity=False))
    assert {f.code for f in empty.findings} == {"INSUFFICIENT_GPU_DEVICES", "INSUFFICIENT_DEVICE_EVENTS"}


def test_unreadable_capture_is_a_rejection(tmp_path):
    missing = assess_capture(tmp_path / "nope.csv", EXPECT)
    assert not missing.accepted and missing.findings[0].code == "PROFILE_CAPTURE_UNREADABLE"
    (tmp_path / "garbage.csv").write_text("not,a,capture\n1,2,3\n")
    assert not assess_capture(tmp_path / "garbage.csv", EXPECT).accepted


def test_real_launch_list_of_the_bench(golden_dir):
    expectation = ProfileExpectation(
        name="bench-launch-list", require_tensor_core_activity=False,
        required_timed_hlo_markers=("cake_matmul_rs_sm100", "cake_rpa_decode_sm100", "cake_rpa_plan_sm100"),
        forbidden_timed_hlo_fragments=("ncclDevKernel",),
    )
    assessment = assess_capture(golden_dir / "ncu_launch_list_bench.csv", expectation)
    assert assessment.accepted, assessment.findings
    assert assessment.marker_launches["cake_rpa_decode_sm100"] >= 1
    per_launch_us = assessment.marker_time_ns["cake_rpa_decode_sm100"] / assessment.marker_launches["cake_rpa_decode_sm100"] / 1e3
    assert 100 < per_launch_us < 400
