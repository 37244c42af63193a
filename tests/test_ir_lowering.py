"""Schedule -> physical kernel -> CUDA plan, the IR verifiers (mutation tests in the reference's
"fail closed" style) and the cost model's known answers."""

from __future__ import annotations

import numpy as np
import pytest

from tpu_cake_b200 import cost_model, cuda_lowering, dialects, ir, schedule_lowering, workloads


def physical(mesh=8, m=128, k=1024, n=1024, **kwargs):
    return schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(mesh_size=mesh, m=m, k=k, n=n), **kwargs)


def test_schedule_lowers_to_the_sixteen_operation_kernel():
    module = physical()
    kernel = module.ops[0]
    assert [op.name for op in kernel.body.ops] == list(cuda_lowering._PHYSICAL_MATMUL_OPS)
    assert kernel.properties["target"] == "b200"
    matmul = kernel.body.ops[11]
    assert (matmul.properties["tile_m"], matmul.properties["tile_k"], matmul.properties["tile_n"]) == (128, 128, 1024)
    collective = kernel.body.ops[12]
    assert collective.properties["group_size"] == 8 and collective.properties["split_dimension"] == 1
    assert collective.properties["collective_plan"] == "axis:t" and "implementation" not in collective.properties


def test_canonical_text_is_stable_and_ignores_names_and_locations():
    first = workloads.distributed_matmul_schedule(mesh_size=8, m=128, k=1024, n=1024)
    second = workloads.distributed_matmul_schedule(mesh_size=8, m=128, k=1024, n=1024)
    second.ops[0].properties["sym_name"] = "renamed"
    second.ops[0].body.ops[0].location = ir.SourceLocation("elsewhere.py", 9, 9)
    assert ir.schedule_sha256(first) == ir.schedule_sha256(second)
    other = workloads.distributed_matmul_schedule(mesh_size=4, m=128, k=1024, n=1024)
    assert ir.schedule_sha256(first) != ir.schedule_sha256(other)
    text = ir.canonical_text(physical())
    assert '"tpu_schedule.mxu_matmul"' in text and 'role = "alloc0"' in text and "lhs_tile" not in text


def test_lowered_plan_matches_reference_fields():
    module = physical(tile=schedule_lowering.MatmulTile(128, 256), collective_implementation=dialects.CollectiveImplementation.P2P_OWNER_PUSH)
    plan = cuda_lowering.lower_physical_matmul_to_cuda(module)
    assert plan.schedule_sha256 == ir.schedule_sha256(module)
    assert plan.lhs_local_shape == (128, 128) and plan.rhs_local_shape == (128, 1024)
    assert plan.partial_local_shape == (128, 1024) and plan.output_local_shape == (128, 128)
    assert plan.output_sharding == ("", "t") and plan.scatter_dimension == 1
    assert (plan.tile_m, plan.tile_k, plan.tile_n) == (128, 128, 256)
    assert plan.collective_implementation is cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE
    assert plan.collective_link_bandwidths == (("t", 900_000_000_000),)
    along_m = schedule_lowering.lower_distributed_matmul(
        workloads.distributed_matmul_schedule(mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension="M"),
        tile=schedule_lowering.MatmulTile(128, 256),
    )
    big = cuda_lowering.lower_physical_matmul_to_cuda(along_m, output_dtype="bf16")
    assert big.output_local_shape == (1024, 8192) and big.scatter_dimension == 0 and big.output_dtype == "bf16"


def test_lowering_rejects_other_programs_with_operation_name_in_message():
    module = workloads.distributed_matmul_schedule(mesh_size=4)
    module.ops[0].body.ops[1].properties["reducer"] = "max"
    with pytest.raises((schedule_lowering.UnsupportedLoweringError, ir.VerifyException)):
        schedule_lowering.lower_distributed_matmul(module)
    module = workloads.distributed_matmul_schedule(mesh_size=4)
    del module.ops[0].body.ops[1]
    with pytest.raises((schedule_lowering.UnsupportedLoweringError, ir.VerifyException)):
        schedule_lowering.lower_distributed_matmul(module)
    with pytest.raises(cuda_lowering.UnsupportedLoweringError, match="tiles"):
        cuda_lowering.lower_physical_matmul_to_cuda(physical(tile=schedule_lowering.MatmulTile(64, 128)))


@pytest.mark.parametrize(
    "mutate, fragment",
    [
        (lambda k: k.body.ops[11].properties.__setitem__("tile_k", 64), "tile_k must equal"),
        (lambda k: k.body.ops[11].properties.__setitem__("tile_m", 96), "tiles must be positive and divide"),
        (lambda k: k.body.ops[12].properties.__setitem__("group_size", 1), "group_size must exceed 1"),
        (lambda k: k.body.ops[12].properties.__setitem__("split_dimension", 0), "destination must be"),
        (lambda k: k.body.ops.pop(14), "every DMA must be waited on"),
        (lambda k: k.body.ops[8].operands.__setitem__(2, k.body.ops[7].operands[2]), "semaphore reused"),
        (lambda k: k.properties.__setitem__("vmem_capacity_bytes", 1024), "exceed the capacity"),
        (lambda k: k.body.ops[11].properties.__setitem__("stage", 4), "not live at stage"),
    ],
)
def test_physical_verifier_fails_closed(mutate, fragment):
    module = physical()
    mutate(module.ops[0])
    with pytest.raises(ir.VerifyException, match=fragment):
        module.verify()


def test_logical_verifier_fails_closed():
    with pytest.raises(ir.VerifyException, match="not divisible"):
        workloads.distributed_matmul_schedule(mesh_size=3, m=16, k=32, n=16)
    module = workloads.distributed_matmul_schedule(mesh_size=4)
    module.ops[0].body.ops[0].properties["contracting_dimension"] = "M"
    with pytest.raises(ir.VerifyException, match="contracting dimension"):
        module.verify()


def test_cost_model_known_answers():
    """The reference's integers for mesh 8, 128 x 1024 x 1024 (its tests/test_cost_model.py:31-34)."""
    plan = cuda_lowering.lower_physical_matmul_to_cuda(physical())
    counts = cost_model.matmul_counts(plan)
    assert counts.operations_per_device == 33_554_432
    assert counts.hbm_read_bytes_per_device == 819_200
    assert counts.hbm_write_bytes_per_device == 589_824
    assert counts.ici_bidirectional_bytes_per_device == 917_504
    report = cost_model.estimate_distributed_matmul(plan)
    assert report.limiting_resource == "ici" and report.lower_bound_ns == report.communication_ns
    big = cuda_lowering.plan_distributed_matmul(
        mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension=0, output_dtype="bf16",
        collective_implementation=cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT,
    )
    big_report = cost_model.estimate_distributed_matmul(big)
    assert big_report.counts.operations_per_device == 2 * 8192 * 2048 * 8192
    assert big_report.counts.link_egress_bytes_per_device == 117_440_512
    assert big_report.limiting_resource == "compute"
    assert abs(float(big_report.compute_ns) - 168_756.0) < 1_000.0


def test_rpa_cost_convention_matches_bench_bytes():
    lengths, _ = workloads.decode_metadata(workloads.DECODE_64)
    counts = cost_model.estimate_rpa_decode(lengths, q_heads=32, kv_heads=8, head_dim=128, page_size=16)
    assert counts.hbm_bytes == workloads.decode_algorithmic_bytes(lengths, 32, 8, 128, 16)
    assert counts.flops == 4 * 128 * 32 * int(np.asarray(lengths, dtype=np.int64).sum())


# ------------------------------------------------------------------------------------ RPA op types


def test_prototype_attention_op_verifies_and_lowers():
    from tpu_cake_b200 import rpa_cuda_lowering

    module = workloads.paged_attention_schedule(batch=4, q_heads=8, kv_heads=2, head_dim=128, pages=32, page_size=16, max_pages=8)
    plan = rpa_cuda_lowering.lower_paged_attention_to_cuda(module)
    assert plan.query_shape == (4, 8, 128) and plan.cache_shape == (32, 16, 2, 128)
    assert plan.page_table_shape == (4, 8) and plan.bias_shape == (8, 128) and plan.softmax_scale == 1.0 / 128
    assert len(plan.schedule_sha256) == 64 and plan.source_sha256() != plan.schedule_sha256
    toy = workloads.paged_attention_schedule()  # the reference's toy shape: verifies, head_dim 32 is not lowered
    with pytest.raises(rpa_cuda_lowering.UnsupportedRpaLowering, match="head_dim 128"):
        rpa_cuda_lowering.lower_paged_attention_to_cuda(toy)


@pytest.mark.parametrize(
    "kwargs, message",
    [
        ({"q_heads": 6, "kv_heads": 4}, "divide evenly"),
        ({"max_pages": 16}, None),  # bias extent follows max_pages: still valid
    ],
)
def test_prototype_attention_op_rules(kwargs, message):
    if message is None:
        workloads.paged_attention_schedule(**kwargs)
        return
    with pytest.raises(ir.VerifyException, match=message):
        workloads.paged_attention_schedule(**kwargs)


def test_fused_attention_op_strict_and_cuda_authorities():
    from tpu_cake_b200 import dialects, rpa_cuda_lowering

    shape = dict(q_heads=8, kv_heads=4, head_dim=128, pages=3712, page_size=1, page_indices=8192)
    strict = workloads.fused_rpa_schedule(tokens=4, **shape)
    plan = rpa_cuda_lowering.lower_fused_rpa_to_cuda(strict)
    assert isinstance(plan, rpa_cuda_lowering.CudaFusedRpaPlan) and plan.softmax_scale == 1.0 / 128
    assert plan.relative_states_shape == (4, 8, 16) and plan.relative_projection_shape == (16, 512)
    # The reference's authority refuses another scale and ragged query runs ...
    with pytest.raises(ir.VerifyException, match="must equal 1 / head dimension"):
        workloads.fused_rpa_schedule(tokens=4, softmax_scale="0.088388", execution_authority=dialects.FUSED_RPA_UPSTREAM_AUTHORITY, **shape)
    with pytest.raises(ir.VerifyException, match="one query token per sequence"):
        workloads.fused_rpa_schedule(tokens=40, sequences=4, execution_authority=dialects.FUSED_RPA_UPSTREAM_AUTHORITY, **shape)
    with pytest.raises(ir.VerifyException, match="delegated execution authority"):
        workloads.fused_rpa_schedule(tokens=4, execution_authority="someone-else", **shape)
    # ... this backend's authority takes both.
    ragged = workloads.fused_rpa_schedule(tokens=40, sequences=4, softmax_scale="0.088388", **shape)
    mixed = rpa_cuda_lowering.lower_fused_rpa_to_cuda(ragged)
    assert isinstance(mixed, rpa_cuda_lowering.CudaMixedRpaPlan) and mixed.sequences == 4 and mixed.query_shape == (40, 8, 128)
    assert abs(mixed.softmax_scale - 0.088388) < 1e-12


def test_cuda_decode_resource_contract_op():
    from tpu_cake_b200 import dialects, rpa_cuda_lowering

    module = workloads.paged_attention_schedule(batch=4, q_heads=8, kv_heads=2, head_dim=128)
    plan = rpa_cuda_lowering.lower_paged_attention_to_cuda(module)
    contract = rpa_cuda_lowering.decode_resource_contract(plan)
    assert contract["shared_memory_bytes"] == 6 * (2 * 32 * 512 + 2048) + 1280 <= dialects.B200_SHARED_MEMORY_PER_CTA
    kernel = module.ops[0]
    attention = next(op for op in kernel.body.ops if op.name == "tpu_schedule.ragged_paged_attention")
    good = ir.Operation("tpu_schedule.cuda_rpa_decode", list(attention.operands), [],
                        {"stage": 2, "attention": attention.name, "backend": "cake-b200/sm_100a", **contract})
    dialects.verify_operation(good)
    bad = ir.Operation("tpu_schedule.cuda_rpa_decode", list(attention.operands), [],
                       {"stage": 2, "attention": attention.name, "backend": "cake-b200/sm_100a", **{**contract, "kv_chunk_tokens": 48}})
    with pytest.raises(ir.VerifyException, match="multiple of the stage size"):
        dialects.verify_operation(bad)
    wrong_bytes = ir.Operation("tpu_schedule.cuda_rpa_decode", list(attention.operands), [],
                               {"stage": 2, "attention": attention.name, "backend": "cake-b200/sm_100a", **{**contract, "shared_memory_bytes": 4096}})
    with pytest.raises(ir.VerifyException, match="shared_memory_bytes must be"):
        dialects.verify_operation(wrong_bytes)


def _gather_kernel(*, source_sharding=("", "t", ""), destination_shape=(256, 64, 128), destination_sharding=("", "", ""), reducer=None,
                   implementation=dialects.CollectiveImplementation.P2P_PEER_STORE):
    """The sharded decode's collective on its own: every rank's [256, 8, 128] output rows gathered
    along the head dimension over an 8-way axis."""
    builder = dialects.KernelBuilder("gather", "b200", (), vmem_capacity_bytes=1 << 30, smem_capacity_bytes=232448, mesh={"t": 8},
                                     interconnect_bandwidth_bytes_per_second={"t": 900_000_000_000})
    local = builder.alloc(dialects.buffer((256, 8, 128), ("B", "H", "D"), "bf16", memory="vmem", sharding=source_sharding, lifetime=(0, 1)), "local_output")
    gathered = builder.alloc(dialects.buffer(destination_shape, ("B", "H", "D"), "bf16", memory="vmem", sharding=destination_sharding, lifetime=(0, 1)), "gathered_output")
    op = builder.collective_all_gather(local, gathered, stage=0, mesh_axis="t", group_size=8, concat_dimension=1, implementation=implementation)
    if reducer is not None:
        op.properties["reducer"] = reducer
    return builder


def test_all_gather_collective_rules():
    """The all-gather the KV-head-sharded decode ends with is expressible, carried by peer stores or
    NCCL, with the reference's rules (src/tpu_cake/dialects/tpu_schedule.py:1914-1923): one concat
    dimension, no reducer, the mesh axis leaves the gathered dimension, the extent grows by the group."""
    module = _gather_kernel().module()
    collective = module.ops[0].body.ops[2]
    assert collective.properties["kind"] == "all_gather" and collective.properties["implementation"] == "p2p_peer_store"
    assert '"tpu_schedule.collective"' in ir.canonical_text(module)
    _gather_kernel(implementation=dialects.CollectiveImplementation.NCCL).module()
    for kwargs, message in (
        ({"source_sharding": ("", "", "")}, "must remove its mesh axis"),
        ({"destination_shape": (256, 8, 128)}, "destination must be"),
        ({"destination_sharding": ("", "t", "")}, "must be sharded over"),
        ({"reducer": "sum"}, "no reducer"),
        ({"implementation": dialects.CollectiveImplementation.P2P_OWNER_PUSH}, "NCCL or by peer stores"),
    ):
        with pytest.raises(ir.VerifyException, match=message):
            _gather_kernel(**kwargs).module()


def test_generic_physical_cost_model():
    """The static report of a physical kernel: for the matmul kernel it reproduces the closed-form
    counts (the reference's known integers for mesh 8, 128 x 1024 x 1024: ring-equivalent bytes
    917,504, 2 * 128 * 128 * 1024 FLOP), for the attention kernels it prices the declared capacity,
    and an over-full on-chip budget or an unknown operation is refused."""
    from decimal import Decimal

    from tpu_cake_b200 import physical_cost_model

    module = physical(collective_implementation=dialects.CollectiveImplementation.P2P_OWNER_PUSH_BF16)
    report = physical_cost_model.analyze_physical_kernel(module)
    plan = cuda_lowering.lower_physical_matmul_to_cuda(module)
    closed_form = cost_model.estimate_distributed_matmul(plan)
    region = report.mxu_regions[0]
    assert (region.m, region.k, region.n, region.flops) == (128, 128, 1024, 2 * 128 * 128 * 1024) == (128, 128, 1024, closed_form.counts.operations_per_device)
    collective = report.collectives[0]
    assert collective.ring_equivalent_bidirectional_bytes_per_device == Decimal(closed_form.counts.ici_bidirectional_bytes_per_device) == Decimal(917504)
    assert collective.switch_egress_bytes_per_device == Decimal(closed_form.counts.link_egress_bytes_per_device)
    assert report.priced_compute_time_floor_ns == closed_form.compute_ns and report.priced_ici_time_floor_ns == closed_form.communication_ns
    assert report.memory.explicit_hbm_dma_read_bytes_per_device == 2 * (128 * 128 + 128 * 1024)
    assert report.memory.peak_live_vmem_bytes_per_device <= report.resource_peaks[0].capacity and report.device_count == 8
    assert dict(report.canonical_operation_inventory)["tpu_schedule.dma_start"] == 3 and len(report.stages) == 6
    sharded = physical_cost_model.analyze_physical_kernel(workloads.inkling_sharded_rpa_schedule())
    work = sharded.attention[0]
    assert (work.sequences, work.q_heads, work.kv_heads, work.token_capacity) == (4, 8, 4, 3712)
    assert sharded.predicted_limiting_priced_resource == "hbm" and "upper bound" in " ".join(sharded.assumptions)
    assert isinstance(sharded.to_json()["priced_hbm_time_floor_ns"], str)
    gather = _gather_kernel().module()
    traffic = physical_cost_model.analyze_physical_kernel(gather).collectives[0]
    assert traffic.kind == "all_gather" and traffic.payload_bytes_per_device == 256 * 64 * 128 * 2
    bad = physical()
    bad.ops[0].body.ops[11].name = "tpu_schedule.vector_compute"
    with pytest.raises((physical_cost_model.UnsupportedPhysicalCostModelError, ir.VerifyException)):
        physical_cost_model.analyze_physical_kernel(bad)
