"""The canonical text of physical kernels is the reference's, byte for byte.

Known answers: the schedule hashes the reference pins in its own tests and sources for programs
that can be rebuilt here from their definitions. xDSL is not installed, so these SHA-256 values are
the only witness of the exact bytes -- and a sufficient one.
"""

from __future__ import annotations

import pytest

from tpu_cake_b200 import ir, schedule_lowering, workloads, xdsl_text
from tpu_cake_b200.dialects import KernelBuilder, buffer
from tpu_cake_b200.ir import Operation

TPU7X = schedule_lowering.LoweringTarget("tpu7x", 64 << 20, 16 << 20, 600_000_000_000)  # src/tpu_cake/lowering.py:47-52
EXTERNAL = {"memory": "hbm", "ownership": "external", "lifetime": (0, 0)}


def rpa_kernel(name, inputs, mesh=None, **properties):
    """KernelBuilder with the capacities of the reference's RPA schedules (96 MiB / 1 MiB)."""
    mesh = dict(mesh or {})
    builder = KernelBuilder(name, "tpu7x", inputs, vmem_capacity_bytes=96 << 20, smem_capacity_bytes=1 << 20, mesh=mesh,
                            interconnect_bandwidth_bytes_per_second={axis: 600_000_000_000 for axis in mesh})
    builder.kernel.properties.update(properties)
    return builder


def test_default_distributed_matmul_kernel_has_the_pinned_hash():
    """tests/test_pallas_lowering.py:54-60: mesh 4, 16 x 32 x 16, whole-shard tiles."""
    physical = schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(), target=TPU7X)
    assert ir.schedule_sha256(physical) == "395c5e60a6ae43e2c86b61b06271666010d79d103175cb43a4c01c9fb22a8819"
    text = ir.canonical_text(physical)
    assert text.startswith('"builtin.module"() ({\n  "tpu_schedule.kernel"() <{dma_engine_count = #builtin.int<2>, ')
    assert text.endswith('    "tpu_schedule.yield"() : () -> ()\n  }) : () -> ()\n}) : () -> ()\n')


@pytest.mark.parametrize(
    "implementation, expected",
    [(None, "9593beb3ad1607b65f12ac02cfe4bf2adbf6279405aa307f46c155e430d40990"),
     ("pallas_bidirectional_ring", "23917a172499112cebd52bb26333f11b367f1b67190546e90af847ec8b71fe97")],
)
def test_mesh8_matmul_kernels_have_the_confirmation_hashes(implementation, expected):
    """src/tpu_cake/matmul_collective_confirmation.py:42-48,87,108: mesh 8, 1024 x 65536 x 1024,
    tiles 128 x 128, with the compiler's reduce-scatter and with the ring named as implementation."""
    logical = workloads.distributed_matmul_schedule(mesh_size=8, m=1024, k=65536, n=1024)
    physical = schedule_lowering.lower_distributed_matmul(logical, target=TPU7X, tile=schedule_lowering.MatmulTile(128, 128))
    if implementation is not None:
        collective = next(op for op in physical.walk() if op.name == "tpu_schedule.collective")
        collective.properties["implementation"] = implementation
    assert ir.schedule_sha256(physical) == expected


def fused_inputs():
    return (
        buffer((4, 4, 32), "T Hq D".split(), "bf16", **EXTERNAL),
        buffer((4, 2, 32), "T Hkv D".split(), "bf16", **EXTERNAL),
        buffer((4, 2, 32), "T Hkv D".split(), "bf16", **EXTERNAL),
        buffer((32, 16, 2, 2, 128), "P S Hkv2p Pack Dpad".split(), "bf16", **EXTERNAL),
        buffer((4,), ("N",), "i32", **EXTERNAL),
        buffer((32,), ("PI",), "i32", **EXTERNAL),
        buffer((5,), ("N1",), "i32", **EXTERNAL),
        buffer((5,), ("N1",), "i32", **EXTERNAL),
        buffer((3,), ("R3",), "i32", **EXTERNAL),
        buffer((4, 4, 16), "T Hq R".split(), "bf16", **EXTERNAL),
        buffer((16, 128), "R E".split(), "bf16", **EXTERNAL),
    )


def test_fused_rpa_kernel_has_the_pinned_hash():
    """tests/test_rpa_lowering.py:140-146 over src/tpu_cake/workloads/inkling_rpa.py:145-195: a
    kernel without a mesh (one device, no links) around the fused attention operation."""
    builder = rpa_kernel("inkling_fused_rpa_decode", fused_inputs())
    builder.fused_ragged_paged_attention((*builder.inputs, builder.inputs[0], builder.inputs[3]), stage=0, softmax_scale="0.03125",
                                         vmem_limit_bytes=96 << 20)
    assert ir.schedule_sha256(builder.module()) == "e1de39a3dfa8f4c930207fbe5218aa1f956b19b0b933e993fe35ae916e8ecad7"


def test_sharded_rpa_surface_kernel_has_the_contract_hash():
    """contracts/inkling-sharded-rpa-surface.json plan.schedule_sha256 over
    src/tpu_cake/workloads/inkling_rpa.py:198-262: a 2 x 4 mesh, so the topology has two axes."""
    inputs = (
        buffer((4, 8, 128), "T Hq D".split(), "bf16", sharding=("data", "tensor", ""), **EXTERNAL),
        buffer((4, 4, 128), "T Hkv D".split(), "bf16", sharding=("data", "tensor", ""), **EXTERNAL),
        buffer((4, 4, 128), "T Hkv D".split(), "bf16", sharding=("data", "tensor", ""), **EXTERNAL),
        buffer((3712, 1, 4, 2, 128), "P S Hkv2p Pack Dpad".split(), "bf16", sharding=("data", "", "tensor", "", ""), **EXTERNAL),
        buffer((4,), ("N",), "i32", sharding=("data",), **EXTERNAL),
        buffer((8192,), ("PI",), "i32", sharding=("data",), **EXTERNAL),
        buffer((5,), ("N1",), "i32", sharding=("data",), **EXTERNAL),
        buffer((5,), ("N1",), "i32", sharding=("data",), **EXTERNAL),
        buffer((3,), ("R3",), "i32", sharding=("data",), **EXTERNAL),
        buffer((4, 8, 16), "T Hq R".split(), "bf16", sharding=("data", "tensor", ""), **EXTERNAL),
        buffer((16, 512), "R E".split(), "bf16", **EXTERNAL),
    )
    builder = rpa_kernel("inkling_sharded_fused_rpa_decode", inputs, mesh={"data": 2, "tensor": 4})
    builder.fused_ragged_paged_attention((*builder.inputs, builder.inputs[0], builder.inputs[3]), stage=0, softmax_scale="0.0078125",
                                         vmem_limit_bytes=96 << 20)
    assert ir.schedule_sha256(builder.module()) == "12007604b3b6305899bd2f13d311aa77889199fc0398a3615c142f7966572b13"


def decode_core_module():
    """src/tpu_cake/workloads/inkling_rpa.py:265-401: argument modes on the kernel, scratch in both
    on-chip spaces, a ten-slot semaphore and an operation with 26 operands and 22 properties."""
    inputs = (
        buffer((4, 4, 1, 2, 128), "Hkv T Hqp Pack Dpad".split(), "bf16", **EXTERNAL),
        buffer((4, 4, 2, 128), "T Hkv2p Pack Dpad".split(), "bf16", **EXTERNAL),
        buffer((3712, 1, 4, 2, 128), "P S Hkv2p Pack Dpad".split(), "bf16", **EXTERNAL),
        buffer((4,), ("N",), "i32", **EXTERNAL),
        buffer((8192,), ("PI",), "i32", **EXTERNAL),
        buffer((5,), ("N1",), "i32", **EXTERNAL),
        buffer((5,), ("N1",), "i32", **EXTERNAL),
        buffer((3,), ("R3",), "i32", **EXTERNAL),
        buffer((4, 4, 2, 128), "Hkv T Hqpk Rpad".split(), "bf16", **EXTERNAL),
        buffer((128, 4608), "Rpad Epad".split(), "bf16", **EXTERNAL),
    )
    builder = rpa_kernel("inkling_owned_rpa_decode_core", inputs, argument_modes=("inout", "input", "inout", *("input",) * 7))
    vmem = {"memory": "vmem", "lifetime": (0, 0)}
    smem = {"memory": "smem", "lifetime": (0, 0)}
    scratch = [
        builder.alloc(buffer((4, 4, 2, 128), "Hkv T Hqpk Rpad".split(), "bf16", **vmem), "relative_states_resident"),
        builder.alloc(buffer((128, 4608), "Rpad Epad".split(), "bf16", **vmem), "relative_projection_resident"),
        builder.alloc(buffer((2, 128, 5, 2, 128), "Slot Bkv Hkv2pPad Pack Dpad".split(), "bf16", **vmem), "paged_kv_double_buffer"),
        builder.alloc(buffer((2, 4, 8, 1, 2, 128), "Slot Hkv Bq Hqp Pack Dpad".split(), "bf16", **vmem), "query_double_buffer"),
        builder.alloc(buffer((2, 4, 8, 1, 2, 128), "Slot Hkv Bq Hqp Pack Dpad".split(), "bf16", **vmem), "output_double_buffer"),
        builder.alloc(buffer((4, 16, 128), "Hkv QH Lane".split(), "bf16", **vmem), "online_softmax_l"),
        builder.alloc(buffer((4, 16, 128), "Hkv QH Lane".split(), "bf16", **vmem), "online_softmax_m"),
        builder.alloc(buffer((4, 16, 128), "Hkv QH Dpad".split(), "bf16", **vmem), "attention_accumulator"),
        builder.alloc(buffer((4, 8, 2, 256, 4), "Hkv Bq Hq KVD Work".split(), "f32", **vmem), "compiler_attention_intermediates"),
        builder.alloc(buffer((1,), ("One",), "i32", **smem), "cumulative_mask_lengths"),
        builder.alloc(buffer((3,), ("SemId",), "i32", **smem), "semaphore_ids"),
        builder.alloc(buffer((4,), ("OutputId",), "i32", **smem), "output_ids"),
        builder.alloc(buffer((6,), ("UpdateId",), "i32", **smem), "cache_update_ids"),
    ]
    semaphores = builder.semaphore()
    semaphores.owner.properties["slots"] = 10
    properties = {
        "stage": 0, "query_fetch_size": 8, "kv_fetch_size": 128, "query_compute_size": 8, "kv_compute_size": 128, "buffer_slots": 2,
        "dma_channels": 5, "prefetch_distance": 1, "relative_extent": 512, "softmax_scale": "0.0078125", "softmax_dtype": "float32",
        "execution_authority": "tpu-cake-owned-pallas-decode-core-v1", "attention_case": "decode",
        "masking_authority": "decode-kv-length-no-custom-mask-v1", "relative_dimension": 16, "cumulative_mask_initial": (0,),
        "semaphore_ids_initial": (0, 0, 0), "output_ids_initial": (-1,) * 4, "cache_update_ids_initial": (-1,) * 6,
        # src/tpu_cake/rpa_lowering.py:54-58
        "backend_repository_revision": "9e1a7d39ccdcf9f396e024bfc45935f4f50f70c7",
        "backend_file_revision": "ac88a2ecfa905965b43edbbb5e6510eb272d09e5",
        "backend_sha256": "12c6aeeade66538d3bb638f048850c3d69095ade4ec42559cd8b3566bfc68897",
    }
    builder.block.ops.append(Operation("tpu_schedule.rpa_decode_core", [*builder.inputs, builder.inputs[0], builder.inputs[2], *scratch, semaphores],
                                       [], properties))
    return builder.module()


def test_owned_decode_core_kernel_has_the_pinned_hash():
    """tests/test_rpa_lowering.py:223-228 and :342-344."""
    assert ir.schedule_sha256(decode_core_module()) == "41946eb01074fd2ecd2831190321631f09d9c25fb7c3ee68a28ebc272f6d576a"


def every_kernel():
    yield schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(), target=TPU7X)
    yield schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension="M"),
                                                     tile=schedule_lowering.MatmulTile(128, 256), collective_implementation="p2p_owner_push_bf16")
    yield workloads.inkling_fused_rpa_schedule()
    yield workloads.inkling_sharded_rpa_schedule()
    yield workloads.paged_attention_schedule()
    yield decode_core_module()


def test_saved_text_parses_back_to_the_same_bytes_and_verifies():
    for module in every_kernel():
        text = ir.canonical_text(module)
        parsed = xdsl_text.parse_reference_physical_kernel(text)
        assert ir.canonical_text(parsed) == text
        parsed.verify()
        assert [op.name for op in parsed.walk()] == [op.name for op in module.walk()]


def test_text_that_would_not_print_back_is_refused():
    text = ir.canonical_text(schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(), target=TPU7X))
    with pytest.raises(ValueError, match="XDSL_TEXT_NOT_CANONICAL"):
        # properties out of order: xDSL would accept it, the canonical form does not contain it
        xdsl_text.parse_reference_physical_kernel(text.replace("dma_engine_count = #builtin.int<2>, ici_link_count = #builtin.int<1>",
                                                               "ici_link_count = #builtin.int<1>, dma_engine_count = #builtin.int<2>"))
    with pytest.raises(ValueError, match="XDSL_TEXT_UNSUPPORTED_ENGINE_COUNT property=mxu_count"):
        xdsl_text.parse_reference_physical_kernel(text.replace("mxu_count = #builtin.int<1>", "mxu_count = #builtin.int<2>"))
    with pytest.raises(ValueError, match="XDSL_TEXT_UNSUPPORTED_LAYOUT"):
        xdsl_text.parse_reference_physical_kernel(text.replace("#tpu_schedule.layout<[#builtin.int<0>, #builtin.int<1>]>",
                                                               "#tpu_schedule.layout<[#builtin.int<1>, #builtin.int<0>]>", 1))
    with pytest.raises(ValueError, match="XDSL_TEXT_UNDEFINED_VALUE value=%99"):
        xdsl_text.parse_reference_physical_kernel(text.replace('"tpu_schedule.dma_wait"(%10)', '"tpu_schedule.dma_wait"(%99)'))
    with pytest.raises(ValueError, match="XDSL_TEXT_PARSE_ERROR line=1"):
        xdsl_text.parse_reference_physical_kernel("module {}\n")
    with pytest.raises(ValueError, match="XDSL_TEXT_UNSUPPORTED_OPERATION operation=tpu_schedule.vector_compute"):
        xdsl_text.parse_reference_physical_kernel(text.replace('"tpu_schedule.dma_wait"(%10)', '"tpu_schedule.vector_compute"(%10)'))


def test_a_parsed_kernel_that_breaks_a_dialect_rule_fails_verification():
    text = ir.canonical_text(schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(), target=TPU7X))
    broken = text.replace("tile_k = #builtin.int<8>", "tile_k = #builtin.int<4>")
    module = xdsl_text.parse_reference_physical_kernel(broken)
    with pytest.raises(ir.VerifyException):
        module.verify()


def test_verify_schedule_command_accepts_a_saved_physical_text(tmp_path, capsys):
    from tpu_cake_b200 import cli

    physical = schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(), target=TPU7X)
    path = tmp_path / "physical.xdsl"
    path.write_text(ir.canonical_text(physical))
    assert cli.main(["verify-schedule", str(path)]) == 0
    assert capsys.readouterr().out.strip() == (
        f"SCHEDULE_ACCEPTED path={path} schedule_sha256=395c5e60a6ae43e2c86b61b06271666010d79d103175cb43a4c01c9fb22a8819"
    )


def test_physical_cost_commands_work_from_a_saved_kernel(tmp_path, capsys):
    """estimate-physical-cost / verify-physical-cost (src/tpu_cake/cli.py:439-469): the report is
    derived from the saved text alone, and a report that was edited is refused."""
    import json

    from tpu_cake_b200 import cli

    physical = schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule(mesh_size=8, m=128, k=1024, n=1024))
    schedule = tmp_path / "physical.xdsl"
    schedule.write_text(ir.canonical_text(physical))
    report = tmp_path / "cost.json"
    assert cli.main(["estimate-physical-cost", str(schedule), "--output", str(report)]) == 0
    derived = capsys.readouterr().out
    assert derived.startswith(f"PHYSICAL_COST_DERIVED schedule_sha256={ir.schedule_sha256(physical)} mxu_regions=1 ")
    assert cli.main(["verify-physical-cost", str(report), "--schedule", str(schedule)]) == 0
    assert capsys.readouterr().out == derived.replace("PHYSICAL_COST_DERIVED", "PHYSICAL_COST_REPLAYED")
    document = json.loads(report.read_text())
    document["device_count"] += 1
    report.write_text(json.dumps(document))
    with pytest.raises(ValueError, match="PHYSICAL_COST_REPORT_MISMATCH"):
        cli.main(["verify-physical-cost", str(report), "--schedule", str(schedule)])


def test_logical_program_prints_in_the_reference_syntax():
    """No hash of a logical program is pinned by the reference, so this checks the shape the
    dialect definitions prescribe (src/tpu_cake/dialects/distributed_tensor.py:55-160,1020-1043,
    1202-1226,1437-1447): one mesh property, structured tensor types, sorted properties."""
    text = ir.canonical_text(workloads.distributed_matmul_schedule(mesh_size=8, m=128, k=1024, n=1024))
    lines = text.splitlines()
    assert lines[1] == '  "dtensor.program"() <{mesh = #dtensor.mesh<["t"], [#builtin.int<8>]>, sym_name = "program"}> ({'
    lhs = ('!dtensor.tensor<bf16, [#dtensor.dimension<"M", #builtin.int<128>>, #dtensor.dimension<"K", #builtin.int<1024>>], '
           '#dtensor.sharding<[#dtensor.axis_list<[]>, #dtensor.axis_list<["t"]>]>, #dtensor.pending_reductions<[], []>>')
    assert lines[2].startswith(f"  ^bb0(%0: {lhs}, %1: !dtensor.tensor<bf16, ")
    assert lines[3].startswith('    %2 = "dtensor.einsum_local"(%0, %1) <{accumulation_type = f32, contracting_dimension = "K"}> : (')
    assert lines[3].endswith('#dtensor.pending_reductions<["t"], ["sum"]>>')
    assert lines[4].startswith('    %3 = "dtensor.reduce_scatter"(%2) <{axes = ["t"], reducer = "sum", scatter_dimensions = ["N"]}> : (')
    assert lines[5].startswith('    "dtensor.return"(%3) : (') and lines[5].endswith(") -> ()")
    assert lines[6:] == ["  }) : () -> ()", "}) : () -> ()"]


def test_logical_program_parses_back_and_lowers_to_the_same_kernel(tmp_path, capsys):
    from tpu_cake_b200 import cli

    logical = workloads.distributed_matmul_schedule(mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension="M")
    text = ir.canonical_text(logical)
    parsed = xdsl_text.parse_reference_module(text)
    parsed.verify()
    assert ir.canonical_text(parsed) == text
    assert ir.schedule_sha256(schedule_lowering.lower_distributed_matmul(parsed)) == ir.schedule_sha256(schedule_lowering.lower_distributed_matmul(logical))
    path = tmp_path / "distributed.xdsl"
    path.write_text(text)
    assert cli.main(["verify-schedule", str(path)]) == 0
    assert capsys.readouterr().out.startswith(f"SCHEDULE_ACCEPTED path={path} schedule_sha256={ir.schedule_sha256(logical)}")
    with pytest.raises(ValueError, match="XDSL_TEXT_UNSUPPORTED_ACCUMULATION accumulation_type=bf16"):
        xdsl_text.parse_reference_module(text.replace("accumulation_type = f32", "accumulation_type = bf16"))
    # a sharding the mesh does not have: well-formed text, refused by the dialect's verifier
    broken = xdsl_text.parse_reference_module(text.replace('#dtensor.mesh<["t"]', '#dtensor.mesh<["u"]'))
    with pytest.raises(ir.VerifyException):
        broken.verify()


def test_damaged_text_is_refused_or_is_another_canonical_schedule():
    """A truncation, a deleted character or a stray bracket or quote in a saved schedule either ends
    in ValueError (never in another exception) or -- when it only changed a name or a number -- gives
    a text that is itself canonical, i.e. prints back to exactly those bytes."""
    refused = accepted = 0
    for text in (ir.canonical_text(schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule())),
                 ir.canonical_text(workloads.distributed_matmul_schedule())):
        for cut in range(0, len(text) - 1, 11):
            for damaged in (text[:cut], text[:cut] + text[cut + 1:], text[:cut] + "<" + text[cut:], text[:cut] + '"' + text[cut:]):
                try:
                    module = xdsl_text.parse_reference_module(damaged)
                except ValueError:
                    refused += 1
                    continue
                accepted += 1
                assert ir.canonical_text(module) == damaged
    assert refused > 20 * accepted > 0


def test_schedules_written_by_the_reference_lower_to_cuda_plans_with_its_hashes():
    """The drop-in in one step: the text the reference writes for its own tpu7x kernels (the pinned
    hashes above say these are those bytes) is parsed, verified and lowered by this backend, and the
    plan carries the schedule hash the reference computed."""
    from tpu_cake_b200 import cuda_lowering, rpa_cuda_lowering

    logical = workloads.distributed_matmul_schedule(mesh_size=8, m=1024, k=65536, n=1024)
    kernel = schedule_lowering.lower_distributed_matmul(logical, target=TPU7X, tile=schedule_lowering.MatmulTile(128, 128))
    parsed = xdsl_text.parse_reference_module(ir.canonical_text(kernel))
    parsed.verify()
    plan = cuda_lowering.lower_physical_matmul_to_cuda(parsed)
    assert plan.schedule_sha256 == "9593beb3ad1607b65f12ac02cfe4bf2adbf6279405aa307f46c155e430d40990"
    assert (plan.mesh_size, plan.lhs_local_shape, plan.rhs_local_shape, plan.output_local_shape) == (8, (1024, 8192), (8192, 1024), (1024, 128))
    assert (plan.tile_m, plan.tile_k, plan.tile_n, plan.scatter_dimension) == (128, 8192, 128, 1)
    assert plan.collective_link_bandwidths == (("t", 600_000_000_000),)

    builder = rpa_kernel("inkling_fused_rpa_decode", fused_inputs())
    builder.fused_ragged_paged_attention((*builder.inputs, builder.inputs[0], builder.inputs[3]), stage=0, softmax_scale="0.03125",
                                         vmem_limit_bytes=96 << 20)
    parsed = xdsl_text.parse_reference_module(ir.canonical_text(builder.module()))
    parsed.verify()
    rpa_plan = rpa_cuda_lowering.lower_inkling_rpa_to_cuda(parsed)
    assert rpa_plan.schedule_sha256 == "e1de39a3dfa8f4c930207fbe5218aa1f956b19b0b933e993fe35ae916e8ecad7"
    assert rpa_plan.query_shape == (4, 4, 32)


def test_a_saved_schedule_names_the_run_that_reproduces_it():
    """run-matmul --from-physical: the arguments read from a saved kernel regenerate that kernel
    byte for byte, for a kernel of this backend (b200 target, an implementation named) and for one
    the reference wrote (tpu7x target, none named); the invocation record replays the same plan."""
    from tpu_cake_b200 import runner

    own = schedule_lowering.lower_distributed_matmul(
        workloads.distributed_matmul_schedule(mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension="M"),
        tile=schedule_lowering.MatmulTile(128, 256), collective_implementation="p2p_owner_push_bf16")
    theirs = schedule_lowering.lower_distributed_matmul(
        workloads.distributed_matmul_schedule(mesh_size=8, m=1024, k=65536, n=1024), target=TPU7X, tile=schedule_lowering.MatmulTile(128, 128))
    for kernel, strategy, declared in ((own, "p2p_fused_epilogue_bf16_transport", True), (theirs, "nccl_reduce_scatter", False)):
        import tempfile
        from pathlib import Path

        with tempfile.TemporaryDirectory() as folder:
            path = Path(folder) / "physical.xdsl"
            path.write_text(ir.canonical_text(kernel))
            what = runner.invocation_of_saved_schedule(path)
        assert what["collective_strategy"] == strategy and what["declare_implementation"] is declared
        assert what["expected_schedule_sha256"] == ir.schedule_sha256(kernel)
        invocation = {**what, "tile": [what["tile"].m, what["tile"].n], "output_dtype": "f32"}
        _, physical, plan = runner.lower_invocation(invocation)
        assert ir.canonical_text(physical) == ir.canonical_text(kernel)
        assert plan.schedule_sha256 == what["expected_schedule_sha256"]
    assert what["target"] == {"name": "tpu7x", "vmem_capacity_bytes": 64 << 20, "smem_capacity_bytes": 16 << 20,
                              "ici_bandwidth_bytes_per_second": 600_000_000_000}
    assert (what["mesh_size"], what["m"], what["k"], what["n"], what["scatter_dimension"]) == (8, 1024, 65536, 1024, "N")


def fabricate_rpa_bundle(root, schedule, outputs_from):
    """A bundle with the files ``validate_fused_rpa_bundle`` reads, its outputs taken from
    ``outputs_from(inputs, scale)`` instead of a device."""
    import json

    import numpy as np

    from tpu_cake_b200 import rpa_cuda_lowering, rpa_runner

    plan = rpa_cuda_lowering.lower_inkling_rpa_to_cuda(schedule)
    inputs = workloads.inkling_fused_rpa_inputs(97)
    expectation = rpa_runner.expected_fused_rpa(inputs, softmax_scale=plan.softmax_scale)
    outputs = outputs_from(inputs, plan.softmax_scale)
    for folder, names, arrays in (("inputs", rpa_cuda_lowering.FUSED_INPUT_NAMES, inputs), ("outputs", ("output", "updated_cache"), outputs),
                                  ("oracle", ("output", "updated_cache"), expectation)):
        (root / folder).mkdir()
        for index, (name, array) in enumerate(zip(names, arrays, strict=True)):
            np.save(root / folder / f"{index:02d}-{name}.npy", array.view(np.uint16) if array.dtype.itemsize == 2 else array)
    (root / "physical.xdsl").write_text(ir.canonical_text(schedule))
    (root / "lowered_cuda.py").write_text(plan.render_executable_source())
    (root / "invocation.json").write_text(json.dumps({"kv_chunk_tokens": 0}))
    (root / "result.json").write_text(json.dumps({"artifacts": [], "schedule_sha256": plan.schedule_sha256, "cuda_source_sha256": plan.source_sha256()}))
    return plan


def test_rpa_bundle_replays_from_its_saved_kernel(tmp_path):
    """validate_fused_rpa_bundle lowers the kernel saved in the bundle again -- this backend's own
    schedule of the experiment, or the reference's (tpu7x target, other dimension names, the pinned
    hash) when the run was started from its file -- and refuses a bundle whose kernel was swapped."""
    from tpu_cake_b200 import rpa_runner

    def oracle(inputs, scale):
        return rpa_runner.expected_fused_rpa(inputs, softmax_scale=scale)

    own = tmp_path / "own"
    own.mkdir()
    fabricate_rpa_bundle(own, workloads.inkling_fused_rpa_schedule(), oracle)
    rpa_runner.validate_fused_rpa_bundle(own)

    builder = rpa_kernel("inkling_fused_rpa_decode", fused_inputs())
    builder.fused_ragged_paged_attention((*builder.inputs, builder.inputs[0], builder.inputs[3]), stage=0, softmax_scale="0.03125",
                                         vmem_limit_bytes=96 << 20)
    saved = tmp_path / "reference.xdsl"
    saved.write_text(ir.canonical_text(builder.module()))
    theirs = tmp_path / "theirs"
    theirs.mkdir()
    plan = fabricate_rpa_bundle(theirs, rpa_runner.fused_rpa_schedule_of(saved), oracle)
    assert plan.schedule_sha256 == "e1de39a3dfa8f4c930207fbe5218aa1f956b19b0b933e993fe35ae916e8ecad7"
    rpa_runner.validate_fused_rpa_bundle(theirs)

    (theirs / "physical.xdsl").write_text((own / "physical.xdsl").read_text())
    with pytest.raises(ValueError, match="LOWERED_CODE_IDENTITY_DOES_NOT_REPLAY"):
        rpa_runner.validate_fused_rpa_bundle(theirs)

    other = schedule_lowering.lower_distributed_matmul(workloads.distributed_matmul_schedule())
    wrong = tmp_path / "matmul.xdsl"
    wrong.write_text(ir.canonical_text(other))
    with pytest.raises(ValueError, match="FUSED_RPA_SCHEDULE_SHAPE_MISMATCH"):
        rpa_runner.fused_rpa_schedule_of(wrong)
