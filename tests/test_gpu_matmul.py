"""GPU parity of cake_matmul_rs_sm100 / cake_reduce_slots_sm100 against the CPU oracle, through
the C ABI."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import matmul_rs as oracle
from tests.helpers import BF16, bf16_to_torch, bits_to_bf16
from tpu_cake_b200 import _native, cuda_lowering, workloads

pytestmark = pytest.mark.gpu

PATTERNS = ("constant", "one-hot-stripes", "signed-periodic", "block-diagonal", "low-rank")


def run_single(lhs: np.ndarray, rhs: np.ndarray, device, *, tile_n=256, output_dtype="f32") -> np.ndarray:
    m, k = lhs.shape
    n = rhs.shape[1]
    plan = cuda_lowering.plan_distributed_matmul(mesh_size=1, m=m, k=k, n=n, tile_n=tile_n, output_dtype=output_dtype)
    executable, _ = plan.build()
    try:
        out = torch.full(plan.output_local_shape, float("nan"), dtype=torch.float32 if output_dtype == "f32" else torch.bfloat16, device=device)
        executable(bf16_to_torch(lhs, device), bf16_to_torch(rhs, device), out)
        assert executable.status() == (0, 0, 0, 0)
        assert executable.launches_per_call == 1
        return out.float().cpu().numpy()
    finally:
        executable.close()


def test_reference_inputs_local_problem_meets_reference_tolerance(cuda_device):
    """mesh 8, 128 x 1024 x 1024 (the reference's CPU-runnable case): every rank's local
    contraction, summed in rank order on the host, against numpy on the exact bf16 inputs with the
    reference's allclose(1e-3, 1e-3)."""
    lhs, rhs = workloads.distributed_matmul_inputs(8, 128, 1024, 1024)
    expected = oracle.matmul_reference(lhs.astype(np.float32), rhs.astype(np.float32))
    total = np.zeros_like(expected)
    for rank in range(8):
        lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, 8, rank)
        partial = run_single(lhs_r, rhs_r, cuda_device, tile_n=128)
        reference_partial = oracle.local_partials(lhs.astype(np.float32), rhs.astype(np.float32), 8)[rank]
        assert np.allclose(partial, reference_partial, atol=1e-3, rtol=1e-3)
        total += partial
    assert np.allclose(total, expected, atol=1e-3, rtol=1e-3)
    whole = run_single(lhs, rhs, cuda_device)
    assert np.allclose(whole, expected, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("pattern", PATTERNS)
def test_structured_patterns_are_exact_on_device(cuda_device, golden_dir, pattern):
    """The reference's closed-form operand patterns have exactly representable products: the
    f32-accumulating tensor-core path must reproduce them bit for bit."""
    vectors = np.load(golden_dir / "matmul_structured_patterns.npz")
    lhs = bits_to_bf16(vectors[f"{pattern}/lhs_bf16_bits"])
    rhs = bits_to_bf16(vectors[f"{pattern}/rhs_bf16_bits"])
    actual = run_single(lhs, rhs, cuda_device, tile_n=64)
    np.testing.assert_array_equal(actual, vectors[f"{pattern}/product_f32"])


@pytest.mark.parametrize("shape", [(128, 64, 256), (1, 8, 8), (200, 136, 264), (257, 72, 40), (384, 1000, 520)])
@pytest.mark.parametrize("tile_n", (64, 128, 256))
def test_ragged_shapes_and_tiles(cuda_device, shape, tile_n):
    m, k, n = shape
    generator = np.random.default_rng(m * 1000 + n)
    lhs = generator.normal(size=(m, k)).astype(np.float32).astype(BF16)
    rhs = generator.normal(size=(k, n)).astype(np.float32).astype(BF16)
    expected = oracle.matmul_reference(lhs.astype(np.float32), rhs.astype(np.float32))
    actual = run_single(lhs, rhs, cuda_device, tile_n=tile_n)
    assert np.allclose(actual, expected, atol=1e-3, rtol=1e-3)
    rounded = run_single(lhs, rhs, cuda_device, tile_n=tile_n, output_dtype="bf16")
    np.testing.assert_array_equal(rounded, oracle.quantize_bf16(actual))


def test_repeat_runs_are_bit_identical(cuda_device):
    lhs, rhs = workloads.distributed_matmul_inputs(1, 512, 2048, 768)
    first = run_single(lhs, rhs, cuda_device)
    second = run_single(lhs, rhs, cuda_device)
    np.testing.assert_array_equal(first, second)


def _emulated_ranks(lhs, rhs, world, device, *, scatter_dimension, transport, output_dtype, strategy, tile_n):
    """Runs every mesh position's kernels on one GPU: all pushes first, then all reductions, so no
    launch ever waits on a later one."""
    lib = _native.load()
    m, k = lhs.shape
    n = rhs.shape[1]
    stream = torch.cuda.current_stream(device).cuda_stream
    handles, operands = [], []
    for rank in range(world):
        desc = _native.MatmulRsDesc(
            m=m, n=n, k_local=k // world, world=world, rank=rank, scatter_dim=scatter_dimension,
            out_dtype=_native.CAKE_DTYPE_F32 if output_dtype == "f32" else _native.CAKE_DTYPE_BF16,
            transport_dtype=_native.CAKE_DTYPE_F32 if transport == "f32" else _native.CAKE_DTYPE_BF16,
            strategy=strategy, tile_m=128, tile_n=tile_n, rhs_layout=0, wait_budget_ms=0,
        )
        handle = ctypes.c_void_p()
        _native.check(lib.cake_matmul_rs_create(ctypes.byref(desc), ctypes.byref(handle)))
        handles.append(handle)
        lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, world, rank)
        operands.append((bf16_to_torch(lhs_r, device), bf16_to_torch(rhs_r, device)))
    out_rows = m // world if scatter_dimension == 0 else m
    out_cols = n // world if scatter_dimension == 1 else n
    torch_out = torch.float32 if output_dtype == "f32" else torch.bfloat16
    results = []
    try:
        if strategy == _native.CAKE_RS_P2P_OWNER_PUSH:
            slots, flags = [], []
            for handle in handles:
                slot, flag = ctypes.c_void_p(), ctypes.c_void_p()
                _native.check(lib.cake_symm_alloc(lib.cake_matmul_rs_slot_bytes(handle), ctypes.byref(slot)))
                _native.check(lib.cake_symm_alloc(lib.cake_matmul_rs_flag_bytes(handle), ctypes.byref(flag)))
                slots.append(slot.value)
                flags.append(flag.value)
            array = ctypes.c_void_p * world
            for handle in handles:
                _native.check(lib.cake_matmul_rs_bind_peers(handle, array(*slots), array(*flags)))
            for repeat in range(4):  # exercises both slot parities and the growing call numbers in the flags
                outs = [torch.full((out_rows, out_cols), float("nan"), dtype=torch_out, device=device) for _ in range(world)]
                # On odd repeats the last position runs the one-kernel form (its reduction warps
                # work while its own contraction still pushes): by then every other position has
                # pushed, so that launch too waits on nothing that is enqueued after it.
                fused_last = repeat % 2 == 1
                for rank, (handle, (lhs_d, rhs_d)) in enumerate(zip(handles, operands)):
                    if fused_last and rank == world - 1:
                        _native.check(lib.cake_matmul_rs_enqueue(handle, lhs_d.data_ptr(), rhs_d.data_ptr(), outs[rank].data_ptr(), stream))
                    else:
                        _native.check(lib.cake_matmul_rs_enqueue_push(handle, lhs_d.data_ptr(), rhs_d.data_ptr(), stream))
                for rank, (handle, out) in enumerate(zip(handles, outs)):
                    if not (fused_last and rank == world - 1):
                        _native.check(lib.cake_matmul_rs_enqueue_reduce(handle, out.data_ptr(), stream))
                torch.cuda.synchronize(device)
                results.append([out.float().cpu().numpy() for out in outs])
            for handle in handles:
                word = _native.CakeStatus()
                _native.check(lib.cake_matmul_rs_status(handle, stream, ctypes.byref(word)))
                assert word.code == 0
            for pointer in slots + flags:
                lib.cake_symm_free(pointer)
        else:
            tdtype = torch.float32 if transport == "f32" else torch.bfloat16
            partials = []
            for handle, (lhs_d, rhs_d) in zip(handles, operands):
                partial = torch.full((world, out_rows, out_cols), float("nan"), dtype=tdtype, device=device)
                _native.check(lib.cake_matmul_rs_enqueue(handle, lhs_d.data_ptr(), rhs_d.data_ptr(), partial.data_ptr(), stream))
                partials.append(partial)
            torch.cuda.synchronize(device)
            total = torch.zeros((world, out_rows, out_cols), dtype=torch.float32, device=device)
            for partial in partials:  # rank order, like the oracle
                total += partial.float()
            results.append([total[r].cpu().numpy() for r in range(world)])
    finally:
        for handle in handles:
            lib.cake_matmul_rs_destroy(handle)
    return results


@pytest.mark.parametrize("scatter_dimension", (0, 1))
@pytest.mark.parametrize("transport, output_dtype", [("f32", "f32"), ("bf16", "bf16"), ("bf16", "f32")])
def test_p2p_owner_push_all_ranks_on_one_gpu(cuda_device, scatter_dimension, transport, output_dtype):
    """mesh 8 on 128 x 1024 x 1024 with the reference's inputs, both scatter dimensions (the
    reference scatters N; the large configuration scatters M, 16 rows per rank, so every 128-row
    tile is split between 8 owners)."""
    world = 8
    lhs, rhs = workloads.distributed_matmul_inputs(world, 128, 1024, 1024)
    expected = oracle.matmul_reduce_scatter(
        lhs.astype(np.float32), rhs.astype(np.float32), world=world, scatter_dimension=scatter_dimension,
        transport_dtype=transport, out_dtype=output_dtype,
    )
    runs = _emulated_ranks(lhs, rhs, world, cuda_device, scatter_dimension=scatter_dimension, transport=transport,
                           output_dtype=output_dtype, strategy=_native.CAKE_RS_P2P_OWNER_PUSH, tile_n=128)
    full = oracle.matmul_reference(lhs.astype(np.float32), rhs.astype(np.float32))
    for outputs in runs:
        for rank in range(world):
            if transport == "f32":
                assert np.allclose(outputs[rank], expected[rank], atol=1e-3, rtol=1e-3)
            else:
                # bf16 transport: partials are rounded once before the f32 sum; compare with the
                # oracle that rounds the same way (one bf16 ulp of the partial magnitude).
                assert oracle.relative_l2_error(outputs[rank], expected[rank]) < 4e-3
        assembled = np.concatenate(outputs, axis=scatter_dimension)
        assert oracle.relative_l2_error(assembled, full) < 1e-2
    for later in runs[1:]:
        for rank in range(world):
            np.testing.assert_array_equal(later[rank], runs[0][rank])


@pytest.mark.parametrize("shape, world, scatter_dimension, transport", [
    ((3, 16, 8), 2, 1, "bf16"),     # local output 3 x 4 bf16: 24 bytes per source, nothing 16-byte aligned
    ((5, 16, 24), 2, 1, "f32"),     # 5 x 12 f32: whole pieces but rows not in groups of 8
    ((96, 96, 40), 3, 0, "bf16"),   # a mesh size the vector reduction does not cover
    ((256, 192, 520), 4, 0, "f32"), # rows aligned, 520 columns: vector pieces, ragged last chunk
    ((384, 128, 768), 2, 1, "bf16"),
    ((512, 8192, 1024), 2, 0, "bf16"),   # K per rank 4096: deep enough that a rank's own tiles come last
    ((256, 16384, 512), 4, 1, "bf16"),   # the same owner order on four positions, scattering N
])
def test_p2p_owner_push_odd_shapes(cuda_device, shape, world, scatter_dimension, transport):
    """Shapes whose local output is not a whole number of 16-byte pieces, 128-byte chunks or
    128-row tiles go through the element-wise push and reduction; the last two are deep enough in K
    that the kernel walks its peers' tiles first and its own last. All must match the oracle."""
    m, k, n = shape
    generator = np.random.default_rng(m * 131 + n)
    lhs = generator.normal(size=(m, k)).astype(np.float32).astype(BF16)
    rhs = generator.normal(size=(k, n)).astype(np.float32).astype(BF16)
    expected = oracle.matmul_reduce_scatter(lhs.astype(np.float32), rhs.astype(np.float32), world=world,
                                            scatter_dimension=scatter_dimension, transport_dtype=transport, out_dtype="f32")
    runs = _emulated_ranks(lhs, rhs, world, cuda_device, scatter_dimension=scatter_dimension, transport=transport,
                           output_dtype="f32", strategy=_native.CAKE_RS_P2P_OWNER_PUSH, tile_n=128)
    for outputs in runs:
        for rank in range(world):
            if transport == "f32":
                assert np.allclose(outputs[rank], expected[rank], atol=1e-3, rtol=1e-3)
            else:
                assert oracle.relative_l2_error(outputs[rank], expected[rank]) < 4e-3
    for later in runs[1:]:
        for rank in range(world):
            np.testing.assert_array_equal(later[rank], runs[0][rank])


def test_reduction_gives_up_when_a_peer_never_pushes(cuda_device):
    """Two mesh positions on one GPU, a wait budget of 5 ms, and position 1 does not push: position
    0's reduction must give up (CAKE_ERR_TIMEOUT, code 2, missing source 1) without touching its
    output -- the wait runs out and the kernel returns, nothing faults or hangs. Position 1 then
    pushes late; a reduction consumes nothing, so enqueueing it again completes the step."""
    lib = _native.load()
    world, m, k, n = 2, 256, 512, 512
    lhs, rhs = workloads.distributed_matmul_inputs(world, m, k, n)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    handles, operands, slots, flags = [], [], [], []
    for rank in range(world):
        desc = _native.MatmulRsDesc(m=m, n=n, k_local=k // world, world=world, rank=rank, scatter_dim=0, out_dtype=_native.CAKE_DTYPE_F32,
                                    transport_dtype=_native.CAKE_DTYPE_F32, strategy=_native.CAKE_RS_P2P_OWNER_PUSH, tile_m=128, tile_n=256,
                                    rhs_layout=0, wait_budget_ms=5)
        handle = ctypes.c_void_p()
        _native.check(lib.cake_matmul_rs_create(ctypes.byref(desc), ctypes.byref(handle)))
        handles.append(handle)
        lhs_r, rhs_r = workloads.shard_matmul_inputs(lhs, rhs, world, rank)
        operands.append((bf16_to_torch(lhs_r, cuda_device), bf16_to_torch(rhs_r, cuda_device)))
        slot, flag = ctypes.c_void_p(), ctypes.c_void_p()
        _native.check(lib.cake_symm_alloc(lib.cake_matmul_rs_slot_bytes(handle), ctypes.byref(slot)))
        _native.check(lib.cake_symm_alloc(lib.cake_matmul_rs_flag_bytes(handle), ctypes.byref(flag)))
        slots.append(slot.value)
        flags.append(flag.value)
    try:
        array = ctypes.c_void_p * world
        for handle in handles:
            _native.check(lib.cake_matmul_rs_bind_peers(handle, array(*slots), array(*flags)))
        outs = [torch.full((m // world, n), float("nan"), dtype=torch.float32, device=cuda_device) for _ in range(world)]
        _native.check(lib.cake_matmul_rs_enqueue_push(handles[0], operands[0][0].data_ptr(), operands[0][1].data_ptr(), stream))
        _native.check(lib.cake_matmul_rs_enqueue_reduce(handles[0], outs[0].data_ptr(), stream))
        word = _native.CakeStatus()
        code = lib.cake_matmul_rs_status(handles[0], stream, ctypes.byref(word))
        assert code == _native.CAKE_ERR_TIMEOUT
        assert word.code == 2 and word.detail1 == 1
        assert bool(torch.isnan(outs[0]).all())
        # The late peer arrives; both reductions now complete.
        _native.check(lib.cake_matmul_rs_enqueue_push(handles[1], operands[1][0].data_ptr(), operands[1][1].data_ptr(), stream))
        for handle, out in zip(handles, outs):
            _native.check(lib.cake_matmul_rs_enqueue_reduce(handle, out.data_ptr(), stream))
        for handle in handles:
            _native.check(lib.cake_matmul_rs_status(handle, stream, ctypes.byref(word)))
            assert word.code == 0
        expected = oracle.matmul_reduce_scatter(lhs.astype(np.float32), rhs.astype(np.float32), world=world, scatter_dimension=0)
        for rank in range(world):
            assert np.allclose(outs[rank].cpu().numpy(), expected[rank], atol=1e-3, rtol=1e-3)
        # And the next call, on the other slot parity, is an ordinary one.
        for handle, (lhs_d, rhs_d) in zip(handles, operands):
            _native.check(lib.cake_matmul_rs_enqueue_push(handle, lhs_d.data_ptr(), rhs_d.data_ptr(), stream))
        for handle, out in zip(handles, outs):
            out.fill_(float("nan"))
            _native.check(lib.cake_matmul_rs_enqueue_reduce(handle, out.data_ptr(), stream))
        for handle in handles:
            _native.check(lib.cake_matmul_rs_status(handle, stream, ctypes.byref(word)))
            assert word.code == 0
        for rank in range(world):
            assert np.allclose(outs[rank].cpu().numpy(), expected[rank], atol=1e-3, rtol=1e-3)
    finally:
        for handle in handles:
            lib.cake_matmul_rs_destroy(handle)
        for pointer in slots + flags:
            lib.cake_symm_free(pointer)


@pytest.mark.parametrize("world, scatter_dimension, tile_n", [(2, 0, 256), (4, 1, 64), (8, 1, 128)])
def test_owner_major_partial_layout_for_library_collective(cuda_device, world, scatter_dimension, tile_n):
    lhs, rhs = workloads.distributed_matmul_inputs(world, 256, 1024, 512)
    expected = oracle.matmul_reduce_scatter(lhs.astype(np.float32), rhs.astype(np.float32), world=world, scatter_dimension=scatter_dimension)
    outputs = _emulated_ranks(lhs, rhs, world, cuda_device, scatter_dimension=scatter_dimension, transport="f32",
                              output_dtype="f32", strategy=_native.CAKE_RS_LOCAL_PARTIAL, tile_n=tile_n)[0]
    for rank in range(world):
        assert np.allclose(outputs[rank], expected[rank], atol=1e-3, rtol=1e-3)


def test_large_configuration_properties(cuda_device):
    """8192 x 16384 x 8192 at one mesh position (the benchmark workload): sampled rows against the
    oracle, and the row-sum identity C 1 = A (B 1) over the whole output."""
    m, k, n = 8192, 16384, 8192
    generator = torch.Generator(device=cuda_device).manual_seed(20261125)
    lhs = (torch.randn((m, k), generator=generator, device=cuda_device) * k**-0.5).to(torch.bfloat16)
    rhs = (torch.randn((k, n), generator=generator, device=cuda_device) * k**-0.5).to(torch.bfloat16)
    plan = cuda_lowering.plan_distributed_matmul(mesh_size=1, m=m, k=k, n=n, output_dtype="bf16")
    executable, _ = plan.build()
    out = executable(lhs, rhs)
    assert executable.status() == (0, 0, 0, 0)
    rows = np.array([0, 1, 127, 128, 4095, 4096, 8191, 5000, 6001, 77], dtype=np.int64)
    lhs_rows = lhs[torch.from_numpy(rows).to(cuda_device)].float().cpu().numpy()
    rhs_host = rhs.float().cpu().numpy()
    expected = oracle.matmul_reference(lhs_rows, rhs_host)
    actual = out[torch.from_numpy(rows).to(cuda_device)].float().cpu().numpy()
    assert oracle.max_abs_error(actual, expected) < 2e-2
    assert oracle.relative_l2_error(actual, expected) < 1e-2
    row_sums = out.double().sum(dim=1).cpu().numpy()
    identity_sums = (lhs.double() @ rhs.double().sum(dim=1)).cpu().numpy()
    # bf16 rounding of 8192 outputs of magnitude ~1/128 each: absolute error well under 1e-2.
    assert np.max(np.abs(row_sums - identity_sums)) < 2e-2
    executable.close()


@pytest.mark.parametrize("mesh_size, strategy", [(2, "p2p_fused_epilogue_bf16_transport"), (8, "p2p_fused_epilogue"), (4, "nccl_reduce_scatter")])
def test_runner_writes_a_complete_bundle(cuda_device, tmp_path, mesh_size, strategy):
    """run-matmul on the reference's CPU-runnable shape: ledger reaches TIMED, artifacts exist and
    the saved output passes the reference's tolerance against the saved oracle."""
    from tpu_cake_b200 import runner
    from tpu_cake_b200.run_ledger import RunLedger, RunState

    out = tmp_path / "run"
    with pytest.raises(ValueError, match="MESH_NOT_AVAILABLE"):
        runner.run_distributed_matmul(out, mesh_size=mesh_size, m=128, k=1024, n=1024, warmup_iterations=1, measured_iterations=3,
                                      collective_strategy=strategy)
    assert not out.exists()
    result = runner.run_distributed_matmul(out, mesh_size=mesh_size, m=128, k=1024, n=1024, warmup_iterations=1,
                                           measured_iterations=3, collective_strategy=strategy, emulate_on_one_gpu=True)
    assert result.passed and result.median_ns > 0 and len(result.samples_ns) == 3
    assert result.execution == "emulated-on-one-gpu"
    for name in ("invocation.json", "profiler_config.json", "source_state.json", "source_diff.patch", "experiment.json",
                 "distributed.xdsl", "physical.xdsl", "lowered_cuda.py", "cost_model_input.json", "cost_model.json",
                 "kernel_manifest.json", "lhs.npy", "rhs.npy", "output.npy", "oracle.npy", "ledger.sqlite", "result.json"):
        assert (out / name).exists(), name
    with RunLedger(out / "ledger.sqlite") as ledger:
        states = [event.state for event in ledger.history(result.run_id)]
    assert states == [RunState.CREATED, RunState.VERIFIED, RunState.LOWERED, RunState.COMPILED, RunState.CORRECT, RunState.TIMED]
    if "bf16" in strategy:
        assert oracle.relative_l2_error(np.load(out / "output.npy"), np.load(out / "oracle.npy")) < 1e-2
    else:
        assert np.allclose(np.load(out / "output.npy"), np.load(out / "oracle.npy"), atol=1e-3, rtol=1e-3)
    with pytest.raises(FileExistsError):
        runner.run_distributed_matmul(out, mesh_size=mesh_size, m=128, k=1024, n=1024, warmup_iterations=0, measured_iterations=1,
                                      emulate_on_one_gpu=True)


def test_tile_search_through_the_runner(cuda_device, tmp_path):
    """search-matmul on one GPU (the mesh positions emulated): every candidate runs in every round,
    all pass the oracle on the same inputs, and the result names a baseline and per-candidate medians."""
    from tpu_cake_b200 import search

    contract = search.MatmulSearchContract(
        mesh_size=2, m=256, k=1024, n=512, warmup_iterations=1, measured_iterations=3, rounds=5, bootstrap_samples=1000,
        collective_strategy="p2p_fused_epilogue", scatter_dimension="N", output_dtype="f32", execution="emulated-on-one-gpu",
        candidates=(search.MatmulSearchCandidate("tile-128x256", 128, 256), search.MatmulSearchCandidate("tile-128x64", 128, 64)),
    )
    result = search.run_matmul_search(tmp_path / "search", contract)
    assert result.baseline == "tile-128x256" and len(result.run_results) == 10
    assert result.execution_orders[1] == ("tile-128x64", "tile-128x256")
    assert all(row.sample_count == 15 and row.median_ns > 0 for row in result.candidates)
    assert result.winner in (None, "tile-128x64")
    assert (tmp_path / "search" / "round-04" / "tile-128x64" / "result.json").exists()
    # Resume: the finished runs are validated and reused (same samples, nothing re-run) ...
    resumed = search.run_matmul_search(tmp_path / "search", contract)
    assert resumed.candidates == result.candidates and resumed.run_results == result.run_results
    # ... a different contract in the same directory is refused, and so is a run that left no result.
    import dataclasses

    with pytest.raises(ValueError, match="SEARCH_CONTRACT_CHANGED"):
        search.run_matmul_search(tmp_path / "search", dataclasses.replace(contract, measured_iterations=4))
    (tmp_path / "search" / "round-02" / "tile-128x64" / "result.json").unlink()
    with pytest.raises(ValueError, match="SEARCH_RUN_INCOMPLETE"):
        search.run_matmul_search(tmp_path / "search", contract)


def test_receipt_is_written_validated_and_refuses_tampering(cuda_device, tmp_path):
    """finalize-matmul-run on a fresh bundle, verify-matmul-bundle on the result, then three kinds of
    tampering: an artifact byte, a roofline metric, a profile capture with the wrong kernels."""
    import json

    from tpu_cake_b200 import receipt, runner

    out = tmp_path / "run"
    runner.run_distributed_matmul(out, mesh_size=2, m=128, k=1024, n=1024, warmup_iterations=1, measured_iterations=3,
                                  collective_strategy="p2p_fused_epilogue", emulate_on_one_gpu=True)
    header = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'

    def launch(index, kernel):
        return f'"{index}","1","python","h","{kernel}","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","s","gpu__time_duration.sum","ns","9000"\n'

    good = tmp_path / "good.csv"
    good.write_text(header + launch(0, "void cake::cake_matmul_rs_sm100<256, 0>(...)") + launch(1, "void cake::cake_reduce_slots_sm100<float, float>(...)"))
    wrong = tmp_path / "wrong.csv"
    wrong.write_text(header + launch(0, "void cake::cake_matmul_rs_sm100<256, 0>(...)") + launch(1, "ncclDevKernel_ReduceScatter_Sum_f32_RING_LL(...)"))
    with pytest.raises(ValueError, match="PROFILE_CAPTURE_REJECTED"):
        receipt.finalize_matmul_run(out, profile_csv=wrong)
    document = receipt.finalize_matmul_run(out, profile_csv=good)
    assert document["profile"]["attached"] and document["metrics"]["measured_to_two_resource_floor"] > 1.0
    assert receipt.validate_receipt(out)["receipt_id"] == document["receipt_id"]
    metrics_path = out / "roofline" / "metrics.json"
    original = metrics_path.read_text()
    metrics = json.loads(original)
    metrics["peak_efficiency"] *= 2
    metrics_path.write_text(json.dumps(metrics, indent=2) + "\n")
    with pytest.raises(ValueError, match="ARTIFACT_CHANGED path=roofline/metrics.json"):
        receipt.validate_receipt(out)
    metrics_path.write_text(original)
    receipt.validate_receipt(out)
    with open(out / "output.npy", "r+b") as handle:
        handle.seek(200)
        handle.write(b"\x01")
    with pytest.raises(ValueError, match="ARTIFACT_CHANGED path=output.npy"):
        receipt.validate_receipt(out)


@pytest.mark.parametrize(
    "shape, output_dtype",
    [((384, 1000, 520), "f32"), ((2048, 4096, 512), "bf16"), ((4096, 8192, 256), "f32")],
    ids=["one-enqueue", "two-row-blocks", "eight-row-blocks"],
)
def test_host_buffers_in_host_buffer_out(cuda_device, shape, output_dtype):
    """cake_matmul_rs_run_host: the same bits as the device-buffer call, whether the matrix goes
    through in one enqueue (small operands) or in blocks of rows that overlap the copies with the
    contraction (lhs blocks of at least 8 MiB), twice in a row on the same plan."""
    m, k, n = shape
    generator = np.random.default_rng(m + k + n)
    lhs = generator.normal(scale=k**-0.5, size=(m, k)).astype(np.float32).astype(BF16)
    rhs = generator.normal(scale=k**-0.5, size=(k, n)).astype(np.float32).astype(BF16)
    plan = cuda_lowering.plan_distributed_matmul(mesh_size=1, m=m, k=k, n=n, tile_n=256, output_dtype=output_dtype)
    executable, _ = plan.build()
    try:
        torch_dtype = torch.float32 if output_dtype == "f32" else torch.bfloat16
        device_out = torch.full(plan.output_local_shape, float("nan"), dtype=torch_dtype, device=cuda_device)
        executable(bf16_to_torch(lhs, cuda_device), bf16_to_torch(rhs, cuda_device), device_out)
        expected_bits = device_out.cpu().view(torch.int32 if output_dtype == "f32" else torch.int16).numpy()
        host_dtype = np.float32 if output_dtype == "f32" else np.uint16
        for _ in range(2):
            out = np.zeros(plan.output_local_shape, dtype=host_dtype)
            executable.run_host(lhs.view(np.uint16), rhs.view(np.uint16), out)
            np.testing.assert_array_equal(out.view(expected_bits.dtype), expected_bits)
        assert executable.status() == (0, 0, 0, 0)
        reference = oracle.matmul_reference(lhs.astype(np.float32), rhs.astype(np.float32))
        actual = out if output_dtype == "f32" else bits_to_bf16(out).astype(np.float32)
        assert oracle.relative_l2_error(actual, reference) <= (1e-5 if output_dtype == "f32" else 1e-2)
    finally:
        executable.close()
