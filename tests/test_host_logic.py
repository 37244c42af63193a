"""Host-side mirrors of the reference's plugin interface: plan dataclasses, preflight, workloads."""

from __future__ import annotations

import numpy as np
import pytest

from tests.test_oracle_golden import fused_inputs
from tpu_cake_b200 import cuda_lowering, rpa_cuda_lowering, workloads


def test_matmul_plan_mirrors_reference_fields_for_headline_shape():
    plan = cuda_lowering.plan_distributed_matmul(mesh_size=8, m=128, k=1024, n=1024)
    assert plan.lhs_local_shape == (128, 128) and plan.rhs_local_shape == (128, 1024)
    assert plan.partial_local_shape == (128, 1024) and plan.output_local_shape == (128, 128)
    assert plan.lhs_sharding == ("", "t") and plan.rhs_sharding == ("t", "") and plan.output_sharding == ("", "t")
    assert plan.global_lhs_shape == (128, 1024) and plan.global_rhs_shape == (1024, 1024)
    assert plan.global_output_shape == (128, 1024)
    assert plan.tile_k == 128 and plan.scatter_dimension == 1
    assert plan.collective_implementation is cuda_lowering.MatmulCollectiveStrategy.NCCL_REDUCE_SCATTER
    along_m = cuda_lowering.plan_distributed_matmul(mesh_size=8, m=128, k=1024, n=1024, scatter_dimension=0, output_dtype="bf16")
    assert along_m.output_local_shape == (16, 1024) and along_m.output_sharding == ("t", "")


def test_matmul_plan_source_identity_is_stable_and_sensitive():
    a = cuda_lowering.plan_distributed_matmul(mesh_size=8, m=128, k=1024, n=1024)
    b = cuda_lowering.plan_distributed_matmul(mesh_size=8, m=128, k=1024, n=1024)
    c = cuda_lowering.plan_distributed_matmul(mesh_size=8, m=128, k=1024, n=1024, tile_n=128)
    assert a.source_sha256() == b.source_sha256() != c.source_sha256()
    assert "cake_matmul_rs_sm100" in a.render_executable_source()


def test_matmul_plan_rejects_unrepresentable_schedules():
    with pytest.raises(cuda_lowering.UnsupportedLoweringError, match="divisible"):
        cuda_lowering.plan_distributed_matmul(mesh_size=8, m=128, k=1020, n=1024)
    with pytest.raises(cuda_lowering.UnsupportedLoweringError, match="tiles"):
        cuda_lowering.plan_distributed_matmul(mesh_size=1, m=128, k=1024, n=1024, tile_n=512)
    with pytest.raises(cuda_lowering.UnsupportedLoweringError, match="scatter"):
        cuda_lowering.plan_distributed_matmul(mesh_size=8, m=100, k=1024, n=1024, scatter_dimension=0)


def test_p2p_resources_for_large_shape():
    plan = cuda_lowering.plan_distributed_matmul(
        mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension=0, output_dtype="bf16",
        collective_implementation=cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE_BF16_TRANSPORT,
    )
    resources = plan.collective_resources
    local = 1024 * 8192 * 2
    assert resources.receive_slot_bytes == 2 * 8 * local
    assert resources.remote_payload_bytes == 7 * local == 117_440_512
    f32 = cuda_lowering.plan_distributed_matmul(
        mesh_size=8, m=8192, k=16384, n=8192, scatter_dimension=0,
        collective_implementation=cuda_lowering.MatmulCollectiveStrategy.P2P_FUSED_EPILOGUE,
    )
    assert f32.collective_resources.remote_payload_bytes == 234_881_024


def _plan_for(inputs) -> rpa_cuda_lowering.CudaFusedRpaPlan:
    shapes = [tuple(np.asarray(value).shape) for value in inputs]
    return rpa_cuda_lowering.CudaFusedRpaPlan(
        name="inkling_fused_rpa", schedule_sha256="0" * 64, query_shape=shapes[0], key_shape=shapes[1], value_shape=shapes[2],
        fused_cache_shape=shapes[3], kv_lengths_shape=shapes[4], page_indices_shape=shapes[5],
        cumulative_query_lengths_shape=shapes[6], cumulative_kv_lengths_shape=shapes[7], distribution_shape=shapes[8],
        relative_states_shape=shapes[9], relative_projection_shape=shapes[10], output_shape=shapes[0], softmax_scale=1.0 / shapes[0][2],
    )


def test_preflight_accepts_reference_inputs_and_rejects_bad_metadata(golden_dir):
    vectors = np.load(golden_dir / "rpa_reference_vectors.npz")
    inputs = fused_inputs(vectors, 0)
    plan = _plan_for(inputs)
    plan.preflight(*inputs)

    def replaced(index, value):
        return (*inputs[:index], value, *inputs[index + 1 :])

    with pytest.raises(ValueError, match="decode-only distribution"):
        plan.preflight(*replaced(8, np.zeros(3, np.int32)))
    with pytest.raises(ValueError, match="one query token"):
        plan.preflight(*replaced(6, np.array([0, 1, 2, 4, 4], np.int32)))
    with pytest.raises(ValueError, match="positive KV lengths"):
        plan.preflight(*replaced(4, np.array([0, 17, 33, 49], np.int32)))
    with pytest.raises(ValueError, match="outside the fused cache"):
        plan.preflight(*replaced(5, np.full(32, 99, np.int32)))
    pages = inputs[5].copy()
    pages[2] = pages[0]
    with pytest.raises(ValueError, match="updates collide"):
        plan.preflight(*replaced(5, pages))
    pages = inputs[5].copy()
    pages[2] = pages[1]
    with pytest.raises(ValueError, match="aliases logical pages"):
        plan.preflight(*replaced(5, pages))
    pages = inputs[5].copy()
    pages[1] = pages[0]
    shared = (*inputs[:4], np.array([1, 2, 33, 49], np.int32), pages, inputs[6], np.array([0, 16, 32, 80, 144], np.int32), *inputs[8:])
    with pytest.raises(ValueError, match="active write page is shared"):
        plan.preflight(*shared)
    huge = np.full(4, np.iinfo(np.int32).max, np.int32)
    overflow = (*inputs[:4], huge, inputs[5], inputs[6], np.array([0, np.iinfo(np.int32).min, 0, np.iinfo(np.int32).min, 0], np.int32), *inputs[8:])
    with pytest.raises(ValueError, match="exceeds total cache capacity"):
        plan.preflight(*overflow)
    with pytest.raises(ValueError, match="page-aligned"):
        plan.preflight(*replaced(7, np.array([0, 16, 48, 96, 161], np.int32)))
    with pytest.raises(ValueError, match="11 inputs"):
        plan.preflight(*inputs[:10])


def test_fused_plan_validates_contract():
    with pytest.raises(ValueError, match="pack = 2"):
        rpa_cuda_lowering.CudaFusedRpaPlan(
            name="x", schedule_sha256="0" * 64, query_shape=(4, 4, 32), key_shape=(4, 2, 32), value_shape=(4, 2, 32),
            fused_cache_shape=(32, 16, 1, 4, 128), kv_lengths_shape=(4,), page_indices_shape=(32,),
            cumulative_query_lengths_shape=(5,), cumulative_kv_lengths_shape=(5,), distribution_shape=(3,),
            relative_states_shape=None, relative_projection_shape=None, output_shape=(4, 4, 32), softmax_scale=1 / 32,
        )


def test_decode_metadata_is_seeded_and_consistent():
    config = workloads.DECODE_64
    lengths, table = workloads.decode_metadata(config)
    again, table_again = workloads.decode_metadata(config)
    np.testing.assert_array_equal(lengths, again)
    np.testing.assert_array_equal(table, table_again)
    assert lengths.shape == (64,) and lengths.min() >= 128 and lengths.max() <= 8192
    assert table.shape == (64, 512) and table.dtype == np.int32
    used = np.concatenate([table[s, : -(-int(lengths[s]) // 16)] for s in range(64)])
    assert np.unique(used).size == used.size and used.max() < 65536
    sharded_lengths, sharded_table = workloads.decode_metadata(workloads.DECODE_SHARDED_256)
    assert sharded_lengths.min() >= 1024 and sharded_lengths.max() <= 32768 and sharded_table.shape == (256, 1024)
    expected = int(lengths.astype(np.int64).sum()) * 8 * 128 * 4 + 64 * 32 * 128 * 4 + int((-(-lengths.astype(np.int64) // 16)).sum()) * 4 + 8 * 64
    assert workloads.decode_algorithmic_bytes(lengths, 32, 8, 128, 16) == expected


def test_shard_matmul_inputs_partition_k():
    lhs, rhs = workloads.distributed_matmul_inputs(4, 16, 32, 16)
    pieces = [workloads.shard_matmul_inputs(lhs, rhs, 4, r) for r in range(4)]
    assert pieces[0][0].shape == (16, 8) and pieces[0][1].shape == (8, 16)
    np.testing.assert_array_equal(np.concatenate([p[0] for p in pieces], axis=1), lhs)
    np.testing.assert_array_equal(np.concatenate([p[1] for p in pieces], axis=0), rhs)


def test_sharded_surface_partitioning_round_trips():
    """The 2 x 4 data x tensor surface: global shapes follow the partition specs, every position's
    shard has the local plan's shapes, and assembling the shards restores the global arrays."""
    from tests.sharded_cases import build_sharded_surface
    from tpu_cake_b200 import rpa_cuda_lowering

    global_inputs, _ = build_sharded_surface(3)
    shapes = [tuple(np.asarray(v).shape) for v in global_inputs]
    local = rpa_cuda_lowering.CudaFusedRpaPlan(
        name="surface", schedule_sha256="0" * 64, query_shape=(4, 8, 128), key_shape=(4, 4, 128), value_shape=(4, 4, 128),
        fused_cache_shape=(shapes[3][0] // 2, 1, 4, 2, 128), kv_lengths_shape=(4,), page_indices_shape=(shapes[5][0] // 2,),
        cumulative_query_lengths_shape=(5,), cumulative_kv_lengths_shape=(5,), distribution_shape=(3,),
        relative_states_shape=(4, 8, 16), relative_projection_shape=(16, 512), output_shape=(4, 8, 128), softmax_scale=1.0 / 128,
    )
    surface = rpa_cuda_lowering.ShardedCudaFusedRpaPlan(local)
    assert surface.global_input_shapes[0] == (8, 32, 128) and surface.global_input_shapes[3][2] == 16
    assert [tuple(s) for s in surface.global_input_shapes] == shapes
    assert surface.mesh_position(5) == (1, 1) and surface.output_partition_specs == (("data", "tensor", ""), ("data", "", "tensor", "", ""))
    pieces_q, pieces_cache = {}, {}
    for rank in range(8):
        position = surface.mesh_position(rank)
        shard = surface.shard_inputs(global_inputs, position)
        for value, shape in zip(shard, local.input_shapes, strict=True):
            assert tuple(value.shape) == tuple(shape)
        pieces_q[position], pieces_cache[position] = np.asarray(shard[0]), np.asarray(shard[3])
    np.testing.assert_array_equal(surface.assemble(pieces_q, 0).view(np.uint16), np.asarray(global_inputs[0]).view(np.uint16))
    np.testing.assert_array_equal(surface.assemble(pieces_cache, 1).view(np.uint16), np.asarray(global_inputs[3]).view(np.uint16))
    with pytest.raises(ValueError, match="outside the 2x4 mesh"):
        surface.mesh_position(8)
    with pytest.raises(ValueError, match="the surface expects"):
        surface.shard_inputs((global_inputs[0][:4],) + global_inputs[1:], (0, 0))


def test_surface_error_metrics():
    from tpu_cake_b200 import rpa_cuda_lowering

    expected = np.array([[1.0, -2.0], [0.5, 4.0]], dtype=np.float32)
    actual = expected + np.array([[0.0, 0.01], [-0.02, 0.0]], dtype=np.float32)
    maximum, relative = rpa_cuda_lowering.surface_errors(actual, expected)
    assert abs(maximum - 0.02) < 1e-6
    assert abs(relative - np.sqrt((0.01**2 + 0.02**2) / (1 + 4 + 0.25 + 16))) < 1e-6
    with pytest.raises(ValueError, match="ABI_MISMATCH"):
        rpa_cuda_lowering.surface_errors(actual.astype(np.float64), expected)
    with pytest.raises(ValueError, match="NONFINITE"):
        rpa_cuda_lowering.surface_errors(np.full_like(expected, np.nan), expected)
