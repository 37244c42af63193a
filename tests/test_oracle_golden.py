"""The CPU oracle against vectors produced by the reference's own code (tests/golden)."""

from __future__ import annotations

import json

import numpy as np
import pytest

from oracle import matmul_rs, rpa
from tests.helpers import BF16, bits_to_bf16
from tpu_cake_b200 import identity, workloads

PATTERNS = ("constant", "one-hot-stripes", "signed-periodic", "block-diagonal", "low-rank")
FUSED_NAMES = (
    "queries", "keys", "values", "cache", "kv_lengths", "page_indices", "cu_q_lens", "cu_kv_lens",
    "distribution", "relative_states", "relative_projection",
)
BF16_FUSED = {"queries", "keys", "values", "cache", "relative_states", "relative_projection"}


@pytest.fixture(scope="module")
def identity_vectors(golden_dir):
    return json.loads((golden_dir / "identity_vectors.json").read_text())


@pytest.fixture(scope="module")
def rpa_vectors(golden_dir):
    return np.load(golden_dir / "rpa_reference_vectors.npz")


def fused_inputs(vectors, seed: int):
    values = []
    for name in FUSED_NAMES:
        array = vectors[f"fused/seed{seed}/{name}"]
        values.append(bits_to_bf16(array) if name in BF16_FUSED else array)
    return tuple(values)


def test_semantic_identities_match_reference(identity_vectors):
    for key, expected in identity_vectors["semantic_sha256"].items():
        parts = key.split("|")
        assert identity.semantic_sha256(*parts) == expected
        assert str(identity.semantic_seed(*parts)) == identity_vectors["semantic_seed"][key]
    assert identity.semantic_sha256("a", "b", schema=identity.LEGACY_SEMANTIC_IDENTITY_SCHEMA) == identity_vectors["legacy"]
    with pytest.raises(ValueError):
        identity.semantic_sha256("a", "")
    probe = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    assert identity.array_sha256(probe) == identity_vectors["array_sha256"]["arange24_f32_2x3x4"]
    assert identity.array_sha256(np.arange(24, dtype=np.int32).reshape(4, 6)) == identity_vectors["array_sha256"]["arange24_i32_4x6"]


def test_matmul_inputs_reproduce_reference_hashes(identity_vectors):
    pinned = identity_vectors["matmul_c1_inputs"]
    assert workloads.distributed_matmul_workload_identity(8, 128, 1024, 1024) == pinned["workload_identity"]
    lhs, rhs = workloads.distributed_matmul_inputs(8, 128, 1024, 1024)
    assert identity.array_sha256(lhs.astype(np.float32)) == pinned["lhs_sha256"]
    assert identity.array_sha256(rhs.astype(np.float32)) == pinned["rhs_sha256"]


@pytest.mark.slow
def test_matmul_inputs_reproduce_committed_contract_hashes(identity_vectors):
    """The hashes the reference commits in contracts/matmul-collective-confirmation-v1.json for
    mesh 8, 1024 x 65536 x 1024 (512 MiB of float32 draws: a few seconds)."""
    pinned = identity_vectors["confirmation_contract_input_hashes"]
    lhs, rhs = workloads.distributed_matmul_inputs(8, 1024, 65536, 1024)
    assert identity.array_sha256(lhs.astype(np.float32)) == pinned["timing_lhs_sha256"]
    assert identity.array_sha256(rhs.astype(np.float32)) == pinned["timing_rhs_sha256"]


@pytest.mark.parametrize("pattern", PATTERNS)
@pytest.mark.parametrize("scatter_dimension", (0, 1))
def test_structured_patterns_are_exact(golden_dir, pattern, scatter_dimension):
    vectors = np.load(golden_dir / "matmul_structured_patterns.npz")
    lhs = bits_to_bf16(vectors[f"{pattern}/lhs_bf16_bits"]).astype(np.float32)
    rhs = bits_to_bf16(vectors[f"{pattern}/rhs_bf16_bits"]).astype(np.float32)
    product = vectors[f"{pattern}/product_f32"]
    np.testing.assert_array_equal(matmul_rs.matmul_reference(lhs, rhs), product)
    pieces = matmul_rs.matmul_reduce_scatter(lhs, rhs, world=8, scatter_dimension=scatter_dimension)
    np.testing.assert_array_equal(np.concatenate(pieces, axis=scatter_dimension), product)


def test_reduce_scatter_matches_single_product_within_reference_tolerance():
    lhs, rhs = workloads.distributed_matmul_inputs(8, 128, 1024, 1024)
    lhs, rhs = lhs.astype(np.float32), rhs.astype(np.float32)
    expected = matmul_rs.matmul_reference(lhs, rhs)
    for world in (1, 2, 4, 8):
        pieces = matmul_rs.matmul_reduce_scatter(lhs, rhs, world=world, scatter_dimension=1)
        assert pieces[0].shape == (128, 1024 // world)
        assert np.allclose(np.concatenate(pieces, axis=1), expected, atol=1e-3, rtol=1e-3)
    rounded = matmul_rs.matmul_reduce_scatter(lhs, rhs, world=8, scatter_dimension=0, transport_dtype="bf16", out_dtype="bf16")
    assert rounded[0].shape == (16, 1024)
    assert matmul_rs.relative_l2_error(np.concatenate(rounded, axis=0), expected) < 1e-2


@pytest.mark.parametrize("seed", (0, 3))
def test_separate_cache_oracle_matches_reference(rpa_vectors, seed):
    args = [rpa_vectors[f"separate/seed{seed}/{name}"] for name in ("query", "key_cache", "value_cache", "page_table", "sequence_lengths", "bias")]
    actual = rpa.rpa_separate(*args)
    np.testing.assert_allclose(actual, rpa_vectors[f"separate/seed{seed}/output"], rtol=1e-6, atol=1e-6)


def test_separate_cache_oracle_closed_form():
    """q = 1, K = 1, V = arange with independent K / V head counts (the reference's own
    known-answer test): uniform weights over 5 tokens give arange(6) + 12."""
    output = rpa.rpa_separate(
        np.ones((1, 4, 8), np.float32), np.ones((2, 4, 2, 8), np.float32),
        np.arange(48, dtype=np.float32).reshape(2, 4, 1, 6), np.array([[0, 1]], np.int32), np.array([5], np.int32),
        np.zeros((4, 8), np.float32),
    )
    assert output.shape == (1, 4, 6)
    np.testing.assert_allclose(output[0], np.broadcast_to(np.arange(6) + 12, (4, 6)))


@pytest.mark.parametrize("seed", (0, 7))
def test_fused_oracle_matches_reference_bit_for_bit(rpa_vectors, seed):
    inputs = fused_inputs(rpa_vectors, seed)
    output, cache = rpa.rpa_fused(inputs)
    assert output.dtype == BF16 and cache.dtype == BF16
    assert output.shape == (4, 4, 32) and cache.shape == (32, 16, 2, 2, 128)
    np.testing.assert_array_equal(cache.view(np.uint16), rpa_vectors[f"fused/seed{seed}/updated_cache_bf16_bits"])
    expected = bits_to_bf16(rpa_vectors[f"fused/seed{seed}/output_bf16_bits"]).astype(np.float32)
    np.testing.assert_array_equal(output.astype(np.float32), expected)
    assert tuple(inputs[5][:6]) == (7, 2, 19, 4, 25, 1)
    assert not np.array_equal(cache.view(np.uint16), rpa_vectors[f"fused/seed{seed}/cache"])


def test_fused_oracle_mutations_match_reference_and_discriminate(rpa_vectors):
    inputs = fused_inputs(rpa_vectors, 0)
    good_output, good_cache = rpa.rpa_fused(inputs)
    for mutation in rpa.MUTATIONS:
        output, cache = rpa.rpa_fused(inputs, mutation=mutation)
        expected = bits_to_bf16(rpa_vectors[f"fused/seed0/mutation/{mutation}/output_bf16_bits"]).astype(np.float32)
        np.testing.assert_array_equal(output.astype(np.float32), expected)
        cache_equal = np.array_equal(cache.view(np.uint16), good_cache.view(np.uint16))
        assert cache_equal == bool(rpa_vectors[f"fused/seed0/mutation/{mutation}/cache_equal"])
        same = np.allclose(output.astype(np.float32), good_output.astype(np.float32), rtol=0.02, atol=0.02) and cache_equal
        assert not same, mutation


def test_fused_oracle_rejects_non_decode_metadata(rpa_vectors):
    inputs = list(fused_inputs(rpa_vectors, 0))
    inputs[8] = np.zeros(3, np.int32)
    with pytest.raises(ValueError, match="decode-only"):
        rpa.rpa_fused(tuple(inputs))
