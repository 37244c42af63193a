"""Generates the golden fixtures in this directory from the reference checkout.

Run where the reference source tree is available:

    python tests/golden/make_golden.py /path/to/tpu-cake

The reference package cannot be imported normally without jax / xDSL, so this script
 (a) registers a stub ``tpu_cake`` package whose ``__path__`` points at the reference sources, so
     that its ``__init__`` is never executed and numpy-only leaf modules import as they are, and
 (b) for ``tpu_cake.workloads.inkling_rpa`` (whose oracles are plain numpy but whose module imports
     jax and xDSL for unrelated schedule builders) registers inert stand-ins for those imports;
     ``jnp.asarray(x, dtype=jnp.bfloat16)`` is mapped to ml_dtypes' bfloat16, which is the same
     round-to-nearest-even conversion.
The fixtures hold inputs and the reference's own outputs; tests compare the restated oracle under
``oracle/`` with them and never import the reference.
"""

from __future__ import annotations

import importlib
import json
import sys
import types
from pathlib import Path
from unittest import mock

import ml_dtypes
import numpy as np

HERE = Path(__file__).resolve().parent
BF16 = np.dtype(ml_dtypes.bfloat16)


def _install_reference(reference_root: Path) -> None:
    source = reference_root / "src" / "tpu_cake"
    package = types.ModuleType("tpu_cake")
    package.__path__ = [str(source)]
    sys.modules["tpu_cake"] = package
    workloads = types.ModuleType("tpu_cake.workloads")
    workloads.__path__ = [str(source / "workloads")]
    sys.modules["tpu_cake.workloads"] = workloads


def _install_rpa_import_stubs() -> None:
    jnp = types.ModuleType("jax.numpy")
    jnp.bfloat16 = BF16
    jnp.int32 = np.int32
    jnp.float32 = np.float32

    def asarray(value, dtype=None):
        return np.asarray(value).astype(dtype) if dtype is not None else np.asarray(value)

    jnp.asarray = asarray
    jnp.arange = lambda *a, dtype=None: np.arange(*a, dtype=dtype)
    jnp.full = lambda shape, value, dtype=None: np.full(shape, value, dtype=dtype)
    jax = types.ModuleType("jax")
    jax.numpy = jnp
    jax.Array = np.ndarray
    sys.modules["jax"] = jax
    sys.modules["jax.numpy"] = jnp
    for name in (
        "xdsl",
        "xdsl.dialects",
        "xdsl.dialects.builtin",
        "tpu_cake.dialects",
        "tpu_cake.dialects.tpu_schedule",
        "tpu_cake.frontend",
        "tpu_cake.rpa_lowering",
        "tpu_cake.source",
    ):
        sys.modules[name] = mock.MagicMock(name=name)


def _as_u16(array: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(array.astype(BF16)).view(np.uint16)


def make_identity_fixture() -> dict:
    identity = importlib.import_module("tpu_cake.identity")
    out: dict = {"semantic_sha256": {}, "semantic_seed": {}, "array_sha256": {}}
    for parts in (("a",), ("distributed-matmul-workload", "8", "128", "1024", "1024"), ("x", "yz", "é")):
        key = "|".join(parts)
        out["semantic_sha256"][key] = identity.semantic_sha256(*parts)
        out["semantic_seed"][key] = str(identity.semantic_seed(*parts))
    out["legacy"] = identity.semantic_sha256("a", "b", schema=identity.LEGACY_SEMANTIC_IDENTITY_SCHEMA)
    probe = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    out["array_sha256"]["arange24_f32_2x3x4"] = identity.array_sha256(probe)
    out["array_sha256"]["arange24_i32_4x6"] = identity.array_sha256(np.arange(24, dtype=np.int32).reshape(4, 6))
    # The runner's input recipe (runner.py:439-456) for the smallest headline shape.
    workload = identity.semantic_sha256("distributed-matmul-workload", "8", "128", "1024", "1024")
    generator = identity.workload_rng(workload, "device-run", "attempt-0", "inputs")
    lhs = generator.normal(size=(128, 1024)).astype(np.float32).astype(BF16).astype(np.float32)
    rhs = generator.normal(size=(1024, 1024)).astype(np.float32).astype(BF16).astype(np.float32)
    out["matmul_c1_inputs"] = {
        "workload_identity": workload,
        "lhs_sha256": identity.array_sha256(lhs),
        "rhs_sha256": identity.array_sha256(rhs),
        "oracle_sha256": identity.array_sha256(lhs @ rhs),
    }
    return out


def make_confirmation_input_hashes(reference_root: Path) -> dict:
    contract = json.loads((reference_root / "contracts" / "matmul-collective-confirmation-v1.json").read_text())
    found: dict = {}

    def walk(node):
        if isinstance(node, dict):
            for key, value in node.items():
                if key in ("timing_lhs_sha256", "timing_rhs_sha256") and isinstance(value, str):
                    found[key] = value
                walk(value)
        elif isinstance(node, list):
            for value in node:
                walk(value)

    walk(contract)
    return found


def make_structured_patterns() -> None:
    operands = importlib.import_module("tpu_cake.matmul_collective_surface_correctness")
    oracle = importlib.import_module("tpu_cake.matmul_collective_surface_correctness_oracle")
    m, k, n, mesh = 32, 256, 48, 8
    arrays: dict[str, np.ndarray] = {}
    local_k = k // mesh
    for pattern in operands.CORRECTNESS_PATTERNS:
        lhs = np.concatenate(
            [
                operands.make_correctness_operand_shard(
                    pattern, "lhs", m=m, k=k, n=n, k_start=r * local_k, k_stop=(r + 1) * local_k
                )
                for r in range(mesh)
            ],
            axis=1,
        )
        rhs = np.concatenate(
            [
                operands.make_correctness_operand_shard(
                    pattern, "rhs", m=m, k=k, n=n, k_start=r * local_k, k_stop=(r + 1) * local_k
                )
                for r in range(mesh)
            ],
            axis=0,
        )
        arrays[f"{pattern}/lhs_bf16_bits"] = _as_u16(lhs)
        arrays[f"{pattern}/rhs_bf16_bits"] = _as_u16(rhs)
        arrays[f"{pattern}/product_f32"] = oracle.make_correctness_oracle(pattern, m=m, k=k, n=n)
    np.savez_compressed(HERE / "matmul_structured_patterns.npz", **arrays)


def make_rpa_fixtures() -> None:
    _install_rpa_import_stubs()
    rpa = importlib.import_module("tpu_cake.workloads.inkling_rpa")
    arrays: dict[str, np.ndarray] = {}
    # Prototype op (separate caches, dense bias): inputs and output of the reference oracle.
    for seed in (0, 3):
        inputs = rpa.inkling_rpa_inputs(seed)
        names = ("query", "key_cache", "value_cache", "page_table", "sequence_lengths", "bias")
        for name, value in zip(names, inputs, strict=True):
            arrays[f"separate/seed{seed}/{name}"] = np.asarray(value)
        arrays[f"separate/seed{seed}/output"] = rpa.inkling_rpa_reference(*inputs)
    # Closed form pinned by the reference's own test (tests/test_workloads.py:41-61): q = 1, K = 1,
    # V = arange, independent K / V head counts.
    # Fused op: inputs, output, updated cache, and every oracle mutation's output.
    for seed in (0, 7):
        inputs = rpa.inkling_fused_rpa_inputs(seed)
        names = (
            "queries", "keys", "values", "cache", "kv_lengths", "page_indices",
            "cu_q_lens", "cu_kv_lens", "distribution", "relative_states", "relative_projection",
        )
        for name, value in zip(names, inputs, strict=True):
            value = np.asarray(value)
            arrays[f"fused/seed{seed}/{name}"] = _as_u16(value) if value.dtype == BF16 else value
        output, cache = rpa.inkling_fused_rpa_reference(inputs)
        arrays[f"fused/seed{seed}/output_bf16_bits"] = _as_u16(np.asarray(output))
        arrays[f"fused/seed{seed}/updated_cache_bf16_bits"] = _as_u16(np.asarray(cache))
        if seed == 0:
            for mutation in rpa.FusedRpaOracleMutation:
                mutated_output, mutated_cache = rpa.inkling_fused_rpa_reference(inputs, mutation=mutation)
                arrays[f"fused/seed0/mutation/{mutation.value}/output_bf16_bits"] = _as_u16(np.asarray(mutated_output))
                arrays[f"fused/seed0/mutation/{mutation.value}/cache_equal"] = np.asarray(
                    np.array_equal(_as_u16(np.asarray(mutated_cache)), arrays["fused/seed0/updated_cache_bf16_bits"])
                )
    np.savez_compressed(HERE / "rpa_reference_vectors.npz", **arrays)
    # The 2 x 4 sharded surface: its global inputs are 60 MB per seed, so only their hashes are kept
    # (the contract's first correctness seed and a small one).
    identity = importlib.import_module("tpu_cake.identity")
    hashes = {str(seed): [identity.array_sha256(np.asarray(value)) for value in rpa.inkling_sharded_fused_rpa_inputs(seed)]
              for seed in (9423267841700844256, 3)}
    (HERE / "sharded_surface_input_hashes.json").write_text(json.dumps(hashes, indent=2, sort_keys=True) + "\n")


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py PATH_TO_TPU_CAKE_CHECKOUT")
    reference_root = Path(sys.argv[1]).resolve()
    _install_reference(reference_root)
    identity = make_identity_fixture()
    identity["confirmation_contract_input_hashes"] = make_confirmation_input_hashes(reference_root)
    (HERE / "identity_vectors.json").write_text(json.dumps(identity, indent=2, sort_keys=True) + "\n")
    make_structured_patterns()
    make_rpa_fixtures()
    print("wrote", sorted(p.name for p in HERE.iterdir() if p.suffix in (".json", ".npz")))


if __name__ == "__main__":
    main()
