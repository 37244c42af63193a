"""Content identities and seeded input generators shared with the reference.

Same behaviour as src/tpu_cake/identity.py:20-70 of the reference, so that inputs generated here
are bit-identical to the reference's (its committed input hashes reproduce): a semantic hash is a
SHA-256 over a fixed domain tag followed by every part, each prefixed with its byte length as a
big-endian 64-bit integer; a seed is the first eight bytes of that hash; an array hash covers the
dtype string, the repr of the shape and the C-order bytes.
"""

from __future__ import annotations

import hashlib
import json

import numpy as np

SEMANTIC_IDENTITY_SCHEMA = "length-prefixed-v2"
LEGACY_SEMANTIC_IDENTITY_SCHEMA = "separator-v1"
_DOMAIN_TAG = b"tpu-cake-semantic-identity\x00length-prefixed-v2\x00"


def semantic_sha256(*parts: str, schema: str = SEMANTIC_IDENTITY_SCHEMA) -> str:
    if len(parts) == 0 or not all(parts):
        raise ValueError("semantic identity parts must be non-empty")
    if schema == LEGACY_SEMANTIC_IDENTITY_SCHEMA:
        return hashlib.sha256("\x1f".join(parts).encode()).hexdigest()
    if schema != SEMANTIC_IDENTITY_SCHEMA:
        raise ValueError(f"unsupported semantic identity schema: {schema}")
    hasher = hashlib.sha256(_DOMAIN_TAG)
    for part in parts:
        data = part.encode()
        hasher.update(len(data).to_bytes(8, "big") + data)
    return hasher.hexdigest()


def semantic_seed(*parts: str, schema: str = SEMANTIC_IDENTITY_SCHEMA) -> int:
    return int(semantic_sha256(*parts, schema=schema)[:16], 16)


def workload_rng(experiment_id: str, scenario_id: str, attempt: str, tensor_role: str) -> np.random.Generator:
    return np.random.default_rng(semantic_seed(experiment_id, scenario_id, attempt, tensor_role))


def array_sha256(array: np.ndarray) -> str:
    hasher = hashlib.sha256()
    hasher.update(array.dtype.str.encode())
    hasher.update(repr(array.shape).encode())
    hasher.update(array.tobytes(order="C"))
    return hasher.hexdigest()


def json_sha256(value: object) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def text_sha256(text: str) -> str:
    return hashlib.sha256(text.encode()).hexdigest()
