"""A small IR core for the two dialects the hot path speaks.

The reference builds its schedules on xDSL (``dtensor.*``: src/tpu_cake/dialects/
distributed_tensor.py; ``tpu_schedule.*``: src/tpu_cake/dialects/tpu_schedule.py) and identifies
them by the SHA-256 of their canonical generic-format text (src/tpu_cake/canonical.py:44-95).
xDSL is not a dependency here, so this module provides just enough of an IR to build, verify,
print and hash the distributed matmul program and the physical kernel it lowers to: operations with
named properties, typed SSA values, one region per structured op, a generic-MLIR printer with the
reference's canonicalisation rules (symbol names and alloc roles normalised, properties sorted).
The text is MLIR-generic in shape but is not byte-identical to xDSL 0.69's output, so hashes are
identities of this backend's schedules, not replays of the reference's pinned hashes.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Iterable


class VerifyException(ValueError):
    """An operation violates its dialect's rules (same role as xDSL's VerifyException)."""


@dataclass(frozen=True)
class SourceLocation:
    """Where an operation came from (src/tpu_cake/source.py:10-26); never enters the hash."""

    file: str
    line: int
    column: int

    def __str__(self) -> str:
        return f"{self.file}:{self.line}:{self.column}"


ELEMENT_BYTES = {"bf16": 2, "f16": 2, "f32": 4, "i32": 4}


@dataclass(frozen=True)
class DTensorType:
    """Logical distributed tensor: named dimensions, per-dimension sharding axes, and reductions
    still pending over mesh axes (distributed_tensor.py:123-158)."""

    element_type: str
    dimensions: tuple[tuple[str, int], ...]
    sharding: tuple[tuple[str, ...], ...]
    pending_reductions: tuple[tuple[str, str], ...] = ()

    def logical_shape(self) -> tuple[tuple[str, int], ...]:
        return self.dimensions

    def sharding_axes(self) -> tuple[tuple[str, ...], ...]:
        return self.sharding

    def render(self) -> str:
        dims = ", ".join(f'"{name}" = {size}' for name, size in self.dimensions)
        shard = ", ".join("[" + ", ".join(f'"{a}"' for a in axes) + "]" for axes in self.sharding)
        pending = ", ".join(f'"{axis}" = "{op}"' for axis, op in self.pending_reductions)
        return f"!dtensor.tensor<{self.element_type}, [{dims}], [{shard}], [{pending}]>"


@dataclass(frozen=True)
class BufferType:
    """Physical buffer: shape, logical names, memory space, sharding, ownership and the
    [start, end] stage lifetime (tpu_schedule.py:586-624)."""

    shape: tuple[int, ...]
    logical_shape: tuple[str, ...]
    element_type: str
    memory: str = "hbm"  # "hbm" | "vmem" | "smem"
    sharding: tuple[str, ...] = ()
    ownership: str = "local"  # "local" | "external"
    lifetime: tuple[int, int] = (0, 0)

    def nbytes(self) -> int:
        size = ELEMENT_BYTES[self.element_type]
        for extent in self.shape:
            size *= extent
        return size

    def render(self) -> str:
        shape = "x".join(str(v) for v in self.shape)
        names = ", ".join(f'"{n}"' for n in self.logical_shape)
        shard = ", ".join(f'"{a}"' for a in (self.sharding or ("",) * len(self.shape)))
        return (
            f"!tpu_schedule.buffer<memref<{shape}x{self.element_type}>, #tpu_schedule.shape<[{names}]>, "
            f"#tpu_schedule<memory_space {self.memory}>, #tpu_schedule.sharding<[{shard}]>, "
            f"#tpu_schedule<ownership {self.ownership}>, "
            f"#tpu_schedule.lifetime<#builtin.int<{self.lifetime[0]}>, #builtin.int<{self.lifetime[1]}>>>"
        )


@dataclass(frozen=True)
class OpaqueType:
    name: str

    def render(self) -> str:
        return f"!{self.name}"


@dataclass(eq=False)
class Value:
    type: object
    owner: "Operation | Block | None" = None
    index: int = 0


@dataclass(eq=False)
class Block:
    args: list[Value] = field(default_factory=list)
    ops: list["Operation"] = field(default_factory=list)


@dataclass(eq=False)
class Operation:
    name: str
    operands: list[Value] = field(default_factory=list)
    result_types: list[object] = field(default_factory=list)
    properties: dict[str, object] = field(default_factory=dict)
    body: Block | None = None
    location: SourceLocation | None = None

    def __post_init__(self) -> None:
        self.results = [Value(t, self, i) for i, t in enumerate(self.result_types)]

    @property
    def result(self) -> Value:
        return self.results[0]


@dataclass(eq=False)
class Module:
    ops: list[Operation] = field(default_factory=list)

    def verify(self) -> None:
        from . import dialects  # late import: dialects registers its verifiers on import

        for op in self.walk():
            dialects.verify_operation(op)

    def walk(self) -> Iterable[Operation]:
        def visit(op: Operation):
            yield op
            if op.body is not None:
                for inner in op.body.ops:
                    yield from visit(inner)

        for op in self.ops:
            yield from visit(op)


# ----------------------------------------------------------------------------------- printing


def _render_attribute(value: object) -> str:
    if isinstance(value, bool):
        return "true" if value else "false"
    if isinstance(value, int):
        return f"#builtin.int<{value}>"
    if isinstance(value, str):
        return '"' + value.replace("\\", "\\\\").replace('"', '\\"') + '"'
    if isinstance(value, (tuple, list)):
        return "[" + ", ".join(_render_attribute(v) for v in value) + "]"
    if isinstance(value, dict):
        return "{" + ", ".join(f"{k} = {_render_attribute(v)}" for k, v in sorted(value.items())) + "}"
    if hasattr(value, "render"):
        return value.render()
    raise TypeError(f"cannot print attribute {value!r}")


_NORMALISED_SYMBOLS = {"tpu_schedule.kernel": "kernel", "dtensor.program": "program"}


def canonical_text(module: Module) -> str:
    """Generic-format text with the reference's normalisations: properties sorted by key, the
    kernel / program symbol replaced by a fixed name, alloc roles renamed alloc0.. in definition
    order, SSA names numbered in definition order, locations omitted. A physical kernel made only
    of operations the reference's dialect has is printed exactly as the reference prints it
    (``xdsl_text``), so its text and hash are the ones the reference assigns to the same kernel; a
    distributed matmul program is printed in the reference's syntax as well; kernels with this
    backend's own operations use the compact form below."""
    from . import xdsl_text

    if xdsl_text.is_reference_physical_kernel(module):
        return xdsl_text.reference_canonical_text(module)
    if xdsl_text.is_reference_logical_program(module):
        return xdsl_text.reference_logical_text(module)
    names: dict[int, str] = {}
    alloc_roles: dict[str, str] = {}
    lines: list[str] = []

    def name_of(value: Value) -> str:
        key = id(value)
        if key not in names:
            names[key] = f"%{len(names)}"
        return names[key]

    def emit(op: Operation, indent: int) -> None:
        pad = "  " * indent
        properties = dict(op.properties)
        if op.name in _NORMALISED_SYMBOLS and "sym_name" in properties:
            properties["sym_name"] = _NORMALISED_SYMBOLS[op.name]
        if op.name == "tpu_schedule.alloc" and "role" in properties:
            role = properties["role"]
            properties["role"] = alloc_roles.setdefault(role, f"alloc{len(alloc_roles)}")
        results = ", ".join(name_of(r) for r in op.results)
        operands = ", ".join(name_of(v) for v in op.operands)
        props = ", ".join(f"{k} = {_render_attribute(v)}" for k, v in sorted(properties.items()))
        head = f'{pad}{results + " = " if results else ""}"{op.name}"({operands})'
        if props:
            head += f" <{{{props}}}>"
        signature = (
            "(" + ", ".join(v.type.render() for v in op.operands) + ") -> ("
            + ", ".join(t.render() for t in op.result_types) + ")"
        )
        if op.body is None:
            lines.append(f"{head} : {signature}")
            return
        lines.append(f"{head} ({{")
        if op.body.args:
            args = ", ".join(f"{name_of(a)}: {a.type.render()}" for a in op.body.args)
            lines.append(f"{pad}^bb0({args}):")
        for inner in op.body.ops:
            emit(inner, indent + 1)
        lines.append(f"{pad}}}) : {signature}")

    lines.append('"builtin.module"() ({')
    for op in module.ops:
        emit(op, 1)
    lines.append("}) : () -> ()")
    return "\n".join(lines) + "\n"


def schedule_sha256(module: Module) -> str:
    return hashlib.sha256(canonical_text(module).encode()).hexdigest()
