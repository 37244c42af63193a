"""Physical matmul kernels in the reference's own canonical text, byte for byte.

The reference identifies a schedule by the SHA-256 of ``canonical_text(module)``
(src/tpu_cake/canonical.py:76-95, src/tpu_cake/frontend.py:637-638): xDSL 0.69's generic printer
after the normalisations of ``_normalize_semantics`` (properties sorted by name, the kernel symbol
replaced by ``kernel``, allocation roles by ``alloc<i>``). This module renders the 16-operation
kernel that ``lower_distributed_matmul`` emits in exactly that form, including what the compact IR
of this package leaves implicit: the identity ``layout`` parameter of every buffer type
(src/tpu_cake/frontend.py:95), ``ownership kernel`` for local allocations (:83), the semaphore
``slots`` property (src/tpu_cake/dialects/tpu_schedule.py:804-813), the kernel's engine counts
(:3256-3291) and its structured topology, which is a function of mesh and link bandwidth alone
(``rectilinear_topology``, :482-582). The pinned hash of the reference's default program
(tests/test_pallas_lowering.py:54-60) is the known answer this text is tested against.
"""

from __future__ import annotations

import hashlib
from itertools import pairwise, product

from .ir import Block, BufferType, DTensorType, Module, Operation, OpaqueType, Value

TPU7X_CAPACITIES = {"vmem_capacity_bytes": 64 << 20, "smem_capacity_bytes": 16 << 20, "ici_bandwidth_bytes_per_second": 600_000_000_000}


def _int(value: int) -> str:
    return f"#builtin.int<{value}>"


def _string(value: str) -> str:
    return '"' + value.replace("\\", "\\\\").replace('"', '\\"') + '"'


def _array(items) -> str:
    return "[" + ", ".join(items) + "]"


def _buffer(type_: BufferType) -> str:
    rank = len(type_.shape)
    storage = "x".join(str(extent) for extent in type_.shape) + "x" + type_.element_type
    sharding = type_.sharding or ("",) * rank
    ownership = "external" if type_.ownership == "external" else "kernel"
    return (
        f"!tpu_schedule.buffer<memref<{storage}>, #tpu_schedule.shape<{_array(_string(n) for n in type_.logical_shape)}>, "
        f"#tpu_schedule<memory_space {type_.memory}>, #tpu_schedule.sharding<{_array(_string(a) for a in sharding)}>, "
        f"#tpu_schedule.layout<{_array(_int(i) for i in range(rank))}>, #tpu_schedule<ownership {ownership}>, "
        f"#tpu_schedule.lifetime<{_int(type_.lifetime[0])}, {_int(type_.lifetime[1])}>>"
    )


def _type(type_: object) -> str:
    return _buffer(type_) if isinstance(type_, BufferType) else type_.render()


def rectilinear_topology_text(mesh: dict[str, int], bandwidth: dict[str, int], *, channels_per_link: int = 1) -> str:
    """``#tpu_schedule.topology<devices, links, collective plans, transfer plans>`` of a mesh whose
    neighbours along every axis are joined by one link (no wrap-around), as the reference builds it."""
    names, sizes = tuple(mesh), tuple(mesh.values())
    coordinates = tuple(product(*(range(size) for size in sizes)))
    device_of = {coordinate: index for index, coordinate in enumerate(coordinates)}
    devices = [f"#tpu_schedule.device<{_int(index)}, {_array(_int(v) for v in coordinate)}>" for index, coordinate in enumerate(coordinates)]
    links: dict[str, str] = {}
    plans: dict[str, str] = {}
    transfers: dict[str, str] = {}
    for axis_index, axis in enumerate(names):
        if sizes[axis_index] == 1:
            continue
        others = tuple(i for i in range(len(names)) if i != axis_index)
        groups: dict[str, str] = {}
        for group_index, fixed in enumerate(product(*(range(sizes[i]) for i in others))):
            base = dict(zip(others, fixed, strict=True))
            members = tuple(
                device_of[tuple(position if i == axis_index else base[i] for i in range(len(names)))] for position in range(sizes[axis_index])
            )
            route = []
            for source, destination in pairwise(members):
                low, high = min(source, destination), max(source, destination)
                link_id = f"link:{low}-{high}"
                links.setdefault(
                    link_id, f"#tpu_schedule.link<{_string(link_id)}, {_int(low)}, {_int(high)}, {_int(bandwidth[axis])}, {_int(channels_per_link)}>"
                )
                route.append(link_id)
            group_id = f"group:{axis}:{group_index}"
            groups[group_id] = (
                f"#tpu_schedule.collective_group<{_string(group_id)}, {_array(_int(d) for d in sorted(members))}, "
                f"{_array(_string(l) for l in sorted(route))}>"
            )
        plan_id = f"axis:{axis}"
        plans[plan_id] = f"#tpu_schedule.collective_plan<{_string(plan_id)}, {_string(axis)}, {_array(groups[g] for g in sorted(groups))}>"
        for direction in (-1, 1):
            routes: dict[str, str] = {}
            for coordinate, source in device_of.items():
                peer = list(coordinate)
                peer[axis_index] += direction
                if not 0 <= peer[axis_index] < sizes[axis_index]:
                    continue
                destination = device_of[tuple(peer)]
                low, high = min(source, destination), max(source, destination)
                route_id = f"route:{source}->{destination}"
                routes[route_id] = (
                    f"#tpu_schedule.transfer_route<{_string(route_id)}, {_int(source)}, {_int(destination)}, {_array([_string(f'link:{low}-{high}')])}>"
                )
            transfer_id = f"shift:{axis}:{direction:+d}"
            transfers[transfer_id] = f"#tpu_schedule.transfer_plan<{_string(transfer_id)}, {_array(routes[r] for r in sorted(routes))}>"
    return (
        f"#tpu_schedule.topology<{_array(devices)}, {_array(links[k] for k in sorted(links))}, "
        f"{_array(plans[k] for k in sorted(plans))}, {_array(transfers[k] for k in sorted(transfers))}>"
    )


def _kernel_properties(kernel: Operation) -> dict[str, str]:
    p = kernel.properties
    mesh = dict(zip(p["mesh_axis_names"], p["mesh_axis_sizes"], strict=True))
    bandwidth = {}
    for entry in p["topology"]:
        axis, _, value = entry.rpartition(":")
        bandwidth[axis] = int(value)
    optional = {}
    if "argument_modes" in p:
        optional["argument_modes"] = _array(_string(mode) for mode in p["argument_modes"])
    return {
        **optional,
        "dma_engine_count": _int(2),
        "ici_link_count": _int(1),
        "mesh_axis_names": _array(_string(axis) for axis in mesh),
        "mesh_axis_sizes": _array(_int(size) for size in mesh.values()),
        "mxu_count": _int(1),
        "physical_schema": _string(p["physical_schema"]),
        "remote_dma_engine_count": _int(1),
        "smem_capacity_bytes": _int(p["smem_capacity_bytes"]),
        "sym_name": _string("kernel"),
        "target": _string(p["target"]),
        "topology": rectilinear_topology_text(mesh, bandwidth),
        "topology_authority": _string(p["topology_authority"]),
        "vector_unit_count": _int(1),
        "vmem_capacity_bytes": _int(p["vmem_capacity_bytes"]),
    }


def _operation_properties(op: Operation, alloc_index: list[int]) -> dict[str, str]:
    p = op.properties
    if op.name == "tpu_schedule.alloc":
        role = f"alloc{alloc_index[0]}"
        alloc_index[0] += 1
        return {"role": _string(role)}
    if op.name == "tpu_schedule.semaphore_alloc":
        return {"slots": _int(int(p.get("slots", 1)))}
    if op.name == "tpu_schedule.collective":
        rendered = {
            "collective_plan": _string(p["collective_plan"]),
            "concat_dimension": _int(p["concat_dimension"]),
            "group_size": _int(p["group_size"]),
            "kind": f"#tpu_schedule<collective_kind {p['kind']}>",
            "mesh_axis": _string(p["mesh_axis"]),
            "reducer": _string(p["reducer"]),
            "split_dimension": _int(p["split_dimension"]),
            "stage": _int(p["stage"]),
        }
        if "implementation" in p:
            rendered["implementation"] = f"#tpu_schedule<collective_implementation {p['implementation']}>"
        return rendered
    return {key: _generic_attribute(op, key, value) for key, value in p.items()}


def _generic_attribute(op: Operation, key: str, value: object) -> str:
    """Integers are ``IntAttr``, strings ``StringAttr``, sequences ``ArrayAttr`` of those."""
    if isinstance(value, bool):
        raise ValueError(f"XDSL_TEXT_UNSUPPORTED_PROPERTY operation={op.name} property={key}")
    if isinstance(value, int):
        return _int(value)
    if isinstance(value, str):
        return _string(value)
    if isinstance(value, (tuple, list)):
        return _array(_generic_attribute(op, key, item) for item in value)
    raise ValueError(f"XDSL_TEXT_UNSUPPORTED_PROPERTY operation={op.name} property={key}")


_SUPPORTED = {
    "tpu_schedule.alloc", "tpu_schedule.semaphore_alloc", "tpu_schedule.dma_start", "tpu_schedule.dma_wait",
    "tpu_schedule.mxu_matmul", "tpu_schedule.collective", "tpu_schedule.ragged_paged_attention",
    "tpu_schedule.fused_ragged_paged_attention", "tpu_schedule.rpa_decode_core",
}


def is_reference_physical_kernel(module: Module) -> bool:
    """One ``tpu_schedule.kernel`` whose body holds only operations of the reference's dialect."""
    if len(module.ops) != 1 or module.ops[0].name != "tpu_schedule.kernel" or module.ops[0].body is None:
        return False
    return all(op.name in _SUPPORTED or op.name == "tpu_schedule.yield" for op in module.ops[0].body.ops)


def reference_canonical_text(module: Module) -> str:
    """The text ``canonical_text`` of the reference prints for this physical matmul kernel."""
    if len(module.ops) != 1 or module.ops[0].name != "tpu_schedule.kernel" or module.ops[0].body is None:
        raise ValueError("XDSL_TEXT_UNSUPPORTED_MODULE expected one tpu_schedule.kernel")
    kernel = module.ops[0]
    names: dict[int, str] = {}

    def name_of(value: Value) -> str:
        return names.setdefault(id(value), f"%{len(names)}")

    def signature(op: Operation) -> str:
        operands = ", ".join(_type(v.type) for v in op.operands)
        results = [_type(t) for t in op.result_types]
        return f"({operands}) -> " + (results[0] if len(results) == 1 else "(" + ", ".join(results) + ")")

    def properties(rendered: dict[str, str]) -> str:
        return " <{" + ", ".join(f"{key} = {rendered[key]}" for key in sorted(rendered)) + "}>" if rendered else ""

    lines = ['"builtin.module"() ({', f'  "tpu_schedule.kernel"(){properties(_kernel_properties(kernel))} ({{']
    lines.append("  ^bb0(" + ", ".join(f"{name_of(a)}: {_type(a.type)}" for a in kernel.body.args) + "):")
    alloc_index = [0]
    for op in kernel.body.ops:
        if op.name == "tpu_schedule.yield":
            continue
        if op.name not in _SUPPORTED:
            raise ValueError(f"XDSL_TEXT_UNSUPPORTED_OPERATION operation={op.name}")
        results = ", ".join(name_of(r) for r in op.results)
        operands = ", ".join(name_of(v) for v in op.operands)
        head = f'    {results + " = " if results else ""}"{op.name}"({operands})'
        lines.append(f"{head}{properties(_operation_properties(op, alloc_index))} : {signature(op)}")
    lines.append('    "tpu_schedule.yield"() : () -> ()')
    lines.append("  }) : () -> ()")
    lines.append("}) : () -> ()")
    return "\n".join(lines) + "\n"


def reference_schedule_sha256(module: Module) -> str:
    return hashlib.sha256(reference_canonical_text(module).encode()).hexdigest()


# ------------------------------------------------------------------------------ logical programs

_LOGICAL_OPS = {"dtensor.einsum_local", "dtensor.reduce_scatter", "dtensor.return"}


def is_reference_logical_program(module: Module) -> bool:
    """One ``dtensor.program`` made of the operations the distributed matmul uses."""
    if len(module.ops) != 1 or module.ops[0].name != "dtensor.program" or module.ops[0].body is None:
        return False
    return all(op.name in _LOGICAL_OPS for op in module.ops[0].body.ops)


def _dtensor(type_: DTensorType) -> str:
    dimensions = _array(f"#dtensor.dimension<{_string(name)}, {_int(size)}>" for name, size in type_.dimensions)
    sharding = _array(f"#dtensor.axis_list<{_array(_string(a) for a in axes)}>" for axes in type_.sharding)
    pending = f"#dtensor.pending_reductions<{_array(_string(a) for a, _ in type_.pending_reductions)}, {_array(_string(r) for _, r in type_.pending_reductions)}>"
    return f"!dtensor.tensor<{type_.element_type}, {dimensions}, #dtensor.sharding<{sharding}>, {pending}>"


def reference_logical_text(module: Module) -> str:
    """A distributed matmul program in the reference's generic syntax, as its dialect definitions
    (src/tpu_cake/dialects/distributed_tensor.py:55-160, 1020-1043, 1202-1226, 1421-1447) and the
    printer conventions confirmed on the physical kernels give it: the mesh as one ``#dtensor.mesh``
    property, tensor types with ``#dtensor.dimension`` / ``axis_list`` / ``pending_reductions``
    parameters, the einsum's ``accumulation_type``. The reference pins no hash of a logical program,
    so unlike the physical text this one has no known answer to be checked against."""
    program = module.ops[0]
    p = program.properties
    names: dict[int, str] = {}

    def name_of(value: Value) -> str:
        return names.setdefault(id(value), f"%{len(names)}")

    mesh = f"#dtensor.mesh<{_array(_string(a) for a in p['mesh_axis_names'])}, {_array(_int(v) for v in p['mesh_axis_sizes'])}>"
    lines = ['"builtin.module"() ({', f'  "dtensor.program"() <{{mesh = {mesh}, sym_name = "program"}}> ({{']
    lines.append("  ^bb0(" + ", ".join(f"{name_of(a)}: {_dtensor(a.type)}" for a in program.body.args) + "):")
    for op in program.body.ops:
        rendered = {key: _generic_attribute(op, key, value) for key, value in op.properties.items()}
        if op.name == "dtensor.einsum_local":
            rendered["accumulation_type"] = op.result_types[0].element_type
        results = ", ".join(name_of(r) for r in op.results)
        operands = ", ".join(name_of(v) for v in op.operands)
        properties = " <{" + ", ".join(f"{key} = {rendered[key]}" for key in sorted(rendered)) + "}>" if rendered else ""
        result_types = [_dtensor(t) for t in op.result_types]
        signature = "(" + ", ".join(_dtensor(v.type) for v in op.operands) + ") -> " + (result_types[0] if len(result_types) == 1 else "(" + ", ".join(result_types) + ")")
        lines.append(f'    {results + " = " if results else ""}"{op.name}"({operands}){properties} : {signature}')
    lines.append("  }) : () -> ()")
    lines.append("}) : () -> ()")
    return "\n".join(lines) + "\n"


# ----------------------------------------------------------------------------------- parsing


class _Param:
    """``#dialect.name<parameters>`` as read from the text."""

    def __init__(self, name: str, parameters: tuple):
        self.name = name
        self.parameters = parameters


class _Enum:
    """``#dialect<name value>``."""

    def __init__(self, name: str, value: str):
        self.name = name
        self.value = value


class _Reader:
    def __init__(self, text: str):
        self.text = text
        self.at = 0

    def fail(self, what: str) -> ValueError:
        line = self.text.count("\n", 0, self.at) + 1
        return ValueError(f"XDSL_TEXT_PARSE_ERROR line={line} expected={what}")

    def spaces(self) -> None:
        while self.at < len(self.text) and self.text[self.at] in " \n":
            self.at += 1

    def peek(self, token: str) -> bool:
        self.spaces()
        return self.text.startswith(token, self.at)

    def take(self, token: str) -> bool:
        if self.peek(token):
            self.at += len(token)
            return True
        return False

    def expect(self, token: str) -> None:
        if not self.take(token):
            raise self.fail(repr(token))

    def word(self, extra: str = "") -> str:
        self.spaces()
        start = self.at
        while self.at < len(self.text) and (self.text[self.at].isalnum() or self.text[self.at] in "_" + extra):
            self.at += 1
        if start == self.at:
            raise self.fail("a name")
        return self.text[start:self.at]

    def integer(self) -> int:
        self.spaces()
        start = self.at
        if self.at < len(self.text) and self.text[self.at] == "-":
            self.at += 1
        while self.at < len(self.text) and self.text[self.at].isdigit():
            self.at += 1
        try:
            return int(self.text[start:self.at])
        except ValueError:
            raise self.fail("an integer") from None

    def string(self) -> str:
        self.expect('"')
        out = []
        while True:
            if self.at >= len(self.text):
                raise self.fail("a closing quote")
            c = self.text[self.at]
            self.at += 1
            if c == '"':
                return "".join(out)
            if c == "\\":
                if self.at >= len(self.text):
                    raise self.fail("an escaped character")
                out.append(self.text[self.at])
                self.at += 1
            else:
                out.append(c)

    def value_name(self) -> str:
        self.expect("%")
        return "%" + self.word()

    def list_of(self, item, close: str) -> list:
        items = []
        if self.take(close):
            return items
        while True:
            items.append(item())
            if self.take(close):
                return items
            self.expect(",")

    def attribute(self):
        if self.peek('"'):
            return self.string()
        if self.take("["):
            return tuple(self.list_of(self.attribute, "]"))
        if self.take("#builtin.int<"):
            value = self.integer()
            self.expect(">")
            return value
        if self.take("memref<"):
            return self.memref()
        if self.take("#"):
            dialect = self.word()
            if self.take("<"):
                name = self.word()
                value = self.word()
                self.expect(">")
                return _Enum(f"{dialect}.{name}", value)
            self.expect(".")
            name = self.word()
            parameters = tuple(self.list_of(self.attribute, ">")) if self.take("<") else ()
            return _Param(f"{dialect}.{name}", parameters)
        raise self.fail("an attribute")

    def memref(self) -> tuple[tuple[int, ...], str]:
        shape = []
        while True:
            self.spaces()
            if self.text[self.at].isdigit():
                shape.append(self.integer())
                self.expect("x")
            else:
                element = self.word()
                self.expect(">")
                return tuple(shape), element

    def type_(self):
        self.expect("!")
        name = self.word(".")
        if name != "tpu_schedule.buffer":
            return OpaqueType(name)
        self.expect("<")
        parameters = self.list_of(self.attribute, ">")
        return _buffer_from(parameters, self)


def _single(parameter, name: str, reader: _Reader):
    if not isinstance(parameter, _Param) or parameter.name != name or len(parameter.parameters) != 1:
        raise reader.fail(f"#{name}<...>")
    return parameter.parameters[0]


def _buffer_from(parameters: list, reader: _Reader) -> BufferType:
    if len(parameters) != 7 or not isinstance(parameters[0], tuple):
        raise reader.fail("the seven parameters of !tpu_schedule.buffer")
    (shape, element), names, space, sharding, layout, ownership, lifetime = parameters
    names = _single(names, "tpu_schedule.shape", reader)
    sharding = _single(sharding, "tpu_schedule.sharding", reader)
    layout = _single(layout, "tpu_schedule.layout", reader)
    if not isinstance(space, _Enum) or space.name != "tpu_schedule.memory_space" or not isinstance(ownership, _Enum) or ownership.name != "tpu_schedule.ownership":
        raise reader.fail("memory space and ownership of a buffer")
    if not isinstance(lifetime, _Param) or lifetime.name != "tpu_schedule.lifetime" or len(lifetime.parameters) != 2:
        raise reader.fail("#tpu_schedule.lifetime<start, end>")
    if tuple(layout) != tuple(range(len(shape))):
        raise ValueError(f"XDSL_TEXT_UNSUPPORTED_LAYOUT layout={tuple(layout)}")
    if ownership.value not in ("external", "kernel"):
        raise ValueError(f"XDSL_TEXT_UNSUPPORTED_OWNERSHIP ownership={ownership.value}")
    return BufferType(
        shape=tuple(shape), logical_shape=tuple(names), element_type=element, memory=space.value, sharding=tuple(sharding),
        ownership="external" if ownership.value == "external" else "local", lifetime=(int(lifetime.parameters[0]), int(lifetime.parameters[1])),
    )


_DEFAULT_ENGINES = {"dma_engine_count": 2, "ici_link_count": 1, "mxu_count": 1, "remote_dma_engine_count": 1, "vector_unit_count": 1}


def _axis_bandwidths(topology, mesh: dict[str, int], reader: _Reader) -> dict[str, int]:
    if not isinstance(topology, _Param) or topology.name != "tpu_schedule.topology" or len(topology.parameters) != 4:
        raise reader.fail("#tpu_schedule.topology<devices, links, collective plans, transfer plans>")
    _, links, plans, _ = topology.parameters
    by_id = {link.parameters[0]: int(link.parameters[3]) for link in links if isinstance(link, _Param) and len(link.parameters) == 5}
    bandwidth = {}
    for plan in plans:
        if not isinstance(plan, _Param) or len(plan.parameters) != 3:
            raise reader.fail("#tpu_schedule.collective_plan<id, axis, groups>")
        _, axis, groups = plan.parameters
        routes = groups[0].parameters[2] if groups and isinstance(groups[0], _Param) and len(groups[0].parameters) == 3 else ()
        if routes and routes[0] in by_id:
            bandwidth[axis] = by_id[routes[0]]
    for axis, size in mesh.items():
        if axis not in bandwidth:
            if size != 1:
                raise ValueError(f"XDSL_TEXT_TOPOLOGY_WITHOUT_LINKS axis={axis}")
            bandwidth[axis] = 1  # an axis of one device has no link, and none is printed
    return bandwidth


def _parse_physical_kernel(text: str) -> Module:
    """Reads the canonical text of a physical kernel -- as the reference writes it to
    ``physical.xdsl`` -- into this package's IR. Only what prints back to the same bytes is
    accepted: rectilinear topologies, default engine counts, identity layouts; anything else is
    refused with an ``XDSL_TEXT_*`` error rather than approximated."""
    reader = _Reader(text)
    reader.expect('"builtin.module"() ({')
    reader.expect('"tpu_schedule.kernel"()')
    reader.expect("<{")
    raw = dict(reader.list_of(lambda: _property(reader), "}>"))
    for key, default in _DEFAULT_ENGINES.items():
        if raw.get(key) != default:
            raise ValueError(f"XDSL_TEXT_UNSUPPORTED_ENGINE_COUNT property={key} value={raw.get(key)}")
    try:
        mesh = dict(zip(raw["mesh_axis_names"], raw["mesh_axis_sizes"], strict=True))
        bandwidth = _axis_bandwidths(raw["topology"], mesh, reader)
        properties = {
            "sym_name": raw["sym_name"], "target": raw["target"], "vmem_capacity_bytes": raw["vmem_capacity_bytes"],
            "smem_capacity_bytes": raw["smem_capacity_bytes"], "mesh_axis_names": tuple(mesh), "mesh_axis_sizes": tuple(mesh.values()),
            "topology": tuple(f"{axis}:{bandwidth[axis]}" for axis in mesh), "physical_schema": raw["physical_schema"],
            "topology_authority": raw["topology_authority"],
        }
    except KeyError as missing:
        raise ValueError(f"XDSL_TEXT_MISSING_KERNEL_PROPERTY property={missing.args[0]}") from None
    if "argument_modes" in raw:
        properties["argument_modes"] = tuple(raw["argument_modes"])
    reader.expect("({")
    values: dict[str, Value] = {}
    block = Block()
    if reader.take("^bb0("):
        def argument():
            name = reader.value_name()
            reader.expect(":")
            value = Value(reader.type_(), block, len(block.args))
            block.args.append(value)
            values[name] = value
        reader.list_of(argument, ")")
        reader.expect(":")
    while not reader.peek("})"):
        results = []
        if reader.peek("%"):
            results = reader.list_of(reader.value_name, "=")
        name = reader.string()
        reader.expect("(")
        operand_names = reader.list_of(reader.value_name, ")")
        op_properties = dict(reader.list_of(lambda: _property(reader), "}>")) if reader.take("<{") else {}
        reader.expect(":")
        reader.expect("(")
        reader.list_of(reader.type_, ")")
        reader.expect("->")
        result_types = reader.list_of(reader.type_, ")") if reader.take("(") else [reader.type_()]
        try:
            operands = [values[n] for n in operand_names]
        except KeyError as unknown:
            raise ValueError(f"XDSL_TEXT_UNDEFINED_VALUE value={unknown.args[0]}") from None
        if name == "tpu_schedule.semaphore_alloc" and op_properties.get("slots") == 1:
            del op_properties["slots"]
        for key, value in op_properties.items():
            if isinstance(value, _Enum):
                op_properties[key] = value.value
        op = Operation(name, operands, result_types, op_properties)
        if len(results) != len(op.results):
            raise reader.fail("as many result names as result types")
        for result_name, result in zip(results, op.results):
            values[result_name] = result
        block.ops.append(op)
    reader.expect("}) : () -> ()")
    reader.expect("}) : () -> ()")
    reader.spaces()
    if reader.at != len(text):
        raise reader.fail("the end of the text")
    module = Module([Operation("tpu_schedule.kernel", properties=properties, body=block)])
    if not is_reference_physical_kernel(module):
        unknown = next(op.name for op in block.ops if op.name not in _SUPPORTED and op.name != "tpu_schedule.yield")
        raise ValueError(f"XDSL_TEXT_UNSUPPORTED_OPERATION operation={unknown}")
    if reference_canonical_text(module) != text:
        raise ValueError("XDSL_TEXT_NOT_CANONICAL the text does not print back to the same bytes")
    return module


def _property(reader: _Reader) -> tuple[str, object]:
    key = reader.word()
    reader.expect("=")
    return key, reader.attribute()


def _dtensor_from(reader: _Reader) -> DTensorType:
    reader.expect("!dtensor.tensor<")
    element = reader.word()
    reader.expect(",")
    dimensions = reader.attribute()
    reader.expect(",")
    sharding = reader.attribute()
    reader.expect(",")
    pending = reader.attribute()
    reader.expect(">")
    try:
        axes = _single(sharding, "dtensor.sharding", reader)
        if not isinstance(pending, _Param) or pending.name != "dtensor.pending_reductions" or len(pending.parameters) != 2:
            raise reader.fail("#dtensor.pending_reductions<axes, reducers>")
        return DTensorType(
            element_type=element,
            dimensions=tuple((d.parameters[0], int(d.parameters[1])) for d in dimensions),
            sharding=tuple(tuple(_single(a, "dtensor.axis_list", reader)) for a in axes),
            pending_reductions=tuple(zip(pending.parameters[0], pending.parameters[1], strict=True)),
        )
    except (AttributeError, IndexError, TypeError) as malformed:
        raise reader.fail("a !dtensor.tensor type") from malformed


def _parse_logical_program(text: str) -> Module:
    """Reads a distributed matmul program in the syntax ``reference_logical_text`` prints; as for
    kernels, only text that prints back to the same bytes is accepted."""
    reader = _Reader(text)
    reader.expect('"builtin.module"() ({')
    reader.expect('"dtensor.program"()')
    reader.expect("<{")
    raw = dict(reader.list_of(lambda: _property(reader), "}>"))
    mesh = raw.get("mesh")
    if not isinstance(mesh, _Param) or mesh.name != "dtensor.mesh" or len(mesh.parameters) != 2 or "sym_name" not in raw:
        raise reader.fail("the mesh and sym_name properties of dtensor.program")
    properties = {"sym_name": raw["sym_name"], "mesh_axis_names": tuple(mesh.parameters[0]), "mesh_axis_sizes": tuple(mesh.parameters[1])}
    reader.expect("({")
    values: dict[str, Value] = {}
    block = Block()
    if reader.take("^bb0("):
        def argument():
            name = reader.value_name()
            reader.expect(":")
            value = Value(_dtensor_from(reader), block, len(block.args))
            block.args.append(value)
            values[name] = value
        reader.list_of(argument, ")")
        reader.expect(":")
    while not reader.peek("})"):
        results = reader.list_of(reader.value_name, "=") if reader.peek("%") else []
        name = reader.string()
        reader.expect("(")
        operand_names = reader.list_of(reader.value_name, ")")
        op_properties = {}
        if reader.take("<{"):
            def logical_property():
                key = reader.word()
                reader.expect("=")
                return key, (reader.word() if key == "accumulation_type" else reader.attribute())
            op_properties = dict(reader.list_of(logical_property, "}>"))
        reader.expect(":")
        reader.expect("(")
        reader.list_of(lambda: _dtensor_from(reader), ")")
        reader.expect("->")
        result_types = reader.list_of(lambda: _dtensor_from(reader), ")") if reader.take("(") else [_dtensor_from(reader)]
        accumulation = op_properties.pop("accumulation_type", None)
        if accumulation is not None and (not result_types or accumulation != result_types[0].element_type):
            raise ValueError(f"XDSL_TEXT_UNSUPPORTED_ACCUMULATION accumulation_type={accumulation}")
        try:
            operands = [values[n] for n in operand_names]
        except KeyError as unknown:
            raise ValueError(f"XDSL_TEXT_UNDEFINED_VALUE value={unknown.args[0]}") from None
        op = Operation(name, operands, result_types, op_properties)
        if len(results) != len(op.results):
            raise reader.fail("as many result names as result types")
        for result_name, result in zip(results, op.results):
            values[result_name] = result
        block.ops.append(op)
    reader.expect("}) : () -> ()")
    reader.expect("}) : () -> ()")
    reader.spaces()
    if reader.at != len(text):
        raise reader.fail("the end of the text")
    module = Module([Operation("dtensor.program", properties=properties, body=block)])
    if not is_reference_logical_program(module):
        unknown = next(op.name for op in block.ops if op.name not in _LOGICAL_OPS)
        raise ValueError(f"XDSL_TEXT_UNSUPPORTED_OPERATION operation={unknown}")
    if reference_logical_text(module) != text:
        raise ValueError("XDSL_TEXT_NOT_CANONICAL the text does not print back to the same bytes")
    return module


def _guarded(parse, text: str) -> Module:
    """Text that is cut short or has an attribute of the wrong kind where a number, a name or a list
    is due ends in the same kind of error as any other text that is not a canonical schedule."""
    try:
        return parse(text)
    except ValueError:
        raise
    except (AttributeError, IndexError, KeyError, TypeError) as malformed:
        raise ValueError(f"XDSL_TEXT_MALFORMED {type(malformed).__name__}: {malformed}") from malformed


def parse_reference_physical_kernel(text: str) -> Module:
    return _guarded(_parse_physical_kernel, text)


def parse_reference_logical_program(text: str) -> Module:
    return _guarded(_parse_logical_program, text)


parse_reference_physical_kernel.__doc__ = _parse_physical_kernel.__doc__
parse_reference_logical_program.__doc__ = _parse_logical_program.__doc__


def parse_reference_module(text: str) -> Module:
    """A saved schedule of either level (the reference's ``_parse_schedule``, src/tpu_cake/cli.py:419-429)."""
    lines = text.split("\n", 2)
    if len(lines) > 1 and lines[1].lstrip().startswith('"dtensor.program"'):
        return parse_reference_logical_program(text)
    return parse_reference_physical_kernel(text)
