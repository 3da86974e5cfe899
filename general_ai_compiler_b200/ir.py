"""Graph types of the host API: ``TensorSpec``, ``Node``, ``Graph``.

The names, fields and JSON keys are those of GAC's canonical graph
(``src/gac/core/ir.py``: ``TensorSpec`` :60, ``Node`` :122, ``Graph`` :180), so
a graph serialised by either side loads on the other.  The checks are written
from that contract:

* a dimension is a non-negative integer, a non-empty symbol, or ``None``;
* every name (graph, value, node id, op) is a non-empty string;
* a node has at least one output and names each output once;
* a graph is in static single assignment form and topological order: a value
  is defined exactly once (as an input, a constant or a node output) before
  its first use, and every graph output is defined;
* ``value_specs`` may only describe values the graph defines.

Everything that breaks a rule raises ``ValidationError``.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field
from typing import Any, Iterable, Mapping, Union

import numpy as np

from .errors import ValidationError

Dim = Union[int, str, None]
SCHEMA_VERSION = 1


def _require(ok: bool, message: str) -> None:
    if not ok:
        raise ValidationError(message)


def _is_name(value: object) -> bool:
    return isinstance(value, str) and value != ""


def _names(values: Iterable, what: str) -> tuple:
    out = tuple(values)
    for v in out:
        _require(_is_name(v), f"{what}: {v!r} is not a non-empty string")
    return out


def _canonical_dim(d: object) -> Dim:
    if d is None or _is_name(d):
        return d
    integral = isinstance(d, (int, np.integer)) and not isinstance(d, (bool, np.bool_))
    _require(integral and int(d) >= 0, f"dimension {d!r} is neither a non-negative integer, a symbol nor None")
    return int(d)


def _jsonable(v: Any) -> Any:
    """Attribute / metadata values as plain JSON types (NumPy scalars and arrays unwrapped, tuples as lists)."""
    if v is None or isinstance(v, (str, bool, int, float)):
        return v
    if isinstance(v, np.generic):
        return v.item()
    if isinstance(v, np.ndarray):
        return v.tolist()
    if isinstance(v, Mapping):
        return {str(key): _jsonable(item) for key, item in v.items()}
    if isinstance(v, (tuple, list)):
        return [_jsonable(item) for item in v]
    raise ValidationError(f"a value of type {type(v).__name__} has no JSON form")


@dataclass(frozen=True)
class TensorSpec:
    """Logical tensor type: shape (ints, symbols or None), NumPy dtype name, layout tag."""

    shape: tuple
    dtype: Any
    layout: str = "contiguous"

    def __post_init__(self) -> None:
        try:
            dtype_name = np.dtype(self.dtype).name
        except TypeError as exc:
            raise ValidationError(f"{self.dtype!r} does not name a NumPy dtype") from exc
        _require(_is_name(self.layout), "the layout tag of a tensor is a non-empty string")
        object.__setattr__(self, "dtype", dtype_name)
        object.__setattr__(self, "shape", tuple(map(_canonical_dim, self.shape)))

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def is_static(self) -> bool:
        return all(type(d) is int for d in self.shape)

    @property
    def numel(self):
        return int(np.prod(self.shape, dtype=np.int64)) if self.is_static else None

    @property
    def nbytes(self):
        return self.numel * np.dtype(self.dtype).itemsize if self.is_static else None

    def to_dict(self) -> dict:
        return {"shape": list(self.shape), "dtype": self.dtype, "layout": self.layout}

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "TensorSpec":
        try:
            return cls(tuple(data["shape"]), data["dtype"], data.get("layout", "contiguous"))
        except (KeyError, TypeError, AttributeError) as exc:
            raise ValidationError(f"not a tensor spec: {data!r}") from exc


@dataclass(frozen=True)
class Node:
    """One pure operator application; ``inputs``/``outputs`` are value names."""

    id: str
    op: str
    inputs: tuple
    outputs: tuple
    attrs: dict = field(default_factory=dict)
    source_nodes: tuple = ()

    def __post_init__(self) -> None:
        _require(_is_name(self.id), f"a node id is a non-empty string, got {self.id!r}")
        where = f"node {self.id!r}"
        _require(_is_name(self.op), f"{where}: the op is a non-empty string, got {self.op!r}")
        frozen = {
            "inputs": _names(self.inputs, f"{where} inputs"),
            "outputs": _names(self.outputs, f"{where} outputs"),
            # provenance: the nodes of the original graph this one stands for (itself unless a pass merged some)
            "source_nodes": _names(self.source_nodes, f"{where} source_nodes") or (self.id,),
            "attrs": dict(self.attrs),
        }
        outs = frozen["outputs"]
        _require(len(outs) > 0, f"{where}: at least one output is needed")
        _require(len(set(outs)) == len(outs), f"{where}: an output name appears twice in {list(outs)}")
        for key, value in frozen.items():
            object.__setattr__(self, key, value)

    def to_dict(self) -> dict:
        return {"id": self.id, "op": self.op, "inputs": list(self.inputs), "outputs": list(self.outputs),
                "attrs": _jsonable(self.attrs), "source_nodes": list(self.source_nodes)}

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Node":
        try:
            return cls(data["id"], data["op"], tuple(data.get("inputs", ())), tuple(data["outputs"]),
                       dict(data.get("attrs", {})), tuple(data.get("source_nodes", ())))
        except (KeyError, TypeError, AttributeError) as exc:
            raise ValidationError(f"not a node: {data!r}") from exc


@dataclass
class Graph:
    """Topologically ordered tensor graph with named inputs, constants and outputs."""

    name: str
    inputs: dict
    outputs: tuple
    nodes: list
    constants: dict = field(default_factory=dict)
    value_specs: dict = field(default_factory=dict)
    metadata: dict = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.inputs = dict(self.inputs)
        self.outputs = tuple(self.outputs)
        self.nodes = list(self.nodes)
        self.constants = {name: np.asarray(array) for name, array in self.constants.items()}
        self.metadata = copy.deepcopy(dict(self.metadata))
        # inputs and constants describe themselves unless the caller already gave a spec
        specs = {name: TensorSpec(array.shape, array.dtype) for name, array in self.constants.items()}
        specs.update(self.inputs)
        specs.update(self.value_specs)
        self.value_specs = specs

    def clone(self) -> "Graph":
        """A graph that shares no mutable state with this one (nodes and specs are immutable and shared)."""
        constants = {name: array.copy() for name, array in self.constants.items()}
        return Graph(self.name, self.inputs, self.outputs, self.nodes, constants, self.value_specs, self.metadata)

    def _definitions(self) -> dict:
        """value name -> what defines it ("input", "constant" or "node <id>"); raises on a second definition."""
        table: dict = {}

        def define(value: object, by: str) -> None:
            _require(_is_name(value), f"graph {self.name!r}: {by} defines {value!r}, which is not a non-empty string")
            _require(value not in table, f"graph {self.name!r}: {value!r} is defined by {table.get(value)} and again by {by}")
            table[value] = by

        for value in self.inputs:
            define(value, "input")
        for value in self.constants:
            define(value, "constant")
        ids = set()
        for node in self.nodes:
            _require(isinstance(node, Node), f"graph {self.name!r}: {node!r} is not a Node")
            _require(node.id not in ids, f"graph {self.name!r}: two nodes share the id {node.id!r}")
            ids.add(node.id)
            for value in node.inputs:   # topological order: operands exist before the node that reads them
                _require(value in table, f"graph {self.name!r}: node {node.id!r} reads {value!r} before anything defines it")
            for value in node.outputs:
                define(value, f"node {node.id!r}")
        return table

    def validate(self) -> None:
        """Check the rules in the module docstring; returns None or raises ``ValidationError``."""
        _require(_is_name(self.name), f"a graph name is a non-empty string, got {self.name!r}")
        _require(len(self.outputs) > 0, f"graph {self.name!r} has no outputs")
        table = self._definitions()
        for value in self.outputs:
            _require(value in table, f"graph {self.name!r}: output {value!r} is not defined by any input, constant or node")
        typed = dict(self.inputs)
        typed.update(self.value_specs)
        for value, spec in typed.items():
            _require(isinstance(spec, TensorSpec), f"graph {self.name!r}: the spec of {value!r} is not a TensorSpec")
            _require(value in table, f"graph {self.name!r}: value_specs describes {value!r}, which the graph never defines")

    def to_dict(self) -> dict:
        def constant(array: np.ndarray) -> dict:
            return {"dtype": array.dtype.name, "shape": list(array.shape), "data": array.tolist()}

        def specs(table: Mapping[str, TensorSpec]) -> dict:
            return {name: spec.to_dict() for name, spec in table.items()}

        return {
            "schema_version": SCHEMA_VERSION,
            "name": self.name,
            "inputs": specs(self.inputs),
            "outputs": list(self.outputs),
            "nodes": [node.to_dict() for node in self.nodes],
            "constants": {name: constant(array) for name, array in self.constants.items()},
            "value_specs": specs(self.value_specs),
            "metadata": _jsonable(self.metadata),
        }

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Graph":
        version = data.get("schema_version", SCHEMA_VERSION) if isinstance(data, Mapping) else None
        _require(version == SCHEMA_VERSION, f"graph schema version {version!r} is not {SCHEMA_VERSION}")
        try:
            constants = {name: np.asarray(entry["data"], dtype=entry["dtype"]).reshape(entry["shape"])
                         for name, entry in data.get("constants", {}).items()}
            graph = cls(
                name=data["name"],
                inputs={name: TensorSpec.from_dict(spec) for name, spec in data["inputs"].items()},
                outputs=tuple(data["outputs"]),
                nodes=[Node.from_dict(node) for node in data["nodes"]],
                constants=constants,
                value_specs={name: TensorSpec.from_dict(spec) for name, spec in data.get("value_specs", {}).items()},
                metadata=dict(data.get("metadata", {})),
            )
        except (KeyError, TypeError, AttributeError, ValueError) as exc:
            raise ValidationError(f"not a graph: {exc}") from exc
        graph.validate()
        return graph

    @classmethod
    def from_json(cls, text: str) -> "Graph":
        return cls.from_dict(json.loads(text))
