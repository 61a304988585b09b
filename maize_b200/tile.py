"""Descriptor types with the names of the reference's Python surface.

The reference's ``maize.tile`` exports only descriptors (crates/maize_py/src/lib.rs:9-16,
python/maize/_bindings.pyi:1-15): ``DType``, ``Shape``, ``Stride`` and ``Tile``.  They are
kept here, with ``BF16`` added to ``DType`` (the reference lists F32 and F64 only,
crates/maize_py/src/dtype.rs:8-11) because the GEMM path is bf16.
"""
from __future__ import annotations

import enum
from typing import Optional, Union


class DType(enum.Enum):
    F32 = "F32"
    F64 = "F64"
    BF16 = "BF16"

    def to_str(self) -> str:
        return self.value

    @classmethod
    def try_from_str(cls, val: str) -> Optional["DType"]:
        return cls.__members__.get(val)

    @classmethod
    def from_str(cls, val: str) -> "DType":
        got = cls.try_from_str(val)
        if got is None:
            raise ValueError(f"Invalid DType name '{val}'")
        return got

    @property
    def itemsize(self) -> int:
        return {"F32": 4, "F64": 8, "BF16": 2}[self.value]


class _Tuple:
    """Nested tuple of non-negative ints (crates/maize_py/src/tuple.rs)."""

    def __init__(self, *values: Union["_Tuple", int]):
        items = []
        for v in values:
            if isinstance(v, _Tuple):
                items.append(v)
            elif isinstance(v, int) and not isinstance(v, bool) and v >= 0:
                items.append(v)
            else:
                raise TypeError(f"{type(self).__name__} takes non-negative ints or nested {type(self).__name__}s")
        self._items = tuple(items)

    def flatten(self):
        out = []
        for v in self._items:
            out.extend(v.flatten() if isinstance(v, _Tuple) else [v])
        return tuple(out)

    def __len__(self):
        return len(self._items)

    def __iter__(self):
        return iter(self._items)

    def __eq__(self, other):
        return type(other) is type(self) and self._items == other._items

    def __hash__(self):
        return hash((type(self).__name__, self._items))

    def __repr__(self):
        return "(" + ", ".join(repr(v) for v in self._items) + ")"


class Shape(_Tuple):
    def size(self) -> int:
        n = 1
        for v in self.flatten():
            n *= v
        return n


class Stride(_Tuple):
    pass


class Tile:
    """A shape with an element type, as ``maize.tile.Tile`` (crates/maize_py/src/tile.rs:18-29)."""

    def __init__(self, shape: Shape, dtype: DType):
        if not isinstance(shape, Shape) or not isinstance(dtype, DType):
            raise TypeError("Tile(shape: Shape, dtype: DType)")
        self.shape = shape
        self.dtype = dtype

    def nbytes(self) -> int:
        return self.shape.size() * self.dtype.itemsize

    def __eq__(self, other):
        return isinstance(other, Tile) and self.shape == other.shape and self.dtype == other.dtype

    def __repr__(self):
        return f"Tile(shape={self.shape!r}, dtype={self.dtype.to_str()})"
