"""SO(2) field types and the flat node-field layout the kernels read.

A field type is a multiset of SO(2) irreps: ``a_n`` copies of frequency ``n``.
The flat layout (reference: ``representations/field_type.py:238-255, 472-488``)
concatenates, by ascending frequency, ``a_0`` reals for ``n = 0`` and ``a_n``
interleaved ``(re, im)`` pairs for ``n >= 1``.  A multi-head field is the
direct sum of ``H`` equal head types; inside each frequency block the copies
are head-major (head ``h`` owns copies ``h a_n .. (h + 1) a_n - 1``).
"""

from __future__ import annotations

from collections.abc import Iterable, Mapping
from typing import Any


class FieldType:
    """``{frequency: multiplicity}`` with the reference type's read-only API
    (``items``, ``slices``, ``dimension``, ``multiplicity``, ``max_frequency``)."""

    def __init__(self, multiplicities: Mapping[int, int] | Iterable[tuple[int, int]]) -> None:
        pairs = dict(multiplicities.items() if isinstance(multiplicities, Mapping) else multiplicities)
        for n, a in pairs.items():
            if int(n) != n or n < 0 or int(a) != a or a < 1:
                raise ValueError(f"invalid irrep entry {n}: {a}")
        self._items = tuple(sorted((int(n), int(a)) for n, a in pairs.items()))

    @classmethod
    def uniform(cls, copies: int, max_frequency: int) -> FieldType:
        return cls({n: copies for n in range(max_frequency + 1)})

    def items(self) -> tuple[tuple[int, int], ...]:
        return self._items

    @property
    def frequencies(self) -> tuple[int, ...]:
        return tuple(n for n, _ in self._items)

    @property
    def dimension(self) -> int:
        return sum(a * (1 if n == 0 else 2) for n, a in self._items)

    @property
    def max_frequency(self) -> int:
        return max((n for n, _ in self._items), default=0)

    def multiplicity(self, frequency: int) -> int:
        return dict(self._items).get(frequency, 0)

    def scaled(self, factor: int) -> FieldType:
        return FieldType({n: factor * a for n, a in self._items})

    def slices(self) -> dict[int, slice]:
        out: dict[int, slice] = {}
        start = 0
        for n, a in self._items:
            stop = start + a * (1 if n == 0 else 2)
            out[n] = slice(start, stop)
            start = stop
        return out

    def __contains__(self, frequency: object) -> bool:
        return frequency in dict(self._items)

    def __len__(self) -> int:
        return len(self._items)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, FieldType) and other._items == self._items

    def __hash__(self) -> int:
        return hash(self._items)

    def __repr__(self) -> str:
        return "FieldType({" + ", ".join(f"{n}: {a}" for n, a in self._items) + "})"


class FeatureField:
    """Coefficients of a field by frequency: ``(..., a_0)`` reals for frequency 0 and ``(..., a_n, 2)`` real pairs
    ``(re, im)`` for ``n >= 1`` -- the container the driver entries take and return, constructed like the
    reference's ``SO2FeatureField(field_type, coefficients)`` (``representations/field_type.py:370-488``)."""

    def __init__(self, field_type: FieldType, coefficients: Mapping[int, Any]) -> None:
        if set(coefficients) != set(field_type.frequencies):
            raise ValueError(f"coefficients for frequencies {sorted(coefficients)} do not match {field_type!r}")
        for n, a in field_type.items():
            shape = tuple(coefficients[n].shape)
            tail = (a,) if n == 0 else (a, 2)
            if shape[-len(tail):] != tail:
                raise ValueError(f"frequency {n}: trailing shape {shape[-len(tail):]} is not {tail}")
        self.field_type, self.coefficients = field_type, dict(coefficients)

    def __getitem__(self, frequency: int) -> Any:
        return self.coefficients[frequency]

    @classmethod
    def from_flat(cls, field_type: FieldType, flat: Any) -> FeatureField:
        parts = {}
        for n, sl in field_type.slices().items():
            block = flat[..., sl]
            parts[n] = block if n == 0 else block.reshape(*block.shape[:-1], field_type.multiplicity(n), 2)
        return cls(field_type, parts)

    def to_flat(self) -> Any:
        import torch

        return torch.cat([self.coefficients[n] if n == 0 else self.coefficients[n].flatten(-2) for n in self.field_type.frequencies], -1)
