"""Type aliases shared across the package.

Mirrors the small alias module of the reference (``src/jaxdecomp/typing.py:1-12``)
so that annotations in user code port over unchanged.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

GdimsType = Tuple[int, int, int]
PdimsType = Tuple[int, int]
# a spec written with sizes instead of names, e.g. ('x', None, 'y') -> (Nx, 1, Ny)
TransposablePdimsType = Tuple[int, int, int]
HaloExtentType = Tuple[int, int]
Periodicity = Tuple[bool, bool]
AxisName = Optional[str]
SpecType = Sequence[AxisName]
