"""``Region["read"|"write"|"reduce"]`` privilege annotations (python/tessera/distributed/region.py).
They are inert markers on kernel signatures; dtype and mutability come from the arrays."""
from __future__ import annotations

_MODES = ("read", "write", "reduce", "read_write")


class _RegionType:
    def __init__(self, mode: str) -> None:
        self.mode = mode

    def __repr__(self) -> str:
        return f'Region["{self.mode}"]'


class _RegionMeta(type):
    def __getitem__(cls, mode: str) -> _RegionType:
        if mode not in _MODES:
            raise ValueError(f"Unknown Region mode {mode!r}; expected one of {_MODES}")
        return _RegionType(mode)


class Region(metaclass=_RegionMeta):
    pass
