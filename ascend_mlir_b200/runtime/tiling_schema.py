"""TilingSchema: pack named tiling parameters into the little-endian TilingData bytes a kernel takes.

Same contract as the reference's python/runtime/tiling_schema.py: only 'name' and 'type' of each
tiling_params[] entry matter, field order is the schema order, every field must be given exactly once.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Iterable, Union

_INT32 = ("int32", "int32_t")


class TilingSchema:
    def __init__(self, fields: Iterable[dict]) -> None:
        self._fields = [{"name": f["name"], "type": f.get("type", "int64")} for f in fields]

    @classmethod
    def from_names(cls, names: Iterable[str]) -> "TilingSchema":
        return cls({"name": n, "type": "int64"} for n in names)

    @classmethod
    def from_json(cls, path: Union[str, Path]) -> "TilingSchema":
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(f"tiling_space.json not found: {path}")
        try:
            data = json.loads(path.read_text())
        except json.JSONDecodeError as e:
            raise ValueError(f"JSON parse error in '{path}': {e}") from e
        return cls.from_dict(data, str(path))

    @classmethod
    def from_dict(cls, data: dict, origin: str = "<dict>") -> "TilingSchema":
        params = data.get("tiling_params")
        if params is None:
            raise ValueError(f"'{origin}': missing 'tiling_params' array")
        if not isinstance(params, list):
            raise ValueError(f"'{origin}': 'tiling_params' must be a list")
        fields = []
        for i, entry in enumerate(params):
            if not isinstance(entry, dict):
                raise ValueError(f"'{origin}': tiling_params[{i}] must be an object")
            if not entry.get("name"):
                raise ValueError(f"'{origin}': tiling_params[{i}] missing 'name'")
            fields.append({"name": entry["name"], "type": entry.get("type", "int64")})
        return cls(fields)

    def pack(self, **kwargs: int) -> bytes:
        expected = [f["name"] for f in self._fields]
        missing = sorted(set(expected) - set(kwargs))
        extra = sorted(set(kwargs) - set(expected))
        errors = []
        if missing:
            errors.append(f"missing tiling fields: {missing}")
        if extra:
            errors.append(f"unexpected tiling fields: {extra}")
        if errors:
            raise ValueError("\n".join(errors) + f"\n  expected: {expected}")
        out = bytearray()
        for f in self._fields:
            out += struct.pack("<i" if f["type"] in _INT32 else "<q", int(kwargs[f["name"]]))
        return bytes(out)

    @property
    def field_names(self) -> list[str]:
        return [f["name"] for f in self._fields]

    @property
    def fields(self) -> list[dict]:
        return [dict(f) for f in self._fields]

    def __len__(self) -> int:
        return len(self._fields)

    def __repr__(self) -> str:
        return f"TilingSchema({self.field_names})"
