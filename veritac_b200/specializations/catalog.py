"""Find specialization descriptions without importing any runtime (no numpy, torch or CUDA).

Drop-in for the reference's specializations/catalog.py (:13-26): `describe(name)` and
`list_specializations()` read `<name>/specialization.json` next to this file and raise ValueError
for a malformed identifier, an unknown name or a description whose id / schema_version is wrong.
"""
import json
from pathlib import Path

PACKAGES = Path(__file__).resolve().parent
ROOT = PACKAGES.parent
_ALLOWED = frozenset("abcdefghijklmnopqrstuvwxyz0123456789_")


def describe(name):
    if not isinstance(name, str) or not name or not set(name) <= _ALLOWED:
        raise ValueError("invalid specialization identifier")
    path = PACKAGES / name / "specialization.json"
    if not path.is_file():
        raise ValueError(f"unknown specialization: {name}")
    info = json.loads(path.read_text())
    if info.get("id") != name or info.get("schema_version") != 1:
        raise ValueError(f"invalid specialization description: {name}")
    return info


def list_specializations():
    return [describe(p.parent.name) for p in sorted(PACKAGES.glob("*/specialization.json"))]
