"""The specialization catalog: descriptions of the back ends, readable without any runtime.

Each back end keeps a `specialization.json` in its package directory.  `describe(name)` returns one,
`list_specializations()` all of them in name order.  Nothing here imports numpy, torch or the CUDA library, so a
tool can list what exists on a machine that has none of them.  The two functions, their return values and the
ValueError texts are those of the reference's specializations/catalog.py:13-26, which callers match on.
"""
import json
import re
from pathlib import Path

PACKAGES = Path(__file__).resolve().parent          # one sub-directory per specialization
ROOT = PACKAGES.parent
SCHEMA_VERSION = 1
_IDENTIFIER = re.compile(r"[a-z0-9_]+\Z")


def _description_file(name):
    return PACKAGES / name / "specialization.json"


def describe(name):
    """The description of specialization `name`; ValueError for a name that is not lower-case letters, digits
    and underscores, for a name without a description file, and for a file that names another id or schema."""
    if not (isinstance(name, str) and _IDENTIFIER.match(name)):
        raise ValueError("invalid specialization identifier")
    source = _description_file(name)
    if not source.is_file():
        raise ValueError("unknown specialization: %s" % name)
    with open(source, encoding="utf-8") as handle:
        description = json.load(handle)
    if (description.get("id"), description.get("schema_version")) != (name, SCHEMA_VERSION):
        raise ValueError("invalid specialization description: %s" % name)
    return description


def list_specializations():
    names = sorted(entry.name for entry in PACKAGES.iterdir() if _description_file(entry.name).is_file())
    return [describe(name) for name in names]
