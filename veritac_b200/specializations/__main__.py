"""Command line of the specialization catalog: `python -m veritac_b200.specializations list` prints every
description, `... show <id>` prints one.  Reads JSON files only; no device, no numpy, no torch.

Same two commands, same JSON on stdout and the same error texts as the reference's `python -m specializations`.
"""
import json
import sys

from . import catalog

USAGE = "usage: python -m veritac_b200.specializations list | show <specialization>"


def run(argv):
    """Returns (exit status, text).  Status 2 with a usage / error message, as argparse would give."""
    if argv == ["list"]:
        return 0, json.dumps(catalog.list_specializations(), indent=2)
    if len(argv) == 2 and argv[0] == "show":
        try:
            return 0, json.dumps(catalog.describe(argv[1]), indent=2)
        except ValueError as problem:
            return 2, "%s\nerror: %s" % (USAGE, problem)
    return 2, USAGE


if __name__ == "__main__":
    status, text = run(sys.argv[1:])
    print(text, file=sys.stdout if status == 0 else sys.stderr)
    sys.exit(status)
