"""`python -m veritac_b200.specializations list|show <id>`: print descriptions; launches nothing."""
import argparse
import json

from .catalog import describe, list_specializations


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    sub = parser.add_subparsers(dest="command", required=True)
    sub.add_parser("list", help="List specializations without loading hardware dependencies")
    show = sub.add_parser("show", help="Show one specialization description")
    show.add_argument("specialization")
    args = parser.parse_args()
    try:
        result = list_specializations() if args.command == "list" else describe(args.specialization)
    except ValueError as error:
        parser.error(str(error))
    print(json.dumps(result, indent=2))


if __name__ == "__main__":
    main()
