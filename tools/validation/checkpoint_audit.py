"""Hash a checkpoint, or compare two section by section.

    python tools/validation/checkpoint_audit.py hash RUN/checkpoints/iter_0000004
    python tools/validation/checkpoint_audit.py compare A/checkpoints/iter_0000004 B/checkpoints/iter_0000004 [--ignore rng]

Exit code 0 when the two agree in every section that is not ignored.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200.training.checkpoint_audit import checkpoint_hashes, compare  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    h = sub.add_parser("hash")
    h.add_argument("checkpoint")
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    c.add_argument("--ignore", nargs="*", default=[], help="section prefixes to leave out (for example: rng work_state)")
    a = ap.parse_args(argv)
    if a.cmd == "hash":
        print(json.dumps(checkpoint_hashes(a.checkpoint), indent=2))
        return 0
    diff = compare(checkpoint_hashes(a.a), checkpoint_hashes(a.b), a.ignore)
    print(json.dumps({"equal": not diff, "differing_sections": sorted(diff), "detail": diff}, indent=2, default=str))
    return 0 if not diff else 1


if __name__ == "__main__":
    sys.exit(main())
