"""``python -m aspec_b200.build [--force] [-v]`` compiles the native libraries in-tree."""
import argparse

from aspec_b200 import _native


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args()
    _native.build_all(force=args.force, verbose=args.verbose)
    print(_native._KERNEL_LIB)


if __name__ == "__main__":
    main()
