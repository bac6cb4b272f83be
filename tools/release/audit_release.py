"""Audits a built wheel against the source tree it came from.

    python -m tools.release.audit_release dist/aspec_b200-*.whl [--root DIR]

Checks that the wheel holds every Python module of the package, every bundled recipe, Draft / Target description and
sample dataset, the CUDA / C++ sources that ``aspec-b200 build`` compiles, and both console scripts; that it holds
nothing from outside the package (tests, working files, run outputs); and, when a compiled kernel library is inside,
that the source digest stored beside it matches the sources in the same wheel.  Exit code 1 lists the findings.
(reference: tools/audit_release.py, the wheel content audit of its release flow)
"""
from __future__ import annotations

import argparse
import fnmatch
import hashlib
import json
import os
import sys
import zipfile
from typing import List

REQUIRED_PATTERNS = ("aspec_b200/recipes/*.yaml", "aspec_b200/config/drafts/catalog.yaml", "aspec_b200/config/drafts/*.json",
                     "aspec_b200/config/targets/*.json", "aspec_b200/csrc/*.cu", "aspec_b200/csrc/*.cuh",
                     "aspec_b200/csrc/runtime/*.cpp")
FORBIDDEN_PREFIXES = ("tests/", "_work/", "gpurun_out/", "baseline/", "profiles/", "tools/", "examples/")


def tree_files(root: str, patterns) -> List[str]:
    out = []
    for base, _dirs, files in os.walk(os.path.join(root, "aspec_b200")):
        if "__pycache__" in base:
            continue
        for f in files:
            rel = os.path.relpath(os.path.join(base, f), root).replace(os.sep, "/")
            if any(fnmatch.fnmatch(rel, p) for p in patterns):
                out.append(rel)
    return sorted(out)


def audit(wheel: str, root: str) -> dict:
    findings: List[str] = []
    with zipfile.ZipFile(wheel) as z:
        names = set(z.namelist())
        for rel in tree_files(root, ("aspec_b200/*.py", "aspec_b200/**/*.py")):
            if rel not in names:
                findings.append(f"module missing from the wheel: {rel}")
        for rel in tree_files(root, REQUIRED_PATTERNS):
            if rel not in names:
                findings.append(f"bundled file missing from the wheel: {rel}")
        for n in sorted(names):
            if n.startswith(FORBIDDEN_PREFIXES) or "/__pycache__/" in n or n.endswith((".pyc", ".o")):
                findings.append(f"file does not belong in the wheel: {n}")
        entry = [n for n in names if n.endswith(".dist-info/entry_points.txt")]
        scripts = z.read(entry[0]).decode() if entry else ""
        for script in ("aspec-b200", "aspec"):
            if f"{script} = aspec_b200.cli:main" not in scripts:
                findings.append(f"console script {script} is not declared")
        libs = [n for n in names if n.startswith("aspec_b200/lib/") and n.endswith(".so")]
        for lib in libs:
            digest_name = lib[: -len(".so")] + ".sha256"
            if digest_name not in names:
                findings.append(f"{lib} ships without the digest of the sources it was built from")
                continue
            # recompute the digest the in-place build writes, over the sources as the wheel holds them
            import tempfile
            from pathlib import Path
            from aspec_b200 import _native
            runtime = "runtime" in os.path.basename(lib)
            prefix = "aspec_b200/csrc/runtime/" if runtime else "aspec_b200/csrc/"
            kinds = (".cpp", ".h") if runtime else (".cu", ".cuh", ".h")
            with tempfile.TemporaryDirectory() as tmp:
                paths = []
                for src in names:
                    if src.startswith(prefix) and "/" not in src[len(prefix):] and src.endswith(kinds):
                        dest = Path(tmp) / os.path.basename(src)
                        dest.write_bytes(z.read(src))
                        paths.append(dest)
                fresh = _native._digest(paths)
            stored = z.read(digest_name).decode().strip()
            if stored != fresh:
                findings.append(f"{lib} was built from other sources than the wheel holds (digest {stored[:12]} != {fresh[:12]})")
        report = {"wheel": os.path.basename(wheel), "sha256": hashlib.sha256(open(wheel, "rb").read()).hexdigest(),
                  "files": len(names), "modules": sum(n.endswith(".py") for n in names),
                  "recipes": sum(fnmatch.fnmatch(n, "aspec_b200/recipes/*.yaml") for n in names),
                  "kernel_sources": sum(fnmatch.fnmatch(n, "aspec_b200/csrc/*.cu") for n in names),
                  "compiled_libraries": libs, "findings": findings, "ok": not findings}
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("wheel")
    ap.add_argument("--root", default=os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    a = ap.parse_args(argv)
    report = audit(a.wheel, a.root)
    print(json.dumps(report, indent=2))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
