"""Builds the wheel offline, audits it, and writes a release manifest beside it.

    python -m tools.release.build_release --out dist [--with-libraries] [--check-install]

The wheel is pure Python plus the CUDA / C++ sources; ``aspec-b200 build`` compiles them in place after installation.
``--with-libraries`` first compiles the kernel and runtime libraries so that the wheel also carries them (with the
digest of their sources).  ``--check-install`` installs the wheel into a scratch directory and runs the package from
there.  (reference: tools/build_release.py + tools/audit_release.py + tools/check_wheel_install.py)
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import subprocess
import sys
import tempfile

from tools.release.audit_release import audit
from tools.release.check_docs import main as check_docs
from tools.release.check_wheel_install import check_install


def build_wheel(root: str, out: str) -> subprocess.CompletedProcess:
    """Build from a scratch copy of what the wheel is made of, so that the build leaves nothing in the checkout."""
    with tempfile.TemporaryDirectory() as tmp:
        stage = os.path.join(tmp, "src")
        os.makedirs(stage)
        for name in ("pyproject.toml", "README.md"):
            shutil.copy(os.path.join(root, name), stage)
        shutil.copytree(os.path.join(root, "aspec_b200"), os.path.join(stage, "aspec_b200"),
                        ignore=shutil.ignore_patterns("__pycache__", "obj", "*.o"))
        return subprocess.run([sys.executable, "-m", "pip", "wheel", stage, "--no-build-isolation", "--no-deps", "--no-index", "-w", out],
                              capture_output=True, text=True)


def main(argv=None) -> int:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default=os.path.join(root, "dist"))
    ap.add_argument("--with-libraries", action="store_true")
    ap.add_argument("--check-install", action="store_true")
    a = ap.parse_args(argv)
    if check_docs(["--root", root]) != 0:
        print("documentation names files that do not exist: fix it before releasing")
        return 1
    if a.with_libraries:
        from aspec_b200 import _native
        _native.build_all()
    os.makedirs(a.out, exist_ok=True)
    for old in glob.glob(os.path.join(a.out, "aspec_b200-*.whl")):
        os.remove(old)
    res = build_wheel(root, a.out)
    if res.returncode != 0:
        print(res.stdout[-2000:], res.stderr[-2000:])
        return res.returncode
    wheels = glob.glob(os.path.join(a.out, "aspec_b200-*.whl"))
    if len(wheels) != 1:
        print(f"expected one wheel in {a.out}, found {wheels}")
        return 1
    report = audit(wheels[0], root)
    if a.check_install and report["ok"]:
        report["install_check"] = check_install(wheels[0])
        report["ok"] = report["install_check"]["ok"]
    with open(os.path.join(a.out, "release_manifest.json"), "w") as f:
        json.dump(report, f, indent=2)
    print(json.dumps(report, indent=2))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
