"""Installs a wheel into a scratch directory and runs the package from THERE, with the source tree off the path.

    python -m tools.release.check_wheel_install dist/aspec_b200-*.whl

Checks that the installed package imports, finds its bundled recipes and Draft descriptions, plans every recipe, and
that the command line answers.  (reference: tools/check_wheel_install.py)
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

_PROBE = r"""
import json, os, sys
import aspec_b200
from aspec_b200 import assets
from aspec_b200.config.train_config import load_config
from aspec_b200.planning import compile_execution_plan
here = os.path.dirname(aspec_b200.__file__)
recipes = sorted(f for f in os.listdir(os.path.join(here, "recipes")) if f.endswith(".yaml"))
planned = 0
for r in recipes:
    cfg = load_config(assets.find_asset(r), ["output_dir=/tmp/aspec-b200-install-check"])
    if cfg.experiments:
        from aspec_b200.multi_draft import compile_multi_draft_plan
        compile_multi_draft_plan(cfg)
    else:
        compile_execution_plan(cfg)
    planned += 1
print(json.dumps({"package_dir": here, "version": aspec_b200.__version__, "recipes": len(recipes), "planned": planned,
                  "sources": len([f for f in os.listdir(os.path.join(here, "csrc")) if f.endswith(".cu")])}))
"""


def check_install(wheel: str) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        site = os.path.join(tmp, "site")
        res = subprocess.run([sys.executable, "-m", "pip", "install", "--no-deps", "--no-index", "--target", site, wheel],
                             capture_output=True, text=True)
        if res.returncode != 0:
            return {"ok": False, "stage": "install", "output": (res.stdout + res.stderr)[-1500:]}
        env = dict(os.environ, PYTHONPATH=site)
        probe = subprocess.run([sys.executable, "-c", _PROBE], capture_output=True, text=True, cwd=tmp, env=env)
        if probe.returncode != 0:
            return {"ok": False, "stage": "probe", "output": (probe.stdout + probe.stderr)[-1500:]}
        info = json.loads(probe.stdout.strip().splitlines()[-1])
        cli = subprocess.run([sys.executable, "-m", "aspec_b200.cli", "recipes", "list"], capture_output=True, text=True, cwd=tmp, env=env)
        ok = (info["package_dir"].startswith(site) and info["planned"] == info["recipes"] > 0 and info["sources"] > 0
              and cli.returncode == 0)
        return {"ok": ok, **info, "package_dir": os.path.relpath(info["package_dir"], tmp), "cli_recipes_list": cli.returncode}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("wheel")
    a = ap.parse_args(argv)
    report = check_install(a.wheel)
    print(json.dumps(report, indent=2))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
