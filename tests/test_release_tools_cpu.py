"""Release tooling on CPU: the documents name only files that exist, an audit of a wheel built from this tree is clean
and notices what is missing or foreign, and the installed wheel runs with the checkout off the path
(reference: tools/check_docs.py, tools/audit_release.py, tools/check_wheel_install.py)."""
import glob
import os
import subprocess
import sys
import zipfile

import pytest

from tools.release import audit_release, check_docs, check_wheel_install

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_documents_name_only_files_that_exist(tmp_path, capsys):
    assert check_docs.main(["--root", ROOT]) == 0
    stale = tmp_path / "NOTES.md"
    stale.write_text("See `aspec_b200/ops/no_such_file.py`, [the guide](missing.md) and `python -m aspec_b200.no_such_module`.\n"
                     "`aspec_b200/cli.py` and `python -m aspec_b200.cli` are fine; `evidence.json` is an output, not a source.\n")
    assert check_docs.main(["--root", ROOT, str(stale)]) == 1
    out = capsys.readouterr().out
    assert "no_such_file.py" in out and "missing.md" in out and "no_such_module" in out and "3 stale" in out


@pytest.mark.timeout(900)
def test_a_wheel_of_this_tree_passes_the_audit_and_runs_when_installed(tmp_path):
    from tools.release.build_release import build_wheel
    res = build_wheel(ROOT, str(tmp_path))                  # from a scratch copy: nothing is written into the checkout
    assert res.returncode == 0, res.stderr[-2000:]
    assert not os.path.isdir(os.path.join(ROOT, "build")) and not glob.glob(os.path.join(ROOT, "*.egg-info"))
    wheel, = glob.glob(str(tmp_path / "aspec_b200-*.whl"))
    report = audit_release.audit(wheel, ROOT)
    assert report["ok"], report["findings"]
    assert report["recipes"] >= 22 and report["kernel_sources"] >= 8 and report["modules"] > 100
    # a wheel that lost a recipe and gained a test file is caught
    broken = str(tmp_path / "broken.whl")
    with zipfile.ZipFile(wheel) as src, zipfile.ZipFile(broken, "w") as dst:
        for item in src.infolist():
            if item.filename != "aspec_b200/recipes/quickstart_tiny.yaml":
                dst.writestr(item, src.read(item.filename))
        dst.writestr("tests/test_x.py", "")
    bad = audit_release.audit(broken, ROOT)
    assert not bad["ok"] and any("quickstart_tiny.yaml" in f for f in bad["findings"]) and any("tests/test_x.py" in f for f in bad["findings"])
    installed = check_wheel_install.check_install(wheel)
    assert installed["ok"], installed
    assert installed["planned"] == installed["recipes"] == report["recipes"] and installed["package_dir"].startswith("site")
