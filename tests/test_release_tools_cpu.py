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


@pytest.mark.timeout(600)
def test_every_command_line_shown_in_the_documents_and_examples_parses():
    """Each ``aspec_b200.cli`` invocation in README, MIGRATION and the examples names a sub-command that exists and only
    options that sub-command accepts (its ``--help`` lists them)."""
    import re
    files = [os.path.join(ROOT, "README.md"), os.path.join(ROOT, "MIGRATION.md")]
    files += glob.glob(os.path.join(ROOT, "examples", "*", "run.sh")) + glob.glob(os.path.join(ROOT, "examples", "*", "README.md"))
    helps = {}

    def options_of(*sub):
        if sub not in helps:
            # without a sub-command the command line is the train entry's
            module = ["aspec_b200.cli", *sub] if sub else ["aspec_b200.train_entry"]
            out = subprocess.run([sys.executable, "-m", *module, "--help"], cwd=ROOT, capture_output=True, text=True,
                                 env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
            helps[sub] = (out.returncode, set(re.findall(r"(?<![\w-])--[a-z][a-z0-9-]*", out.stdout)))
        return helps[sub]

    checked, problems, overrides = 0, [], set()
    for path in files:
        text = open(path).read().replace("\\\n", " ")
        for line in text.splitlines():
            m = re.search(r"(?:aspec_b200\.cli|\$CLI|aspec-b200)\s+(.*)", line)
            if not m or line.lstrip().startswith("#") and "cli" not in line:
                continue
            words = m.group(1).split("#")[0].split()
            if not words or words[0].startswith(("`", "(", "|")):
                continue
            sub = [] if words[0].startswith("--") else [words[0]]
            if sub and not re.fullmatch(r"[a-z][a-z0-9-]*", sub[0]):
                continue                                      # prose, not a command
            flags = {w.split("=")[0] for w in words if re.fullmatch(r"--[a-z][a-z0-9-]*(=.*)?", w)}
            if not sub:                                        # a training command line: its KEY=VALUE overrides must be configuration keys
                for w in words:
                    key = re.fullmatch(r"'?([a-z_]+(?:\.[a-z_0-9]+)+)=.*", w)
                    if key:
                        overrides.add((os.path.relpath(path, ROOT), key.group(1)))
            rc, allowed = options_of(*sub)
            if rc != 0:
                problems.append(f"{os.path.relpath(path, ROOT)}: unknown sub-command in `{line.strip()[:100]}`")
                continue
            if sub and len(words) > 1 and re.fullmatch(r"[a-z][a-z0-9-]*", words[1]):
                rc2, nested = options_of(sub[0], words[1])     # nested sub-commands (recipes plan, quickstart tiny)
                if rc2 == 0:
                    allowed = allowed | nested
            checked += 1
            for f in sorted(flags - allowed):
                problems.append(f"{os.path.relpath(path, ROOT)}: `{' '.join(sub) or 'train'}` has no option {f}: `{line.strip()[:100]}`")
    from aspec_b200 import assets
    from aspec_b200.config.train_config import load_config
    recipe = assets.find_asset("quickstart_tiny.yaml")
    for where, key in sorted(overrides):
        try:
            load_config(recipe, [f"{key}=1"])
        except Exception as exc:                               # noqa: BLE001 - only the key's existence is checked here
            if "Unknown config key" in str(exc):
                problems.append(f"{where}: `{key}` is not a configuration key")
    assert checked >= 20 and len(overrides) >= 15 and not problems, "\n".join(problems)
