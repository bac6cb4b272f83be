"""Checks the documentation against the tree: every repository path a document names in backticks exists, every
relative Markdown link resolves, and every ``python -m <module>`` it shows can be found.

    python -m tools.release.check_docs [--root DIR] [FILE.md ...]

Without file arguments it checks the user-facing documents (README, MIGRATION, tools/README, examples/**/README).
Exit code 1 lists what is stale.  (reference: tools/check_docs.py, the doc-link checker of its CI)
"""
from __future__ import annotations

import argparse
import glob
import importlib.util
import os
import re
import sys
from typing import List

DEFAULT_DOCS = ("README.md", "MIGRATION.md", "tools/README.md", "examples/README.md", "examples/*/README.md")
_PATHISH = re.compile(r"^[A-Za-z0-9_.\-/]+\.(py|cu|cuh|cpp|h|yaml|yml|json|md|toml|sh|jsonl|txt)$")
_LINK = re.compile(r"\[[^\]]*\]\(([^)#\s]+)(#[^)]*)?\)")
_MODULE = re.compile(r"python3? -m ([A-Za-z_][A-Za-z0-9_.]*)")
_PACKAGE_DIRS = ("", "aspec_b200", "aspec_b200/csrc", "aspec_b200/recipes", "aspec_b200/config", "aspec_b200/config/drafts",
                 "aspec_b200/config/targets", "tests", "tools")


def _exists(root: str, doc_dir: str, path: str) -> bool:
    for base in (doc_dir, *[os.path.join(root, d) for d in _PACKAGE_DIRS]):
        if os.path.exists(os.path.join(base, path)):
            return True
    return False


def check_file(root: str, doc: str) -> List[str]:
    problems = []
    text = open(doc, encoding="utf-8").read()
    doc_dir = os.path.dirname(os.path.abspath(doc))
    rel = os.path.relpath(doc, root)
    migration = os.path.basename(doc) == "MIGRATION.md"
    for lineno, line in enumerate(text.splitlines(), 1):
        if migration and line.startswith("|"):
            line = "|" + line.split("|", 2)[-1]            # the first column of a migration table names the OTHER project's files
        for span in re.findall(r"`([^`\n]+)`", line):
            token = span.split("::")[0].strip()
            # only tokens that look like a file of this tree: a slash or a known top-level name, no placeholders
            if not _PATHISH.match(token) or any(c in token for c in "<>*{}$") or token.startswith(("/", "~", ".")):
                continue
            if "/" not in token and not os.path.exists(os.path.join(root, token)) and not _exists(root, doc_dir, token):
                # a bare file name that is nowhere in the tree is an output file of a run, not a reference
                if not any(glob.glob(os.path.join(root, "**", token), recursive=True)):
                    continue
            if not _exists(root, doc_dir, token) and not glob.glob(os.path.join(root, "**", token), recursive=True):
                problems.append(f"{rel}:{lineno}: `{token}` does not exist")
        for target, _anchor in _LINK.findall(line):
            if re.match(r"^[a-z]+:", target):
                continue                                     # http:, mailto:
            if not os.path.exists(os.path.join(doc_dir, target)):
                problems.append(f"{rel}:{lineno}: link target {target} does not exist")
        for module in _MODULE.findall(line):
            top = module.split(".")[0]
            if top not in ("aspec_b200", "tools"):
                continue
            path = os.path.join(root, *module.split("."))
            if not (os.path.isfile(path + ".py") or os.path.isfile(os.path.join(path, "__main__.py")) or os.path.isfile(os.path.join(path, "__init__.py"))):
                problems.append(f"{rel}:{lineno}: module {module} does not exist")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--root", default=os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    ap.add_argument("files", nargs="*")
    a = ap.parse_args(argv)
    docs = a.files or sorted(p for pat in DEFAULT_DOCS for p in glob.glob(os.path.join(a.root, pat)))
    problems = [p for d in docs for p in check_file(a.root, d)]
    for p in problems:
        print(p)
    print(f"{len(docs)} documents checked, {len(problems)} stale references")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
