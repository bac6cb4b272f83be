"""``aspec-b200`` command dispatcher: ``aspec-b200 COMMAND [OPTIONS]``, ``aspec-b200 --config PATH [KEY=VALUE ...]``,
``aspec-b200 --report RUN_DIRECTORY`` (reference: aspec/cli.py:22-55).  Every command is a module with ``main(argv)``."""
from __future__ import annotations

import importlib
import sys

COMMANDS = {
    "quickstart": "aspec_b200.commands.quickstart",
    "recipes": "aspec_b200.commands.recipes",
    "doctor": "aspec_b200.commands.doctor",
    "export": "aspec_b200.commands.convert_to_hf",
    "stitch-mtp": "aspec_b200.commands.stitch_native_mtp",
    "evaluate": "aspec_b200.commands.evaluate_draft",
    "prepare-data": "aspec_b200.commands.prepare_quality_dataset",
    "prepare-target-data": "aspec_b200.commands.prepare_target_dataset",
    "select-answers": "aspec_b200.commands.prepare_selected_answers",
    "convert-data": "aspec_b200.commands.convert_pretokenized_jsonl",
    "build-workload": "aspec_b200.commands.build_workload",
    "build": "aspec_b200.build",
    "topology": "aspec_b200.topology",
}

USAGE = ("usage: aspec-b200 COMMAND [OPTIONS]\n       aspec-b200 --config PATH [KEY=VALUE ...]\n"
         "       aspec-b200 --report RUN_DIRECTORY [--report-format json]\n\nCommands:\n  " + "\n  ".join(COMMANDS) +
         "\n\nUse aspec-b200 COMMAND --help for command options; python -m aspec_b200.train_entry --help for training options.")


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args or args in (["--help"], ["-h"]):
        print(USAGE)
        return 0
    module = COMMANDS[args.pop(0)] if args[0] in COMMANDS else "aspec_b200.train_entry"
    try:
        rc = importlib.import_module(module).main(args)
    except (ValueError, OSError) as error:
        raise SystemExit(str(error)) from error
    return int(rc or 0)


if __name__ == "__main__":
    sys.exit(main())
