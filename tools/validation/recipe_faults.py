"""Host-side fault injection into a recipe run: the run must end the way the failure model says, and clean up.

    python tools/validation/recipe_faults.py --config RECIPE.yaml --action trainer_raise|trainer_stall|producer_fail
           --out DIR [--step 1] [--rank 0] [section.key=value ...]

* ``trainer_raise``  - trainer ``rank`` raises inside update ``step``: the run fails with that error.
* ``trainer_stall``  - trainer ``rank`` sleeps inside update ``step`` past ``training.optimizer_step_timeout_seconds``:
  the controller's deadline ends the run and terminates the trainers.
* ``producer_fail``  - the Target engine raises after ``--rows`` rows: the run fails with the producer's error.
* ``trainer_exit``   - trainer ``rank``'s process exits at the start of update ``step`` (between updates, nothing of its
  own in flight - what losing a node looks like): the controller notices the missing process and ends the run.

Every fault is made on the host (an exception, a sleep); no GPU is faulted or hung.  After the failure the probe checks
that ``evidence.json`` says ``failed`` with the error recorded, that the cleanup section lists every actor as stopped,
that no staging checkpoint directory is left behind and that no child process of the run survives.  Prints one JSON verdict;
exit code 0 when the run failed in the expected way and left nothing behind.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from aspec_b200 import train_entry  # noqa: E402

EXPECT = {"trainer_raise": "injected failure", "trainer_stall": "Timeout", "producer_fail": "injected producer failure",
          "trainer_exit": "exited"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--action", choices=sorted(EXPECT), required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--step", type=int, default=1)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--rows", type=int, default=3)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    inject = {"trainer_raise": [f"debug.fault_injection={{kind: raise, step: {a.step}, rank: {a.rank}}}"],
              "trainer_stall": [f"debug.fault_injection={{kind: sleep, step: {a.step}, rank: {a.rank}, seconds: 120}}",
                                "training.optimizer_step_timeout_seconds=3"],
              "producer_fail": [f"debug.producer_fail_after={a.rows}"],
              "trainer_exit": [f"debug.fault_injection={{kind: exit, step: {a.step}, rank: {a.rank}}}"]}[a.action]
    import psutil
    me = psutil.Process()
    before = {p.pid for p in me.children(recursive=True)}
    error = None
    t0 = time.perf_counter()
    try:
        train_entry.main(["--config", a.config, *a.overrides, *inject, f"output_dir={a.out}"])
    except BaseException as exc:  # noqa: BLE001 - the failure is the expected outcome
        error = f"{type(exc).__name__}: {exc}"
    seconds = time.perf_counter() - t0
    time.sleep(1.0)
    survivors = [p.pid for p in me.children(recursive=True) if p.pid not in before and p.is_running()
                 and p.status() != psutil.STATUS_ZOMBIE
                 and "multiprocessing.resource_tracker" not in " ".join(p.cmdline())]      # this process's own helper
    ev_path = os.path.join(a.out, "evidence.json")
    ev = json.load(open(ev_path)) if os.path.isfile(ev_path) else {}
    ckpt_dir = os.path.join(a.out, "checkpoints")
    staging = [d for d in (os.listdir(ckpt_dir) if os.path.isdir(ckpt_dir) else []) if d.endswith(".incomplete")]
    checks = {"run_failed": error is not None,
              "expected_error": bool(error and EXPECT[a.action].lower() in error.lower()),
              "evidence_state_failed": ev.get("state") == "failed",
              "evidence_names_the_error": bool((ev.get("failure") or {}).get("message")),
              "no_surviving_children": not survivors,
              "no_staging_checkpoint": not staging}
    print(json.dumps({"probe": "recipe_faults", "action": a.action, "seconds": round(seconds, 2), "error": error,
                      "checks": checks, "ok": all(checks.values())}))
    return 0 if all(checks.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
