"""Run logging and experiment trackers: a console / file logger, a JSONL metrics sink and optional TensorBoard /
Weights & Biases back ends selected by ``logging.report_to`` (reference: aspec/utils/logging.py, aspec/utils/wandb.py).
Trackers that are not installed are reported once and skipped; tracking never stops a run.  ``tracking.json`` in the
run directory records what was active."""
from __future__ import annotations

import json
import logging
import os
import sys
import time
from typing import Any, Dict, List, Optional

_LOGGER_NAME = "aspec_b200"


def setup_logger(level: str = "INFO", log_file: Optional[str] = None, rank: int = 0) -> logging.Logger:
    logger = logging.getLogger(_LOGGER_NAME)
    logger.setLevel(getattr(logging, level.upper(), logging.INFO))
    logger.handlers.clear()
    fmt = logging.Formatter(f"%(asctime)s [rank {rank}] %(levelname)s %(message)s", "%H:%M:%S")
    handler = logging.StreamHandler(sys.stdout)
    handler.setFormatter(fmt)
    logger.addHandler(handler)
    if log_file:
        os.makedirs(os.path.dirname(os.path.abspath(log_file)), exist_ok=True)
        fh = logging.FileHandler(log_file)
        fh.setFormatter(fmt)
        logger.addHandler(fh)
    logger.propagate = False
    return logger


def get_logger() -> logging.Logger:
    return logging.getLogger(_LOGGER_NAME)


class JsonlTracker:
    name = "jsonl"

    def __init__(self, run_dir: str):
        os.makedirs(os.path.join(run_dir, "runs"), exist_ok=True)
        self.path = os.path.join(run_dir, "runs", "metrics.jsonl")

    def log(self, metrics: Dict[str, Any], step: int) -> None:
        with open(self.path, "a") as f:
            f.write(json.dumps({"step": step, "time": time.time(), **metrics}, default=float) + "\n")

    def close(self) -> None:
        pass


class TensorBoardTracker:
    name = "tensorboard"

    def __init__(self, run_dir: str):
        from torch.utils.tensorboard import SummaryWriter            # needs the `tensorboard` package
        self.writer = SummaryWriter(os.path.join(run_dir, "runs", "tensorboard"))

    def log(self, metrics: Dict[str, Any], step: int) -> None:
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.writer.add_scalar(k, v, step)

    def close(self) -> None:
        self.writer.close()


class WandbTracker:
    name = "wandb"

    def __init__(self, run_dir: str, project: str, run_name: Optional[str], config: Optional[dict], mode: str = "offline",
                 group: Optional[str] = None, team: Optional[str] = None, directory: Optional[str] = None):
        import wandb                                                 # optional dependency
        self.run = wandb.init(project=project, name=run_name, dir=directory or run_dir, config=config or {}, mode=mode,
                              group=group, entity=team, reinit=True)

    def log(self, metrics: Dict[str, Any], step: int) -> None:
        self.run.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

    def close(self) -> None:
        self.run.finish()


class Trackers:
    """Fan-out over the configured back ends.  ``report_to``: ``none`` | ``tensorboard`` | ``wandb`` | ``all`` or a
    comma-separated list; the JSONL sink is always on."""

    def __init__(self, run_dir: str, report_to: str = "none", *, project: str = "aspec-b200", run_name: Optional[str] = None,
                 config: Optional[dict] = None, wandb_mode: str = "offline", wandb_group: Optional[str] = None,
                 wandb_team: Optional[str] = None, wandb_dir: Optional[str] = None):
        self.run_dir = run_dir
        self.active: List[Any] = [JsonlTracker(run_dir)]
        self.unavailable: Dict[str, str] = {}
        wanted = {"tensorboard", "wandb"} if report_to == "all" else {w.strip() for w in (report_to or "none").split(",")} - {"none", ""}
        for name in sorted(wanted):
            try:
                if name == "tensorboard":
                    self.active.append(TensorBoardTracker(run_dir))
                elif name == "wandb":
                    self.active.append(WandbTracker(run_dir, project, run_name, config, wandb_mode, wandb_group, wandb_team, wandb_dir))
                else:
                    self.unavailable[name] = "unknown tracker"
            except Exception as exc:                                 # noqa: BLE001 - a tracker never stops a run
                self.unavailable[name] = f"{type(exc).__name__}: {exc}"
                get_logger().warning("tracker %s unavailable: %s", name, exc)
        with open(os.path.join(run_dir, "tracking.json"), "w") as f:
            json.dump({"active": [t.name for t in self.active], "unavailable": self.unavailable, "report_to": report_to}, f, indent=2)

    def log(self, metrics: Dict[str, Any], step: int) -> None:
        for t in self.active:
            try:
                t.log(metrics, step)
            except Exception as exc:                                 # noqa: BLE001
                get_logger().warning("tracker %s failed to log: %s", t.name, exc)

    def close(self) -> None:
        for t in self.active:
            try:
                t.close()
            except Exception:                                        # noqa: BLE001
                pass
