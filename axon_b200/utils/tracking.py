"""Experiment tracking fan-out: ``Tracking(project, experiment, backends, config).log(data, step)``
(reference: axon/utils/tracking.py:30-332). Backends: console, file (JSON lines), tensorboard, wandb,
mlflow, clearml — the hosted ones are imported lazily and only when asked for."""
from __future__ import annotations

import json
import numbers
import os
from typing import Any

SUPPORTED = ("console", "file", "tensorboard", "wandb", "mlflow", "clearml")


def _flatten(raw: dict, sep: str = "/", prefix: str = "") -> dict:
    out = {}
    for k, v in raw.items():
        key = f"{prefix}{sep}{k}" if prefix else str(k)
        if isinstance(v, dict):
            out.update(_flatten(v, sep, key))
        else:
            out[key] = v
    return out


def _jsonable(x):
    if isinstance(x, dict):
        return {str(k): _jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    if isinstance(x, (str, bool, int, float)) or x is None:
        return x
    if hasattr(x, "item"):
        try:
            return x.item()
        except Exception:
            pass
    return str(x)


class _Console:
    def log(self, data, step):
        parts = [f"{k}:{v:.4g}" if isinstance(v, numbers.Real) and not isinstance(v, bool) else f"{k}:{v}"
                 for k, v in sorted(data.items())]
        print(f"step:{step} - " + " - ".join(parts), flush=True)

    def finish(self):
        pass


class FileLogger:
    def __init__(self, project_name: str, experiment_name: str, root: str | None = None):
        root = root or os.environ.get("AXON_FILE_LOGGER_ROOT", ".")
        self.path = os.path.join(root, f"{project_name}-{experiment_name}.jsonl")
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        self._f = open(self.path, "a")

    def log(self, data, step):
        self._f.write(json.dumps({"step": step, "data": _jsonable(data)}) + "\n")
        self._f.flush()

    def finish(self):
        self._f.close()


class _Tensorboard:
    def __init__(self, project_name, experiment_name):
        from torch.utils.tensorboard import SummaryWriter
        d = os.environ.get("TENSORBOARD_DIR", os.path.join("tensorboard_log", project_name, experiment_name))
        os.makedirs(d, exist_ok=True)
        self.w = SummaryWriter(d)

    def log(self, data, step):
        for k, v in data.items():
            if isinstance(v, numbers.Real):
                self.w.add_scalar(k, v, step)

    def finish(self):
        self.w.close()


class _Wandb:
    def __init__(self, project_name, experiment_name, config):
        import wandb
        mode = os.environ.get("WANDB_MODE", "offline")
        self.run = wandb.init(project=project_name, name=experiment_name, config=_jsonable(config) if config else None, mode=mode)
        self._wandb = wandb

    def log(self, data, step):
        self._wandb.log(data=data, step=step)

    def finish(self):
        self._wandb.finish(exit_code=0)


class _Mlflow:
    def __init__(self, project_name, experiment_name, config):
        import mlflow
        self.mlflow = mlflow
        mlflow.set_experiment(project_name)
        mlflow.start_run(run_name=experiment_name)
        if config:
            mlflow.log_params({k: str(v)[:250] for k, v in _flatten(_jsonable(config)).items()})

    def log(self, data, step):
        clean = {k.replace("@", "_at_").replace("[", "_").replace("]", "_").replace(",", "_"): float(v)
                 for k, v in data.items() if isinstance(v, numbers.Real)}
        self.mlflow.log_metrics(metrics=clean, step=step)

    def finish(self):
        self.mlflow.end_run()


class ClearMLLogger:
    def __init__(self, project_name: str, experiment_name: str, config):
        import clearml
        self._task = clearml.Task.init(task_name=experiment_name, project_name=project_name, continue_last_task=True,
                                       output_uri=False)
        if config:
            self._task.connect_configuration(_jsonable(config), name="Hyperparameters")

    def log(self, data, step):
        lg = self._task.get_logger()
        for k, v in data.items():
            if isinstance(v, numbers.Real):
                title, _, series = k.partition("/")
                lg.report_scalar(title=title, series=series or title, value=float(v), iteration=step)

    def finish(self):
        self._task.close()


class Tracking:
    supported_backend = list(SUPPORTED)

    def __init__(self, project_name, experiment_name, default_backend: str | list[str] = "console", config=None):
        backends = [default_backend] if isinstance(default_backend, str) else list(default_backend or ["console"])
        for b in backends:
            if b not in SUPPORTED:
                raise ValueError(f"unknown logger backend '{b}' (supported: {SUPPORTED})")
        self.logger: dict[str, Any] = {}
        cfg = config.to_dict() if hasattr(config, "to_dict") else config
        for b in backends:
            if b == "console":
                self.logger[b] = _Console()
            elif b == "file":
                self.logger[b] = FileLogger(project_name, experiment_name)
            elif b == "tensorboard":
                self.logger[b] = _Tensorboard(project_name, experiment_name)
            elif b == "wandb":
                self.logger[b] = _Wandb(project_name, experiment_name, cfg)
            elif b == "mlflow":
                self.logger[b] = _Mlflow(project_name, experiment_name, cfg)
            elif b == "clearml":
                self.logger[b] = ClearMLLogger(project_name, experiment_name, cfg)
        self._finished = False

    def log(self, data: dict, step: int, backend=None, title=None) -> None:
        data = {k: _jsonable(v) for k, v in data.items()}
        for name, lg in self.logger.items():
            if backend is None or name in backend:
                lg.log(data=data, step=step)

    def finish(self) -> None:
        if self._finished:
            return
        self._finished = True
        for lg in self.logger.values():
            try:
                lg.finish()
            except Exception:
                pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.finish()

    def __del__(self):
        try:
            self.finish()
        except Exception:
            pass
