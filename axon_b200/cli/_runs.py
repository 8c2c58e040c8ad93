"""Run registry: every ``axon train`` gets an 8-hex id and a directory ``<RUNS_DIR>/<id>/`` holding
``meta.json`` {run_id, pid, status, started, log_path, base, experiment} and ``train.log``. Ids
resolve by unique prefix; a run whose process is gone while still marked running reads as crashed
(reference: axon/cli/_runs.py, docs/reference/cli.md:105-117)."""
from __future__ import annotations

import json
import os
import secrets
import subprocess
import sys
import time
from contextlib import contextmanager
from pathlib import Path


def runs_dir() -> Path:
    return Path(os.environ.get("AXON_RUNS_DIR", "~/.axon/runs")).expanduser()


def _pid_alive(pid: int) -> bool:
    if pid <= 0:
        return False
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    try:                                   # a zombie child still answers kill(0)
        with open(f"/proc/{pid}/stat") as f:
            return f.read().rsplit(")", 1)[1].split()[0] != "Z"
    except OSError:
        return True


def create_run(base: str, experiment: str, pid: int | None = None) -> dict:
    rd = runs_dir()
    rd.mkdir(parents=True, exist_ok=True)
    while True:
        rid = secrets.token_hex(4)
        if not (rd / rid).exists():
            break
    d = rd / rid
    d.mkdir()
    meta = {"run_id": rid, "pid": pid if pid is not None else os.getpid(), "status": "running",
            "started": time.strftime("%Y-%m-%dT%H:%M:%S"), "log_path": str(d / "train.log"), "base": base,
            "experiment": experiment}
    write_meta(meta)
    return meta


def write_meta(meta: dict) -> None:
    d = runs_dir() / meta["run_id"]
    tmp = d / "meta.json.tmp"
    tmp.write_text(json.dumps(meta, indent=2))
    tmp.replace(d / "meta.json")


def read_meta(run_id: str) -> dict:
    meta = json.loads((runs_dir() / run_id / "meta.json").read_text())
    if meta.get("status") == "running" and not _pid_alive(int(meta.get("pid", -1))):
        meta["status"] = "crashed"
        write_meta(meta)
    return meta


def list_runs() -> list[dict]:
    rd = runs_dir()
    if not rd.exists():
        return []
    out = []
    for d in rd.iterdir():
        if (d / "meta.json").exists():
            try:
                out.append(read_meta(d.name))
            except (json.JSONDecodeError, OSError):
                continue
    return sorted(out, key=lambda m: m.get("started", ""), reverse=True)


def resolve_run_id(prefix: str) -> str:
    rd = runs_dir()
    matches = [d.name for d in rd.iterdir() if d.is_dir() and d.name.startswith(prefix)] if rd.exists() else []
    if not matches:
        raise KeyError(f"no run matches '{prefix}'")
    if len(matches) > 1:
        raise KeyError(f"run id prefix '{prefix}' is ambiguous: {sorted(matches)}")
    return matches[0]


def set_status(run_id: str, status: str) -> None:
    meta = json.loads((runs_dir() / run_id / "meta.json").read_text())
    meta["status"] = status
    write_meta(meta)


@contextmanager
def tee_to_file(path: str):
    """Duplicate stdout / stderr of this process into ``path`` for the duration of the block."""
    Path(path).parent.mkdir(parents=True, exist_ok=True)

    class Tee:
        def __init__(self, stream, fh):
            self.stream, self.fh = stream, fh

        def write(self, s):
            self.stream.write(s)
            self.fh.write(s)
            self.fh.flush()
            return len(s)

        def flush(self):
            self.stream.flush()
            self.fh.flush()

        def __getattr__(self, name):
            return getattr(self.stream, name)

    with open(path, "a", buffering=1) as fh:
        old = sys.stdout, sys.stderr
        sys.stdout, sys.stderr = Tee(old[0], fh), Tee(old[1], fh)
        try:
            yield
        finally:
            sys.stdout, sys.stderr = old


def launch_training(overrides: list[str], base: str, experiment: str) -> dict:
    """Start ``python -m axon_b200.driver.train_agent_ppo`` detached (own session), logging to the run dir."""
    meta = create_run(base, experiment, pid=0)
    log = open(meta["log_path"], "ab")
    cmd = [sys.executable, "-m", "axon_b200.driver.train_agent_ppo", f"--run-id={meta['run_id']}", *overrides]
    proc = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL, start_new_session=True)
    meta["pid"] = proc.pid
    write_meta(meta)
    return meta
