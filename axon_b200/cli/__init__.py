"""``axon`` command line: ``train``, ``status``, ``logs``, ``cancel`` (reference: axon/cli/, docs/reference/cli.md)."""
from __future__ import annotations

import os
import signal
import sys
import time

import click
import yaml

from ..config.validate_config import validate_axon_config
from ..utils.config import compose_config, flatten_yaml_to_overrides
from . import _runs

_FLAG_MAP = {"model": "model_path", "train_data": "train_files", "val_data": "val_files", "gpus": "num_gpus_per_node",
             "nodes": "num_nodes", "experiment_name": "experiment_name", "output_dir": "output_dir"}


def build_overrides(config_path, flags: dict, raw: tuple) -> list[str]:
    """Precedence: base tree < YAML file (as ++k=v) < flags < raw overrides after ``--``."""
    ov: list[str] = []
    if config_path:
        with open(config_path) as f:
            ov += flatten_yaml_to_overrides(yaml.safe_load(f) or {})
    for flag, key in _FLAG_MAP.items():
        if flags.get(flag) is not None:
            ov.append(f"++{key}={flags[flag]}")
    if flags.get("resume") is not None:
        ov.append(f"++resume_from_checkpoint={flags['resume']}")
    return ov + list(raw)


@click.group()
def main():
    """RL post-training for LLM agents on B200."""


@main.command(context_settings={"ignore_unknown_options": True, "allow_extra_args": True})
@click.option("--config", "-c", "config_path", type=click.Path(exists=True), default=None)
@click.option("--model", "-m", default=None)
@click.option("--train-data", default=None)
@click.option("--val-data", default=None)
@click.option("--gpus", type=int, default=None)
@click.option("--nodes", type=int, default=None)
@click.option("--experiment-name", default=None)
@click.option("--output-dir", default=None)
@click.option("--resume/--no-resume", default=None)
@click.option("--dry-run", is_flag=True)
@click.option("--foreground", "--fg", is_flag=True)
@click.argument("overrides", nargs=-1, type=click.UNPROCESSED)
def train(config_path, model, train_data, val_data, gpus, nodes, experiment_name, output_dir, resume, dry_run,
          foreground, overrides):
    """Compose, validate and launch a training run (detached unless --foreground)."""
    flags = dict(model=model, train_data=train_data, val_data=val_data, gpus=gpus, nodes=nodes,
                 experiment_name=experiment_name, output_dir=output_dir, resume=resume)
    ov = build_overrides(config_path, flags, tuple(o for o in overrides if o != "--"))
    try:
        cfg = compose_config(ov)
        validate_axon_config(cfg)
    except Exception as e:  # noqa: BLE001
        raise click.ClickException(f"invalid configuration: {e}")
    if dry_run:
        click.echo(yaml.safe_dump(cfg.to_dict(), sort_keys=False))
        return
    base = config_path or "config"
    if foreground:
        meta = _runs.create_run(base, cfg.experiment_name)
        click.echo(f"run {meta['run_id']} (foreground), log: {meta['log_path']}")
        try:
            with _runs.tee_to_file(meta["log_path"]):
                from ..driver.train_agent_ppo import run_ppo_agent
                run_ppo_agent(cfg)
            _runs.set_status(meta["run_id"], "finished")
        except BaseException:
            _runs.set_status(meta["run_id"], "failed")
            raise
    else:
        meta = _runs.launch_training(ov, base, cfg.experiment_name)
        click.echo(f"started run {meta['run_id']} (pid {meta['pid']}), log: {meta['log_path']}")


@main.command()
@click.argument("run_id", required=False)
def status(run_id):
    """List runs, or show one run in detail."""
    if run_id:
        try:
            meta = _runs.read_meta(_runs.resolve_run_id(run_id))
        except KeyError as e:
            raise click.ClickException(str(e))
        for k, v in meta.items():
            click.echo(f"{k:12s} {v}")
        return
    runs = _runs.list_runs()
    if not runs:
        click.echo("no runs")
        return
    click.echo(f"{'RUN':10s} {'STATUS':10s} {'STARTED':20s} EXPERIMENT")
    for m in runs:
        click.echo(f"{m['run_id']:10s} {m['status']:10s} {m['started']:20s} {m.get('experiment', '')}")


@main.command()
@click.argument("run_id")
@click.option("-n", "lines", type=int, default=50)
@click.option("-f", "follow", is_flag=True)
def logs(run_id, lines, follow):
    """Tail a run's log."""
    try:
        meta = _runs.read_meta(_runs.resolve_run_id(run_id))
    except KeyError as e:
        raise click.ClickException(str(e))
    path = meta["log_path"]
    if not os.path.exists(path):
        raise click.ClickException(f"no log at {path}")
    with open(path, errors="replace") as f:
        for line in f.readlines()[-lines:]:
            click.echo(line.rstrip("\n"))
        while follow:
            line = f.readline()
            if line:
                click.echo(line.rstrip("\n"))
            else:
                if _runs.read_meta(meta["run_id"])["status"] != "running":
                    break
                time.sleep(0.5)


@main.command()
@click.argument("run_id")
def cancel(run_id):
    """Send SIGTERM to a running run (never SIGKILL)."""
    try:
        meta = _runs.read_meta(_runs.resolve_run_id(run_id))
    except KeyError as e:
        raise click.ClickException(str(e))
    if meta["status"] != "running":
        click.echo(f"run {meta['run_id']} is {meta['status']}; nothing to cancel")
        return
    try:
        os.killpg(os.getpgid(int(meta["pid"])), signal.SIGTERM)
    except (ProcessLookupError, PermissionError):
        os.kill(int(meta["pid"]), signal.SIGTERM)
    _runs.set_status(meta["run_id"], "cancelled")
    click.echo(f"cancelled run {meta['run_id']}")


if __name__ == "__main__":
    main()
