"""Programs in, training batch out.

``ProgramRunner`` instantiates one program per dataset row from the program registry, runs them on a
background asyncio loop against the ``Engine`` (or, with the HTTP endpoint enabled, in child
processes that talk to the engine's routers) and collects the finished ``ProgramState`` objects.
``ProgramProcessor.transform_programs`` flattens every program's training steps (one per leaf of its
prefix tree) into the right-padded ``[B, max_seq_length]`` batch that the trainers consume
(reference: axon/driver/components/program_component.py:121-311, 658-913, 916-963, 1075-1300).

Row assembly is done with numpy index arithmetic over one concatenated token stream instead of
per-row padding calls; a step of a few thousand rows is assembled in a few milliseconds.
"""
from __future__ import annotations

import asyncio
import copy
import dataclasses
import json
import multiprocessing as mp
import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, NamedTuple

import numpy as np
import torch

from ...engine.engine import Engine
from ...engine.state.program_state import ProgramMetrics, ProgramState, Step
from ...programs import PROGRAM_CLASS_MAPPING
from ...protocol import DataProto
from ...tinker.sampling_client import SamplingClient

_CREATE_WORKERS = 16


def _cfg_get(config, key: str, default=None):
    if config is None:
        return default
    if isinstance(config, dict):
        return config.get(key, default)
    return getattr(config, key, default)


@dataclass
class ProgramTransformConfig:
    max_seq_length: int
    max_prompt_length: int
    moe_replay: bool = False
    save_programs_flag: bool = False
    filter_program_errors: bool = True
    train_batch_size: int = 1
    n_samples: int = 1

    @classmethod
    def from_config(cls, config) -> "ProgramTransformConfig":
        decoding = _cfg_get(config, "decoding", None)
        return cls(max_seq_length=_cfg_get(config, "max_seq_length"), max_prompt_length=_cfg_get(config, "max_prompt_length"),
                   moe_replay=bool(_cfg_get(config, "moe_replay", False)),
                   save_programs_flag=bool(_cfg_get(config, "save_programs_flag", False)),
                   filter_program_errors=bool(_cfg_get(config, "filter_program_errors", True)),
                   train_batch_size=int(_cfg_get(config, "train_batch_size", 1) or 1),
                   n_samples=int(_cfg_get(decoding, "n", 1) or 1))


# ------------------------------------------------------------------------------------------ helpers
def _step_arrays(step: Step, moe_replay: bool):
    """Tokens / masks / logprobs of a step, cut after the last trainable token (trailing masked
    tokens carry no loss and only cost compute)."""
    tokens = np.asarray(step.tokens, dtype=np.int64)
    masks = np.asarray(step.masks, dtype=np.int64)
    logprobs = np.asarray(step.logprobs, dtype=np.float32)
    n = len(tokens)
    if len(masks) != n or len(logprobs) != n:
        raise ValueError(f"step {step.uid}: tokens/masks/logprobs lengths differ ({n}/{len(masks)}/{len(logprobs)})")
    nz = np.nonzero(masks)[0]
    keep = int(nz[-1]) + 1 if nz.size else n
    rm = None
    if moe_replay:
        raw = step.moe_routermap
        if isinstance(raw, torch.Tensor):
            raw = raw.cpu().numpy()
        raw = np.asarray(raw, dtype=np.int16) if raw is not None and len(raw) else np.zeros((0, 0, 0), np.int16)
        rm = raw[:keep] if raw.ndim == 3 else np.zeros((0, 0, 0), np.int16)
    return tokens[:keep], masks[:keep], logprobs[:keep], rm


def aggregate_program_metrics(metrics_list: list[ProgramMetrics]) -> dict:
    out: dict[str, float] = {}
    if not metrics_list:
        return out
    names = [f.name for f in dataclasses.fields(metrics_list[0])]
    cols = {n: [getattr(m, n) for m in metrics_list] for n in names}
    for name, vals in cols.items():
        vals = [v for v in vals if v is not None and v >= 0]
        if vals:
            arr = np.asarray(vals, dtype=np.float64)
            out[f"program/{name}_mean"], out[f"program/{name}_min"], out[f"program/{name}_max"] = \
                float(arr.mean()), float(arr.min()), float(arr.max())
    draft = sum(v for v in cols.get("spec_draft_tokens", []) if v and v > 0)
    acc = sum(v for v in cols.get("spec_accepted_tokens", []) if v and v > 0)
    ver = sum(v for v in cols.get("spec_verify_count", []) if v and v > 0)
    if draft > 0:
        out["program/spec_accept_rate"] = acc / draft
    if ver > 0:
        out["program/spec_accept_length"] = (acc + ver) / ver
    return out


def compute_position_ids(input_ids: torch.Tensor, attention_mask: torch.Tensor, multi_modal_inputs=None, processor=None):
    """Text models: running count of real tokens (0 on padding). Qwen-VL style processors get the
    4-row mRoPE layout ``[B, 4, T]`` — a text row followed by temporal/height/width rows."""
    text = (torch.cumsum(attention_mask, dim=1) - 1) * attention_mask
    ip = getattr(processor, "image_processor", None)
    if processor is None or ip is None or "Qwen2VLImageProcessor" not in type(ip).__name__:
        return text
    from ...models.vision import mrope_position_ids
    rows = []
    for i in range(input_ids.shape[0]):
        mm = multi_modal_inputs[i] if multi_modal_inputs and i < len(multi_modal_inputs) else {}
        vis = mrope_position_ids(processor, input_ids[i], attention_mask[i], mm.get("image_grid_thw"),
                                 mm.get("video_grid_thw"), mm.get("second_per_grid_ts"))
        rows.append(torch.cat([text[i:i + 1], vis], dim=0))
    return torch.stack(rows)


def compute_score_placement(program_rewards, step_numbers, attention_mask: torch.Tensor) -> torch.Tensor:
    """Every step's reward goes on its last real token; a scalar program reward is repeated for each
    of the program's steps, a list supplies one value per step."""
    assert len(program_rewards) == len(step_numbers)
    flat: list[float] = []
    for r, n in zip(program_rewards, step_numbers):
        if isinstance(r, (list, tuple)):
            assert len(r) == n, f"{len(r)} step rewards for {n} steps"
            flat.extend(float(x) for x in r)
        else:
            flat.extend([float(r)] * n)
    scores = torch.zeros(attention_mask.shape, dtype=torch.float32)
    last = attention_mask.sum(-1) - 1
    rows = torch.nonzero(last >= 0).flatten()
    scores[rows, last[rows]] = torch.tensor(flat, dtype=torch.float32)[rows]
    return scores


def prepare_program_metadata(batch: DataProto) -> None:
    """``num_program_tokens`` (trainable tokens over all rows of the row's program) and
    ``num_program_steps`` as tensors — denominators of the ``mean-program`` / ``program-mean`` loss
    reductions. Call when every step of each program is in the batch."""
    uids = batch.non_tensor_batch["program_uids"]
    mask = batch.batch["response_mask"]
    _, inv = np.unique(np.asarray([str(u) for u in uids]), return_inverse=True)
    inv_t = torch.from_numpy(inv).to(mask.device)
    per_row = mask.sum(-1)
    totals = torch.zeros(int(inv.max()) + 1 if len(inv) else 0, dtype=per_row.dtype, device=mask.device)
    totals.index_add_(0, inv_t, per_row)
    batch.batch["num_program_tokens"] = totals[inv_t]
    if "num_program_steps" in batch.non_tensor_batch:
        batch.batch["num_program_steps"] = torch.tensor([int(s) for s in batch.non_tensor_batch["num_program_steps"]],
                                                        dtype=torch.float32, device=mask.device)


# --------------------------------------------------------------------------------- ProgramProcessor
class ProgramProcessor:
    """Finished programs -> padded training batch. Holds only the tokenizer / processor."""

    def __init__(self, config: ProgramTransformConfig, tokenizer, processor=None):
        self.config = config
        self.tokenizer = tokenizer
        self.processor = processor

    @property
    def _pad_id(self) -> int:
        pid = getattr(self.tokenizer, "pad_token_id", None)
        return int(pid) if pid is not None else 0

    def transform_single_program(self, program: ProgramState) -> dict[str, Any]:
        steps: list[Step] = program.training_steps
        reward = program.reward
        per_step = [program.step_rewards.get(s.order_idx, reward) for s in steps] if program.step_rewards else None
        top = max((s.order_idx for s in steps), default=0)
        out = {"program_group_id": program.group_id, "program_uid": program.uid,
               "reward": per_step if per_step is not None else reward, "has_step_rewards": per_step is not None,
               "metrics": program.metrics, "step_numbers": len(steps), "metadata": program.metadata,
               "completions": [s.text for s in steps], "tokens": [], "logprobs": [], "masks": [], "moe_routermap": [],
               "multi_modal_data": [s.multi_modal_data for s in steps],
               "steps_id": [s.uid for s in steps], "steps_program_uid": [program.uid] * len(steps),
               "steps_program_group_id": [program.group_id] * len(steps),
               "steps_program_step_id": [f"{program.group_id}_step{s.order_idx}" for s in steps],
               "steps_total_step_num": [len(steps)] * len(steps),
               "steps_is_last_step": [s.order_idx == top for s in steps]}
        for s in steps:
            t, m, lp, rm = _step_arrays(s, self.config.moe_replay)
            out["tokens"].append(t)
            out["masks"].append(m)
            out["logprobs"].append(lp)
            out["moe_routermap"].append(rm)
        return out

    def transform_programs(self, programs: list[ProgramState], experiment_dir: str | None = None, global_steps: int = 0,
                           uid_to_index: dict | None = None) -> tuple[DataProto, dict]:
        T = self.config.max_seq_length
        per_prog = [self.transform_single_program(p) for p in programs]
        for tp in per_prog:
            assert tp["step_numbers"] > 0, "every program used for training needs at least one step"
        metrics = aggregate_program_metrics([tp["metrics"] for tp in per_prog])
        if self.config.save_programs_flag and experiment_dir:
            self.save_programs(per_prog, experiment_dir, global_steps)

        toks = [t[:T] for tp in per_prog for t in tp["tokens"]]
        msks = [m[:T] for tp in per_prog for m in tp["masks"]]
        lps = [l[:T] for tp in per_prog for l in tp["logprobs"]]
        B = len(toks)
        lens = np.fromiter((len(t) for t in toks), dtype=np.int64, count=B)
        rows = np.repeat(np.arange(B), lens)
        cols = np.arange(int(lens.sum())) - np.repeat(np.cumsum(lens) - lens, lens)
        ids = np.full((B, T), self._pad_id, dtype=np.int64)
        att = np.zeros((B, T), dtype=np.int64)
        rmask = np.zeros((B, T), dtype=np.int64)
        slp = np.zeros((B, T), dtype=np.float32)
        if B and lens.sum():
            ids[rows, cols] = np.concatenate(toks)
            att[rows, cols] = 1
            rmask[rows, cols] = np.concatenate(msks)
            slp[rows, cols] = np.concatenate(lps)
        input_ids, attention_mask = torch.from_numpy(ids), torch.from_numpy(att)

        mm_data = [d for tp in per_prog for d in tp["multi_modal_data"]]
        mm_inputs: list[dict] = []
        if self.processor is not None:
            for i, d in enumerate(mm_data):
                if not d:
                    mm_inputs.append({})
                    continue
                text = self.tokenizer.decode(ids[i, :lens[i]].tolist(), skip_special_tokens=True)
                enc = self.processor(text=[text], images=d.image, return_tensors="pt", **dict(d.processor_kwargs))
                enc = dict(enc)
                for k in ("input_ids", "attention_mask", "mm_token_type_ids"):
                    enc.pop(k, None)
                mm_inputs.append(enc)

        tensors = {
            "input_ids": input_ids, "attention_mask": attention_mask,
            "position_ids": compute_position_ids(input_ids, attention_mask, mm_inputs, self.processor),
            "responses": input_ids.clone(),
            "token_level_scores": compute_score_placement([tp["reward"] for tp in per_prog],
                                                          [tp["step_numbers"] for tp in per_prog], attention_mask),
            "response_mask": torch.from_numpy(rmask), "sampler_log_probs": torch.from_numpy(slp),
        }
        if self.config.moe_replay:
            tensors["moe_routermap"] = self._pad_routermaps([r for tp in per_prog for r in tp["moe_routermap"]], T)

        def col(key, dtype=object):
            return np.array([v for tp in per_prog for v in tp[key]], dtype=dtype)
        group_ids = col("steps_program_group_id")
        non_tensors = {
            "uid": group_ids, "step_ids": col("steps_id"), "program_uids": col("steps_program_uid"),
            "program_group_ids": group_ids.copy(), "program_step_ids": col("steps_program_step_id"),
            "num_program_steps": col("steps_total_step_num"), "is_last_step": col("steps_is_last_step"),
            "has_step_rewards": np.array([tp["has_step_rewards"] for tp in per_prog for _ in range(tp["step_numbers"])], dtype=object),
            "is_padding": np.array([False] * B, dtype=object),
        }
        if self.processor is not None and any(mm_inputs):
            non_tensors["multi_modal_inputs"] = np.array(mm_inputs, dtype=object)
        if uid_to_index:
            non_tensors["index"] = np.array([uid_to_index.get(u, -1) for u in group_ids], dtype=np.int64)
        batch = DataProto.from_dict(tensors=tensors, non_tensors=non_tensors)
        prepare_program_metadata(batch)
        return batch, metrics

    @staticmethod
    def _pad_routermaps(maps: list, T: int) -> torch.Tensor:
        shape = next(((m.shape[1], m.shape[2]) for m in maps if m is not None and m.ndim == 3 and m.size), (0, 0))
        out = np.full((len(maps), T, shape[0], shape[1]), -1, dtype=np.int16)
        for i, m in enumerate(maps):
            if m is not None and m.ndim == 3 and m.size:
                n = min(T, m.shape[0])
                out[i, :n] = m[:n]
        return torch.from_numpy(out)

    def create_dummy_batch(self, original_batch: DataProto, batch_size: int | None = None, n_samples: int | None = None,
                           global_steps: int = 0) -> DataProto:
        """A batch of the production schema filled to ``max_seq_length`` — one single-step program per
        sample — for memory stress tests and warm-up of the training path."""
        bs = batch_size or self.config.train_batch_size
        n = n_samples or self.config.n_samples
        T, P = self.config.max_seq_length, self.config.max_prompt_length
        uids = list(original_batch.non_tensor_batch.get("uid", []))[:bs] if original_batch is not None else []
        uids += [f"dummy-{global_steps}-{i}" for i in range(len(uids), bs)]
        programs = []
        tok = max(0, min(self._pad_id + 1, getattr(self.tokenizer, "vocab_size", 2) - 1))
        for g, uid in enumerate(uids):
            for k in range(n):
                st = Step(uid=f"{uid}-{k}-s0", session_id=f"{uid}-{k}", order_idx=0)
                st.tokens = [tok] * T
                st.masks = [0] * P + [1] * (T - P)
                st.logprobs = [0.0] * T
                st.token_len = T
                ps = ProgramState(group_id=str(uid), uid=f"{uid}-{k}", session_id=f"{uid}-{k}", done=True,
                                  reward=float((g + k) % 2))
                ps.training_steps = [st]
                programs.append(ps)
        cfg = dataclasses.replace(self.config, moe_replay=False, save_programs_flag=False)
        batch, _ = ProgramProcessor(cfg, self.tokenizer, None).transform_programs(programs)
        return batch

    def save_programs(self, transformed: list[dict], experiment_dir: str, global_steps: int) -> None:
        """One JSON line per program under ``generations/{step}.jsonl``."""
        out_dir = os.path.join(experiment_dir, "generations")
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, f"{global_steps}.jsonl"), "w") as f:
            for tp in transformed:
                rec = {"program_uid": tp["program_uid"], "program_group_id": tp["program_group_id"], "reward": tp["reward"],
                       "num_steps": tp["step_numbers"], "completions": tp["completions"], "metadata": tp["metadata"],
                       "num_tokens": [int(len(t)) for t in tp["tokens"]]}
                f.write(json.dumps(rec, default=str) + "\n")

    def visualize_program(self, batch: DataProto, sample_idx: int = 0, max_chars: int = 2000) -> str:
        """Decoded row with the trained region bracketed, for eyeballing masks."""
        ids = batch.batch["input_ids"][sample_idx]
        n = int(batch.batch["attention_mask"][sample_idx].sum())
        rm = batch.batch["response_mask"][sample_idx][:n].tolist()
        parts, cur, flag = [], [], None
        for t, m in zip(ids[:n].tolist(), rm):
            if flag is not None and m != flag:
                parts.append((flag, cur))
                cur = []
            cur.append(t)
            flag = m
        if cur:
            parts.append((flag, cur))
        text = "".join(("[[" + self.tokenizer.decode(c) + "]]") if f else self.tokenizer.decode(c) for f, c in parts)
        score = float(batch.batch["token_level_scores"][sample_idx].sum())
        return f"score={score:.3f} tokens={n} trained={sum(rm)}\n{text[:max_chars]}"


# ------------------------------------------------------------------------------------ ProgramRunner
@dataclass
class ProgramConfig:
    program_name: str = "react"
    program_kwargs: dict = field(default_factory=dict)
    program_timeout: float | None = None
    filter_program_errors: bool = True
    endpoint_enable: bool = False
    endpoint_host: str = "127.0.0.1"
    endpoint_port: int = 8000
    max_concurrency: int = 64
    max_subprocess_concurrency: int = 64
    terminate_on_error: bool = False
    partial_rollout_enable: bool = False
    collect_poll_interval: float = 0.05

    @classmethod
    def from_config(cls, config) -> "ProgramConfig":
        prog = _cfg_get(config, "program", {}) or {}
        prog = prog.to_dict() if hasattr(prog, "to_dict") else dict(prog)
        ep = _cfg_get(config, "engine_endpoint", {}) or {}
        pr = _cfg_get(config, "partial_rollout", {}) or {}
        return cls(program_name=prog.get("name", "react"), program_kwargs={k: v for k, v in prog.items() if k != "name"},
                   program_timeout=_cfg_get(config, "program_timeout", None),
                   filter_program_errors=bool(_cfg_get(config, "filter_program_errors", True)),
                   endpoint_enable=bool(_cfg_get(ep, "enable", False)), endpoint_host=_cfg_get(ep, "host", "127.0.0.1"),
                   endpoint_port=int(_cfg_get(ep, "port", 8000)), max_concurrency=int(_cfg_get(config, "max_concurrency", 64) or 0),
                   max_subprocess_concurrency=int(_cfg_get(config, "max_subprocess_concurrency", 64) or 64),
                   terminate_on_error=bool(_cfg_get(config, "terminate_on_error", False)),
                   partial_rollout_enable=bool(_cfg_get(pr, "enable", False)))


def _subprocess_entry(program, sem) -> None:
    with sem:
        asyncio.run(program.run_program())


class ProgramRunner:
    """Creates programs for a batch of dataset rows and drives them to completion.

    In-process programs are asyncio tasks on a dedicated loop thread (``set_tasks_loop``); with the
    endpoint enabled each program runs ``run_program`` in its own child process and reaches the
    engine over HTTP. ``run_and_collect`` returns once the engine reports that every live session is
    either finished or parked on a partial-rollout future."""

    def __init__(self, config: ProgramConfig, engine: Engine, sampling_client=None, hybrid_engine: bool = False):
        self.config = config
        self.engine = engine
        self.sampling_client = sampling_client
        self.hybrid_engine = hybrid_engine
        self._limit = config.max_concurrency if config.max_concurrency > 0 else 10 ** 9
        self._run_sem: asyncio.Semaphore | None = None
        self._process_sem = None
        self._tasks_loop: asyncio.AbstractEventLoop | None = None
        self.queued_programs: list = []
        self.subprocess_handles: list[mp.Process] = []
        self.failures: list[BaseException] = []

    def set_tasks_loop(self, loop: asyncio.AbstractEventLoop) -> None:
        self._tasks_loop = loop

    def shutdown(self) -> None:
        if self._tasks_loop is not None and self._tasks_loop.is_running():
            self._tasks_loop.call_soon_threadsafe(self._tasks_loop.stop)
        self._tasks_loop = None
        for p in self.subprocess_handles:
            if p.is_alive():
                p.terminate()
        self.subprocess_handles = []

    # -- creation ------------------------------------------------------------------------------
    def create_programs(self, batch: DataProto, global_steps: int) -> tuple[list, dict]:
        self.engine.set_global_steps(global_steps)
        cls = PROGRAM_CLASS_MAPPING[self.config.program_name]
        env_args = list(batch.non_tensor_batch["env_args"])
        uids = [str(u) for u in batch.non_tensor_batch["uid"]]
        idx = batch.non_tensor_batch.get("index", None)
        uid_to_index = {u: int(idx[i]) for i, u in enumerate(uids)} if idx is not None else {}
        sample_params = batch.meta_info.get("sample_params", {}) or {}

        def make(i: int):
            kw = copy.deepcopy(self.config.program_kwargs)
            row = json.loads(env_args[i]) if isinstance(env_args[i], str) else env_args[i]
            base = kw.get("env_args", {})
            if isinstance(base, dict):
                kw["env_args"] = {**base, **row}
            if "program_timeout" not in kw and self.config.program_timeout is not None:
                kw["program_timeout"] = self.config.program_timeout
            prog = cls(**kw)
            if not isinstance(base, dict):
                prog.env_args = row
            if self.config.endpoint_enable:
                prog.set_endpoint_url(f"http://{self.config.endpoint_host}:{self.config.endpoint_port}")
            else:
                prog.set_engine(self.engine)
            prog.set_group_id(uids[i])
            if sample_params:
                prog.set_sample_params(dict(sample_params))
            return prog

        with ThreadPoolExecutor(max_workers=_CREATE_WORKERS) as pool:
            programs = list(pool.map(make, range(len(env_args))))
        self.queued_programs = programs
        return programs, uid_to_index

    # -- execution -----------------------------------------------------------------------------
    async def run_and_collect(self, val: bool = False) -> tuple[list[ProgramState], dict]:
        eng = self.engine
        if self.hybrid_engine and self.sampling_client is not None:
            await self.sampling_client.wake_up()
        eng.set_validation_mode(val)
        if not val:
            await eng.run_in_engine_loop_async(eng.resume_partial_rollout_programs())
        if self.queued_programs:
            if not self.config.endpoint_enable:
                await asyncio.gather(*(p.init_session(group_id=p.group_id, sample_params=getattr(p, "sample_params", None))
                                       for p in self.queued_programs))
                self._launch_in_process(self.queued_programs)
            else:
                self._launch_subprocesses(self.queued_programs)
            self.queued_programs = []
        last_note = time.monotonic()
        while True:
            if self.failures and self.config.terminate_on_error:
                raise self.failures[0]
            if self.config.endpoint_enable and any(p.is_alive() for p in self.subprocess_handles):
                safe = False
            else:
                safe = await eng.run_in_engine_loop_async(eng.all_programs_safe_to_collect())
            if safe:
                break
            await asyncio.sleep(self.config.collect_poll_interval)
            if time.monotonic() - last_note >= 30:
                print("[program-runner] waiting: " + await eng.run_in_engine_loop_async(eng.get_session_diagnostics()), flush=True)
                last_note = time.monotonic()
        engine_metrics = await eng.run_in_engine_loop_async(eng.get_engine_metrics())
        finished = await eng.run_in_engine_loop_async(eng.get_finished_programs(validation=val))
        engine_metrics["engine/returned_programs"] = len(finished)
        self.subprocess_handles = [p for p in self.subprocess_handles if p.is_alive()]
        eng.set_validation_mode(False)
        if self.hybrid_engine and self.sampling_client is not None:
            await self.sampling_client.sleep()
        return finished, engine_metrics

    def _launch_in_process(self, programs) -> None:
        assert self._tasks_loop is not None, "set_tasks_loop() must be called before running in-process programs"

        async def guarded(program):
            if self._run_sem is None:
                self._run_sem = asyncio.Semaphore(self._limit)
            try:
                async with self._run_sem:
                    await program.run_program()
            except Exception as e:   # the engine has already closed the session with the failure reward
                import traceback
                traceback.print_exc()
                self.failures.append(e)

        for p in programs:
            asyncio.run_coroutine_threadsafe(guarded(p), self._tasks_loop)

    def _launch_subprocesses(self, programs) -> None:
        ctx = mp.get_context("spawn")
        if self._process_sem is None:
            self._process_sem = ctx.Semaphore(self.config.max_subprocess_concurrency)
        for p in programs:
            proc = ctx.Process(target=_subprocess_entry, args=(p, self._process_sem), daemon=True)
            proc.start()
            self.subprocess_handles.append(proc)


# ------------------------------------------------------------------------------------------ factory
class ProgramComponents(NamedTuple):
    sampling_client: SamplingClient
    engine: Engine
    program_processor: ProgramProcessor
    program_runner: ProgramRunner
    tasks_loop: asyncio.AbstractEventLoop | None


def create_program_components(config, tokenizer, processor, server_addresses: list, sampler_servers: list | None = None,
                              hybrid_engine: bool = False, thread_name_prefix: str = "Pipeline") -> ProgramComponents:
    """The standard set for rollouts — used by the driver process and, in the asynchronous mode, by
    the sampler workers that run programs next to their servers."""
    addresses = list(sampler_servers) if sampler_servers else list(server_addresses)
    sampling_client = SamplingClient(addresses, tokenizer=tokenizer)
    pr = _cfg_get(config, "partial_rollout", {}) or {}
    engine_kwargs = dict(_cfg_get(config, "engine_args", {}) or {})
    decoding = _cfg_get(config, "decoding", {}) or {}
    decoding = decoding.to_dict() if hasattr(decoding, "to_dict") else dict(decoding)
    engine = Engine(sampling_client=sampling_client, tokenizer=tokenizer, processor=processor,
                    max_seq_length=_cfg_get(config, "max_seq_length", 8192),
                    max_prompt_length=_cfg_get(config, "max_prompt_length", 1024), max_steps=_cfg_get(config, "max_steps", 64),
                    max_tokens_per_step=_cfg_get(config, "max_tokens_per_step", None),
                    prompt_truncation=_cfg_get(config, "prompt_truncation", None),
                    enable_partial_rollout=bool(_cfg_get(pr, "enable", False)),
                    partial_rollout_n_iters=int(_cfg_get(pr, "n_iters", 1) or 1), moe_replay=bool(_cfg_get(config, "moe_replay", False)),
                    default_sample_params={k: v for k, v in decoding.items() if k != "n"}, **engine_kwargs)
    processor_ = ProgramProcessor(ProgramTransformConfig.from_config(config), tokenizer, processor)
    pcfg = ProgramConfig.from_config(config)
    runner = ProgramRunner(pcfg, engine, sampling_client=sampling_client, hybrid_engine=hybrid_engine)
    loop = None
    if not pcfg.endpoint_enable:
        loop = asyncio.new_event_loop()
        threading.Thread(target=loop.run_forever, name=f"{thread_name_prefix}-ProgramsLoop", daemon=True).start()
        runner.set_tasks_loop(loop)
    return ProgramComponents(sampling_client, engine, processor_, runner, loop)
