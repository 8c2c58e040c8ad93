"""Colocated (hybrid-engine) RL step on one process per GPU.

Each rank hosts the policy trainer and the sampler on the SAME device and the SAME bf16 weight
buffer (the sampler reads the trainer's flat parameters in place), so the trainer->sampler weight
sync of the hybrid topology is a stream-ordered hand-over with no copy. One ``step``:

    prompts (pinned host) --H2D--> rollout (continuous batching, n samples per prompt)
      -> rewards -> training batch (reference schema) -> group-relative advantages
      -> old log-probs (forward) -> mini-batches: forward_backward + optim_step
      -> weight hand-over to the sampler -> scalar metrics (D2H)

Memory phases follow the reference's hybrid engine (sleep / wake, optimizer offload:
axon/driver/sync_ppo.py:285-454, axon/sampler/mixins/sync_mixin.py:86-168): the KV pool exists only
during rollout; gradient and (optionally) optimizer buffers exist only during training.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np
import torch
import torch.distributed as dist

from ..models.dense import DenseModel
from ..protocol import DataProto
from ..sampler.engine import GenerationEngine
from ..sampler.kv_cache import PagedKVCache
from ..sampler.params import SamplingParams
from ..trainer.algos import compute_advantage
from ..trainer.policy import OptimConfig, PolicyEngine


@dataclass
class RLStepConfig:
    n_samples: int = 8                   # group size
    max_prompt_length: int = 1024
    max_response_length: int = 4096
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    loss: str = "ppo"
    loss_args: dict = field(default_factory=lambda: {"clip_ratio": 0.2})
    advantage: str = "grpo"
    advantage_args: dict = field(default_factory=dict)
    mini_batch_size: int = 64            # prompts per optimizer step (x n_samples rows)
    ppo_epochs: int = 1
    max_token_len_per_gpu: int = 8192
    use_sampler_logprobs: bool = False
    kv_memory_fraction: float = 0.85     # of the memory free at rollout time
    kv_expected_fill: float = 0.4        # share of the worst case (every sequence at full length at once) the KV pool is sized for
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 32768
    offload_optimizer: bool | None = None  # None: decide from free memory
    recompute: str = "auto"                # activation recomputation: auto | full | selective | none
    optim: OptimConfig = field(default_factory=OptimConfig)


def build_training_batch(prompts: list[list[int]], outputs, rewards, group_ids, pad_id: int, max_len: int) -> DataProto:
    """Rows in the reference's training schema: right-padded full sequences, ``responses == input_ids``,
    ``response_mask`` on generated tokens, the scalar reward on the last generated token."""
    B = len(outputs)
    T = min(max_len, max(len(p) + len(o.token_ids) for p, o in zip(prompts, outputs)))
    ids = np.full((B, T), pad_id, dtype=np.int64)
    att = np.zeros((B, T), dtype=np.int64)
    resp = np.zeros((B, T), dtype=np.float32)
    slp = np.zeros((B, T), dtype=np.float32)
    score = np.zeros((B, T), dtype=np.float32)
    for i, (p, o) in enumerate(zip(prompts, outputs)):
        seq = (p + o.token_ids)[:T]
        n, lp = len(seq), len(p)
        ids[i, :n] = seq
        att[i, :n] = 1
        resp[i, lp:n] = 1
        slp[i, lp:n] = o.logprobs[: n - lp]
        if n > lp:
            score[i, n - 1] = rewards[i]
    pos = np.broadcast_to(np.arange(T), (B, T)) * att
    tensors = {"input_ids": torch.from_numpy(ids), "attention_mask": torch.from_numpy(att),
               "position_ids": torch.from_numpy(pos.copy()), "responses": torch.from_numpy(ids.copy()),
               "response_mask": torch.from_numpy(resp), "sampler_log_probs": torch.from_numpy(slp),
               "token_level_scores": torch.from_numpy(score), "token_level_rewards": torch.from_numpy(score.copy())}
    nt = {"uid": np.array(group_ids, dtype=object)}
    return DataProto.from_dict(tensors, nt)


def attach_valid_counts(mini: DataProto, process_group=None) -> None:
    """Mini-batch-global denominators so every micro-batch / rank divides by the same numbers
    (``process_mini_batch`` in the reference: axon/driver/driver_utils.py:436)."""
    rm = mini.batch["response_mask"]
    tok = rm.sum().float()
    rows = (rm.sum(-1) > 0).sum().float()
    cnt = torch.stack([tok, rows])
    # an explicit group decides (a group of one rank needs no reduction); without one the default group is used
    if process_group is not None:
        reduce = dist.get_world_size(process_group) > 1
    else:
        reduce = dist.is_initialized() and dist.get_world_size() > 1
    if reduce:
        dev = "cuda" if dist.get_backend(process_group) == "nccl" else "cpu"
        c = cnt.to(dev)
        dist.all_reduce(c, group=process_group)
        cnt = c.cpu()
    B = len(mini)
    mini.batch["valid_token_count"] = cnt[0].expand(B).clone()
    mini.batch["valid_batch_size"] = cnt[1].expand(B).clone()
    mini.batch["valid_program_count"] = cnt[1].expand(B).clone()
    mini.batch["per_row_token_count"] = rm.sum(-1)


class ColocatedRLRunner:
    """One GRPO/PPO-style RL step per ``step()`` call on this rank's GPU (data parallel across ranks)."""

    def __init__(self, model: DenseModel, cfg: RLStepConfig, process_group=None, reward_fn=None, seed: int = 0):
        self.model, self.cfg, self.pg = model, cfg, process_group
        self.device = model.device
        self.policy = PolicyEngine(model, cfg.optim, process_group, cfg.max_token_len_per_gpu, cfg.temperature)
        self.engine: GenerationEngine | None = None
        self.reward_fn = reward_fn
        # without an explicit group the runner is data parallel over the default group (if one exists)
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        if process_group is None and dist.is_initialized():
            self.pg = dist.group.WORLD
        self.rng = np.random.default_rng(seed + 7919 * self.rank)
        self.seed = seed
        self.global_step = 0
        self.timing: dict[str, float] = {}
        self.phase_detail: dict = {}
        self._kv_peak_pages: int | None = None      # peak KV occupancy seen in earlier rollouts (pages)
        if self.device.type == "cuda":
            # Make step 1 look like every later step: the optimizer state exists from the start, and if
            # rollouts will need its memory the pinned host buffers it moves to are allocated now
            # (pinning tens of GB takes tens of seconds and must not land inside a step).
            self.policy.init_optimizer()
            if self._will_offload():
                self.policy.prepare_offload_buffers()

    def _kv_need(self) -> tuple[int, int]:
        need = PagedKVCache.bytes_per_page(self.model.cfg, self.model.params.flat.element_size())
        want_pages = self.cfg.max_num_seqs * ((self.cfg.max_prompt_length + self.cfg.max_response_length) // 128 + 1)
        return need, want_pages

    def _will_offload(self) -> bool:
        if self.cfg.offload_optimizer is not None:
            return bool(self.cfg.offload_optimizer)
        need, want_pages = self._kv_need()
        if self._kv_peak_pages is not None:
            # observed: the most pages any rollout so far held at once, with a quarter on top and a page per sequence
            want_pages = min(want_pages, int(self._kv_peak_pages * 1.25) + self.cfg.max_num_seqs)
            grads = 0 if self.model.params.grad_flat is None or getattr(self.model.params, "grads_persistent", False) \
                else self.model.params.grad_flat.numel() * 4
            return (self._free_bytes() + grads) * self.cfg.kv_memory_fraction < want_pages * need
        grads = 0 if self.model.params.grad_flat is None or getattr(self.model.params, "grads_persistent", False) \
            else self.model.params.grad_flat.numel() * 4
        # No rollout seen yet: size for a share of the worst case. Sequences finish at different times and samples of
        # a prompt share its pages, so the pool never holds the worst case; once a rollout has been observed its
        # peak occupancy decides (above). If the pool ever runs short the engine preempts and re-prefills. Moving
        # the optimizer state (12 bytes per parameter) over PCIe twice per step is only worth it when the expected
        # demand does not fit beside it.
        return (self._free_bytes() + grads) * self.cfg.kv_memory_fraction < want_pages * need * self.cfg.kv_expected_fill

    # ------------------------------------------------------------------ memory phases
    def _free_bytes(self) -> int:
        if self.device.type != "cuda":
            return 2 << 30
        torch.cuda.empty_cache()
        return torch.cuda.mem_get_info(self.device)[0]

    def _enter_rollout(self) -> None:
        ta = time.perf_counter()
        self.model.params.free_grads()
        need, want_pages = self._kv_need()
        off = self._will_offload()
        if off:
            self.policy.offload_optimizer()
        tb = time.perf_counter()
        pages = int(min(want_pages, self._free_bytes() * self.cfg.kv_memory_fraction // need))
        if self.engine is None:
            self.engine = GenerationEngine(self.model, num_pages=pages, max_num_seqs=self.cfg.max_num_seqs,
                                           max_num_batched_tokens=self.cfg.max_num_batched_tokens,
                                           seed=self.seed + self.rank)
        else:
            self.engine.wake_up(pages)
        self.engine.set_max_model_len(self.cfg.max_prompt_length + self.cfg.max_response_length)
        self.phase_detail = dict(offload=tb - ta, kv_alloc=time.perf_counter() - tb, kv_pages=pages, offloaded=bool(off))

    def _enter_training(self) -> None:
        if self.engine is not None:          # trainer-only ranks of a disaggregated run have no engine
            self.engine.sleep()
        self.policy.load_optimizer()
        if self.cfg.recompute == "auto" and self.device.type == "cuda":
            # keep as many activations as the memory left after parameters, gradients and optimizer
            # state allows (per token and layer: selective 2(3H + qkv) bytes, none adds 4F bytes)
            c = self.model.cfg
            tok = self.policy.max_tokens
            grads = 0 if self.model.params.grad_flat is not None else self.model.params.numel * 4
            free = self._free_bytes() - grads - (6 << 30)
            sel = 2 * (3 * c.hidden_size + c.qkv_size) * tok * c.num_hidden_layers
            non = sel + 4 * c.intermediate_size * tok * c.num_hidden_layers
            self.model.recompute = "none" if free > 1.25 * non else "selective" if free > 1.25 * sel else "full"
        elif self.cfg.recompute != "auto":
            self.model.recompute = self.cfg.recompute

    # ------------------------------------------------------------------ one RL step
    def step(self, prompt_ids: torch.Tensor, prompt_lens: torch.Tensor | None = None,
             response_caps: np.ndarray | None = None, rewards: np.ndarray | None = None) -> dict:
        """prompt_ids: int32 [P, Lp] (pinned host or device). response_caps: optional per-sample
        ``max_tokens`` [P * n] (synthetic length control; EOS is ignored for those rows). rewards:
        optional precomputed per-sample rewards [P * n]; otherwise ``reward_fn(prompt, output)``."""
        c = self.cfg
        t0 = time.perf_counter()
        prompts_dev = prompt_ids.to(self.device, non_blocking=True)
        P = prompts_dev.shape[0]
        lens = prompt_lens.tolist() if prompt_lens is not None else [prompts_dev.shape[1]] * P
        prompts_h = prompts_dev.cpu().tolist()   # the engine's scheduler keeps token lists on the host
        prompts, groups, params = [], [], []
        for i in range(P):
            for j in range(c.n_samples):
                prompts.append(prompts_h[i][: lens[i]])
                groups.append(f"{self.global_step}-{self.rank}-{i}")
                cap = int(response_caps[i * c.n_samples + j]) if response_caps is not None else c.max_response_length
                params.append(SamplingParams(temperature=c.temperature, top_k=c.top_k, top_p=c.top_p,
                                             max_tokens=cap, ignore_eos=response_caps is not None))
        self._enter_rollout()
        t1 = time.perf_counter()
        pre0 = self.engine.stats.get("preempted", 0)
        host0, steps0 = self.engine.stats.get("decode_host_prep_s", 0.0), self.engine.stats.get("decode_steps", 0)
        outs = self.engine.generate(prompts, params)
        self.phase_detail["decode_host_prep_s"] = self.engine.stats.get("decode_host_prep_s", 0.0) - host0
        self.phase_detail["decode_steps"] = self.engine.stats.get("decode_steps", 0) - steps0
        self.phase_detail["preempted"] = self.engine.stats.get("preempted", 0) - pre0      # sequences pushed back for lack of KV pages
        peak = self.engine.cache.num_pages - self.engine.cache.min_free
        self.phase_detail["kv_peak_pages"] = peak
        if self.phase_detail["preempted"] == 0:
            self._kv_peak_pages = max(peak, self._kv_peak_pages or 0)
        else:                                    # the pool was too small: the true demand is unknown, size for the rule of thumb again
            self._kv_peak_pages = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t2 = time.perf_counter()
        self._enter_training()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t2x = time.perf_counter()
        out = self.train_on_samples(prompts, outs, rewards, groups)
        self.timing["prepare_and_old_logprob"] += t2x - t2
        self.timing.update(setup=t1 - t0, rollout=t2 - t1, total=time.perf_counter() - t0, enter_training=t2x - t2,
                           offload=self.phase_detail.get("offload", 0.0), kv_alloc=self.phase_detail.get("kv_alloc", 0.0))
        out.update({f"time/{k}": v for k, v in self.timing.items()})
        return out

    def train_on_samples(self, prompts: list[list[int]], outs, rewards, groups: list[str]) -> dict:
        """The training half of a step on finished rollouts: rewards -> batch in the reference schema -> advantages ->
        old log-probs -> mini-batches of forward_backward + optim_step. ``outs[i]`` belongs to ``prompts[i]``; rows
        with equal ``groups[i]`` form one advantage group. Used by ``step`` and, on trainer-only ranks of a
        disaggregated run, directly."""
        c = self.cfg
        t2 = time.perf_counter()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t2a = time.perf_counter()
        if rewards is None:
            rewards = np.array([self.reward_fn(p, o) for p, o in zip(prompts, outs)], dtype=np.float32) \
                if self.reward_fn is not None else self.rng.binomial(1, 0.5, len(outs)).astype(np.float32)
        data = build_training_batch(prompts, outs, rewards, groups, self.model.cfg.pad_token_id,
                                    c.max_prompt_length + c.max_response_length)
        data.meta_info.update(temperature=c.temperature, global_steps=self.global_step)
        compute_advantage(data, {"advantage": c.advantage, "advantage_args": c.advantage_args})
        t2b = time.perf_counter()
        if c.use_sampler_logprobs:
            data.batch["old_log_probs"] = data.batch["sampler_log_probs"].clone()
        else:
            old = self.policy.forward(data, want_entropy=False)
            data.batch["old_log_probs"] = old.batch["log_probs"].cpu()
        rm = data.batch["response_mask"]
        gap = ((data.batch["old_log_probs"].exp() - data.batch["sampler_log_probs"].exp()).abs() * rm).sum() / rm.sum().clamp_min(1)
        t3 = time.perf_counter()
        rows_per_mini = min(len(data), c.mini_batch_size * c.n_samples)
        metrics: dict[str, list] = {}
        opt = {}
        for _ in range(c.ppo_epochs):
            for s in range(0, len(data), rows_per_mini):
                mini = data.slice(s, s + rows_per_mini)
                mini.meta_info = data.meta_info
                attach_valid_counts(mini, self.pg)
                m = self.policy.forward_backward(mini, c.loss, c.loss_args)
                opt = self.policy.optim_step()
                for k, v in m.items():
                    metrics.setdefault(k, []).extend(v)
        # hand the updated weights to the sampler: same buffer, ordered on the compute stream
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t4 = time.perf_counter()
        self.global_step += 1
        n_tok = int(data.batch["attention_mask"].sum())
        n_resp = int(rm.sum())
        self.timing = dict(prepare_and_old_logprob=t3 - t2, train=t4 - t3, total=t4 - t2,
                           enter_training=t2a - t2, build_batch=t2b - t2a, old_logprob=t3 - t2b)
        self.phase_detail["recompute"] = self.model.recompute
        return {"loss": float(np.sum(metrics.get("loss", [0.0]))), "grad_norm": opt.get("grad_norm", 0.0),
                "tokens": n_tok, "response_tokens": n_resp, "sequences": len(data),
                "reward_mean": float(np.mean(rewards)), "sampler_probs_diff_mean": float(gap),
                "entropy": float(np.mean(metrics.get("entropy", [0.0])))}
