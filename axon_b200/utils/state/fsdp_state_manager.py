"""Checkpoint save / load for the sharded data-parallel trainer.

File names follow the reference's FSDP layout so tooling that walks checkpoints keeps working
(``model_world_size_{W}_rank_{R}.pt``, ``optim_…``, ``extra_state_…``, ``fsdp_config.json``,
``huggingface/``; reference: axon/utils/state/fsdp_state_manager.py:97-364). Contents differ by
design: every rank holds the full bf16 parameters and a 1/W shard of the fp32 master weights and
Adam moments, so the per-rank model file stores that rank's contiguous slice of the flat parameter
buffer and the optimizer file its slice of master / exp_avg / exp_avg_sq plus the step count.

Asynchronous save: tensors are first copied into pinned host buffers on the compute stream (the
training step may continue as soon as that copy is enqueued and synchronised), then a background
thread serialises them; ``wait()`` joins the writer and is called before the next save and on exit.
"""
from __future__ import annotations

import json
import os
import threading

import torch

from .state_manager import BaseStateManager, StateSaveMode
from .utils import delete_oldest_checkpoints


def _barrier(group=None) -> None:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)


class FSDPStateManager(BaseStateManager):
    """``model`` is the policy model (flat parameters), ``optimizer`` the PolicyEngine that owns the
    sharded optimizer state."""

    layout_tag = "zero1-flat"

    def __init__(self, model, optimizer, lr_scheduler=None, processing_class=None, rank=None, world_size=None,
                 process_group=None):
        super().__init__(model, optimizer, lr_scheduler, processing_class, rank, world_size)
        self.pg = process_group
        self._writer: threading.Thread | None = None
        self._writer_error: BaseException | None = None

    # -- helpers -------------------------------------------------------------------------------
    def _name(self, kind: str) -> str:
        return f"{kind}_world_size_{self.world_size}_rank_{self.rank}.pt"

    def wait(self) -> None:
        if self._writer is not None:
            self._writer.join()
            self._writer = None
        if self._writer_error is not None:
            err, self._writer_error = self._writer_error, None
            raise RuntimeError("asynchronous checkpoint write failed") from err

    @staticmethod
    def _to_host(t: torch.Tensor | None, pin: bool) -> torch.Tensor | None:
        if t is None:
            return None
        if t.device.type == "cpu":
            return t.detach().clone()
        out = torch.empty(t.shape, dtype=t.dtype, pin_memory=pin)
        out.copy_(t, non_blocking=True)
        return out

    def _export_state_dict(self, want_hf: bool, pin: bool):
        """HF-named whole tensors on the host for the export (rank 0 only; None elsewhere)."""
        if want_hf and self.rank == 0:
            return {k: self._to_host(v, pin) for k, v in self.model.params.to_hf_state_dict().items()}
        return None

    # -- save ----------------------------------------------------------------------------------
    def save_state(self, local_path: str, global_step: int = 0, max_ckpt_to_keep: int | None = None,
                   save_mode: str | None = None, async_save: bool | None = None):
        if local_path is None:
            return
        self.wait()
        mode = StateSaveMode(save_mode) if save_mode else StateSaveMode.SHARDED
        sharded = mode in (StateSaveMode.SHARDED, StateSaveMode.BOTH)
        want_hf = mode in (StateSaveMode.HF, StateSaveMode.BOTH)
        os.makedirs(local_path, exist_ok=True)
        hf_dir = os.path.join(local_path, "huggingface")
        os.makedirs(hf_dir, exist_ok=True)
        _barrier(self.pg)
        eng, params = self.optimizer, self.model.params
        lo, hi = eng.shard
        eng.load_optimizer()          # state may be parked on the host during rollout
        pin = bool(async_save) and torch.cuda.is_available()
        files: dict[str, dict] = {}
        if sharded:
            files[self._name("model")] = {"flat_shard": self._to_host(params.flat[lo:hi], pin), "range": (lo, hi),
                                          "numel": params.flat.numel(), "dtype": str(params.flat.dtype)}
        files[self._name("optim")] = {"master": self._to_host(eng.master, pin), "exp_avg": self._to_host(eng.exp_avg, pin),
                                      "exp_avg_sq": self._to_host(eng.exp_avg_sq, pin), "step": eng.opt_step, "range": (lo, hi)}
        files[self._name("extra_state")] = {"lr_scheduler": {"opt_step": eng.opt_step, "sched_step": getattr(eng, "sched_step", eng.opt_step)},
                                            "rng": self.get_rng_state(), "global_step": global_step}
        hf_sd = self._export_state_dict(want_hf, pin)
        if torch.cuda.is_available() and params.flat.is_cuda:
            torch.cuda.current_stream().synchronize()

        def write():
            for name, payload in files.items():
                tmp = os.path.join(local_path, name + ".tmp")
                torch.save(payload, tmp)
                os.replace(tmp, os.path.join(local_path, name))
            if self.rank == 0:
                with open(os.path.join(local_path, "fsdp_config.json"), "w") as f:
                    json.dump({"FSDP_version": self.layout_tag, "world_size": self.world_size}, f, indent=4)
                from ..hf_model import save_hf_model
                if hf_sd is not None:
                    save_hf_model(params, hf_dir, cfg=params.cfg, tokenizer=self.processing_class, state_dict=hf_sd)
                else:
                    params.cfg.save_pretrained(hf_dir)
                    if self.processing_class is not None and hasattr(self.processing_class, "save_pretrained"):
                        self.processing_class.save_pretrained(hf_dir)

        def rotate():
            if max_ckpt_to_keep and max_ckpt_to_keep > 0 and self.rank == 0:
                root = os.path.dirname(os.path.dirname(os.path.abspath(local_path)))
                delete_oldest_checkpoints(root, max_ckpt_to_keep)

        if async_save:
            def run():
                try:
                    write()
                    rotate()
                except BaseException as e:       # noqa: BLE001 - surfaced by wait()
                    self._writer_error = e
            self._writer = threading.Thread(target=run, name="ckpt-writer", daemon=True)
            self._writer.start()
        else:
            write()
            _barrier(self.pg)
            threading.Thread(target=rotate, daemon=True).start()

    # -- load ----------------------------------------------------------------------------------
    def load_state(self, local_path: str, save_mode: str | None = None):
        if local_path is None:
            return
        self.wait()
        if os.path.exists(os.path.join(local_path, "dist_ckpt", "metadata.json")) and not os.path.exists(os.path.join(local_path, self._name("optim"))):
            # written by a model-parallel run in the layout-independent array store: every rank reads whole tensors
            from .megatron_state_manager import MegatronStateManager
            return MegatronStateManager(self.model, self.optimizer, dp_rank=self.rank, rank=self.rank, world_size=self.world_size,
                                        process_group=self.pg).load_state(local_path)
        mode = StateSaveMode(save_mode) if save_mode else StateSaveMode.SHARDED
        eng, params = self.optimizer, self.model.params
        lo, hi = eng.shard
        dev = params.flat.device
        cfg_path = os.path.join(local_path, "fsdp_config.json")
        if os.path.exists(cfg_path):
            saved_world = json.load(open(cfg_path)).get("world_size", self.world_size)
            if saved_world != self.world_size:
                raise ValueError(f"checkpoint was written by {saved_world} ranks, this job has {self.world_size}; "
                                 "load it in 'hf' mode or rerun with the original world size")
        if mode in (StateSaveMode.SHARDED, StateSaveMode.BOTH):
            blob = torch.load(os.path.join(local_path, self._name("model")), map_location="cpu", weights_only=False)
            assert tuple(blob["range"]) == (lo, hi) and blob["numel"] == params.flat.numel(), "parameter layout changed"
            params.flat[lo:hi].copy_(blob["flat_shard"].to(dev))
            if self.world_size > 1:
                eng._all_gather_params()
        else:
            from ..hf_model import load_hf_weights
            load_hf_weights(self.model, os.path.join(local_path, "huggingface"))
        opt = torch.load(os.path.join(local_path, self._name("optim")), map_location="cpu", weights_only=False)
        assert tuple(opt["range"]) == (lo, hi), "optimizer shard boundaries changed"
        eng._host_state = None
        eng.master = opt["master"].to(dev)
        eng.exp_avg, eng.exp_avg_sq = opt["exp_avg"].to(dev), opt["exp_avg_sq"].to(dev)
        eng.opt_step = int(opt["step"])
        extra = torch.load(os.path.join(local_path, self._name("extra_state")), map_location="cpu", weights_only=False)
        if "rng" in extra:
            self.load_rng_state(extra["rng"])
        sched = extra.get("lr_scheduler") or {}
        eng.opt_step = int(sched.get("opt_step", eng.opt_step))
        if hasattr(eng, "sched_step"):
            eng.sched_step = int(sched.get("sched_step", eng.opt_step))
        _barrier(self.pg)


class ShardedFamilyStateManager(FSDPStateManager):
    """Checkpoints of a family model with parameter shards (``models/sharded_family.py``): every rank writes its own
    pieces and optimizer state (the files of the flat layout, with the rank's whole local buffer as its range), the HF
    export gathers one layer at a time and is written by rank 0. Resuming needs the writing world size; any other
    layout starts from the HF export."""
    layout_tag = "layer-pieces"

    def __init__(self, model, optimizer, group=None, **kw):
        super().__init__(model, optimizer, process_group=group, **kw)

    def _export_state_dict(self, want_hf: bool, pin: bool):
        if not want_hf:
            return None
        out = {} if self.rank == 0 else None
        shape_of = getattr(self.model.spec, "checkpoint_shape", lambda n: None)
        for name, t in self.model.full_named_tensors():       # a collective: every rank walks all layers
            if out is not None:
                t = t if shape_of(name) is None else t.reshape(shape_of(name))
                out[name] = self._to_host(t, False)
        if torch.cuda.is_available() and self.model.params.flat.is_cuda:
            torch.cuda.current_stream().synchronize()
        return out
