"""Worker-resident training on a batch that was delivered to the trainer ranks
(reference: axon/trainer/mixins/async_mixin.py:60-330).

The mini-batch loop runs inside the workers. Loss denominators are made mini-batch-GLOBAL exactly:
each rank counts its local trained tokens / rows / programs and the counts are summed over the
data-parallel group (the reference multiplies the local count by the group size, which is only
right when every rank holds the same amount). The number of mini-batches is agreed with a MAX
all-reduce so that every rank takes part in every optimizer step.
"""
from __future__ import annotations

import copy

import torch
import torch.distributed as dist

from ...controller.decorator import Dispatch, register
from ...protocol import DataProto
from ...utils.metrics import append_to_dict, compute_data_metrics, compute_timing_metrics, compute_trainer_sampler_mismatch_metrics, reduce_metrics


class AsyncTrainerMixin:
    active_batch: DataProto | None = None

    def _rows_group(self) -> int:
        """Ranks that work on the same rows of a batch: a sequence-parallel group, times the tensor- / pipeline- / context-
        parallel block of a model-parallel trainer (expert-parallel ranks hold different rows)."""
        return int(self.ulysses_sequence_parallel_size) * int(getattr(self, "rows_group_size", 1))

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def set_batch(self, batch: DataProto) -> bool:
        """Whole batch from the driver (host-channel mode): every rank keeps its own shard."""
        dp = self.world_size // self._rows_group()
        shards = batch.chunk(dp)
        self.active_batch = shards[self.rank // self._rows_group()]
        self.active_batch.meta_info = dict(batch.meta_info)
        return True

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def receive_batch_from_sampler(self, batch_uid: str) -> int:
        assert self.bridge_pg is not None, "bridge process group is not connected"
        src = self.world_size                       # bridge rank of sampler rank 0
        size = torch.zeros(1, dtype=torch.int64, device=self.device)
        dist.recv(size, src=src, group=self.bridge_pg)
        buf = torch.empty(int(size.item()), dtype=torch.uint8, device=self.device)
        dist.recv(buf, src=src, group=self.bridge_pg)
        from ...sampler.mixins.async_mixin import decode_object
        if not hasattr(self, "_batch_buffer_dict"):
            self._batch_buffer_dict = {}
        self._batch_buffer_dict[batch_uid] = decode_object(buf)
        return int(size.item())

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def set_batch_from_uid(self, batch_uid: str) -> bool:
        store = getattr(self, "_batch_buffer_dict", {})
        if batch_uid not in store:
            return False
        self.active_batch = store.pop(batch_uid)
        return True

    def _finish_old_log_probs(self, temperature: float) -> dict:
        self.active_batch.meta_info["temperature"] = temperature
        self.active_batch.meta_info["global_token_num"] = self.active_batch.batch["attention_mask"].sum(-1).tolist()
        return compute_trainer_sampler_mismatch_metrics(self.active_batch)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def use_sampler_log_probs(self, temperature: float) -> dict:
        self.active_batch.batch["old_log_probs"] = self.active_batch.batch["sampler_log_probs"].clone()
        return self._finish_old_log_probs(temperature)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def compute_log_prob_on_batch(self, temperature: float) -> dict:
        self.active_batch.meta_info["temperature"] = temperature
        out = self.engine.forward(self.active_batch, temperature=temperature, want_entropy=False)
        self.active_batch.batch["old_log_probs"] = out.batch["log_probs"].to("cpu")
        return self._finish_old_log_probs(temperature)

    def _global_count(self, value: int) -> int:
        if self.world_size == 1:
            return value
        t = torch.tensor([value], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, group=self.pg)
        # inside the optimizer's group only sequence- / context-parallel peers count the same rows again (the ranks of a
        # tensor- or pipeline-parallel block are not in it)
        return int(t.item()) // int(self.ulysses_sequence_parallel_size)

    def _global_max(self, value: int) -> int:
        if self.world_size == 1:
            return value
        t = torch.tensor([value], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
        return int(t.item())

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def train_on_batch(self, loss_fn: str, loss_fn_args: dict, epochs: int = 1, mini_batch_size: int | None = None,
                       mini_batch_shuffle: bool = False, mini_batch_seed: int | None = None) -> DataProto:
        from ...driver.driver_utils import _program_groups, process_mini_batch
        self.load_model(include_model=True, include_optimizer=True)
        try:
            data = self.active_batch
            dp = self.world_size // self._rows_group()
            groups = _program_groups(data.non_tensor_batch["program_uids"])
            uids = list(groups)
            local_mbs = max(1, (mini_batch_size // dp) if mini_batch_size and mini_batch_size > 0 else len(uids))
            n_mb = self._global_max(max(1, -(-len(uids) // local_mbs)))
            gen = torch.Generator().manual_seed(mini_batch_seed) if mini_batch_seed is not None else None
            metrics: dict = {}
            for epoch in range(epochs):
                order = [uids[j] for j in torch.randperm(len(uids), generator=gen).tolist()] if mini_batch_shuffle else uids
                per = -(-len(order) // n_mb)
                for i in range(n_mb):
                    rows = [r for u in order[i * per:(i + 1) * per] for r in groups[u]]
                    if not rows:                                    # this rank ran out of programs: an inert row keeps it in step
                        rows = [0]
                        mb = data.select_idxs(rows)
                        mb.batch["response_mask"] = torch.zeros_like(mb.batch["response_mask"])
                    else:
                        mb = data.select_idxs(rows)
                    mb.meta_info = dict(data.meta_info)
                    process_mini_batch(mb)
                    for key in ("valid_batch_size", "valid_token_count", "valid_program_count"):
                        if key in mb.batch:
                            mb.batch[key] = torch.full_like(mb.batch[key], self._global_count(int(mb.batch[key][0])))
                    out = self.forward_backward(mb, loss_fn=loss_fn, loss_fn_args=loss_fn_args)
                    append_to_dict(metrics, out.meta_info["metrics"])
                    last = epoch == epochs - 1 and i == n_mb - 1
                    append_to_dict(metrics, self.optim_step(step_lr=last).meta_info["metrics"])
            return DataProto(meta_info={"metrics": reduce_metrics(metrics)})
        finally:
            self.offload_model(include_model=True, include_optimizer=True)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_batch_metrics_and_clear(self, timing_raw: dict | None = None) -> dict:
        b = self.active_batch
        out = {"data": compute_data_metrics(b, use_critic=False, include_detail=True),
               "timing": compute_timing_metrics(b, timing_raw or {}, include_detail=True),
               "indices": (b.non_tensor_batch.get("index"), b.non_tensor_batch.get("pass_rate"))}
        self.active_batch = None
        return out
