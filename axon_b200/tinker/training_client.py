"""``TrainingClient``: thin controller-side facade over a trainer worker group exposing the
forward / forward_backward / optim_step / save_state / load_state surface
(reference: axon/tinker/training_client.py:28-202)."""
from __future__ import annotations

from contextlib import contextmanager

from ..protocol import DataProto


class TrainingClient:
    def __init__(self, worker_group, tokenizer=None):
        self.wg = worker_group
        self.tokenizer = tokenizer

    def forward(self, data: DataProto) -> DataProto:
        return self.wg.forward(data)

    def forward_backward(self, data: DataProto, loss_fn: str = "ppo", loss_fn_args: dict | None = None) -> DataProto:
        return self.wg.forward_backward(data, loss_fn=loss_fn, loss_fn_args=loss_fn_args or {})

    def optim_step(self, step_lr: bool = True) -> DataProto:
        return self.wg.optim_step(step_lr=step_lr)

    def save_state(self, path: str, global_step: int = 0, max_ckpt_to_keep: int | None = None,
                   save_mode: str = "sharded", async_save: bool = False):
        return self.wg.save_state(path, global_step=global_step, max_ckpt_to_keep=max_ckpt_to_keep,
                                  save_mode=save_mode, async_save=async_save)

    def load_state(self, path: str, save_mode: str = "sharded"):
        return self.wg.load_state(path, save_mode=save_mode)

    def get_tokenizer(self):
        return self.tokenizer

    @contextmanager
    def load_model_context(self, include_model: bool = True, include_optimizer: bool = True):
        """Bring offloaded parameters / optimizer state onto the device for the duration of the block."""
        self.wg.load_model(include_model=include_model, include_optimizer=include_optimizer)
        try:
            yield self
        finally:
            self.wg.offload_model(include_model=include_model, include_optimizer=include_optimizer)
