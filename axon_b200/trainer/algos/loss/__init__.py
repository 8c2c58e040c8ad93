from . import loss as _loss  # noqa: F401  (registers the loss functions)
from .registry import LossFn, LossRegistryEntry, compute_loss_fn, get_loss_entry, get_loss_fn, register_loss
from .utils import agg_loss, clip_by_value, entropy_from_logits, masked_mean

__all__ = ["LossFn", "LossRegistryEntry", "register_loss", "get_loss_entry", "get_loss_fn", "compute_loss_fn",
           "agg_loss", "masked_mean", "clip_by_value", "entropy_from_logits"]
