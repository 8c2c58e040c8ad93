"""RL algorithm plug-ins: loss and advantage registries."""
from .advantages import AdvantageFn, compute_advantage, register_advantage  # noqa: F401
from .loss import LossFn, agg_loss, compute_loss_fn, register_loss  # noqa: F401
