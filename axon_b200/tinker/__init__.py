from .sampling_client import SamplingClient  # noqa: F401
from .training_client import TrainingClient  # noqa: F401
