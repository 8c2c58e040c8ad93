from .dataset import RLDataset, collate_rl_dataset
from .dataloader import DynamicDataLoader
from .data_sampler import SamplerType, create_data_sampler

__all__ = ["RLDataset", "collate_rl_dataset", "DynamicDataLoader", "SamplerType", "create_data_sampler"]
