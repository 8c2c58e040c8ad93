"""GPU resource pools: how many worker processes run on each node (reference: axon/core/resource_pool.py)."""
from __future__ import annotations


class ResourcePool:
    def __init__(self, process_on_nodes: list[int] | None = None, max_colocate_count: int = 10,
                 n_gpus_per_node: int = 8, name_prefix: str = "", device_offset: int = 0):
        self._store = list(process_on_nodes or [])
        self.max_colocate_count = max_colocate_count
        self.n_gpus_per_node = n_gpus_per_node
        self.name_prefix = name_prefix
        self.device_offset = device_offset      # first local GPU index this pool may use

    def add_node(self, process_count: int) -> None:
        self._store.append(process_count)

    @property
    def world_size(self) -> int:
        return sum(self._store)

    def __call__(self) -> list[int]:
        return self._store

    @property
    def store(self) -> list[int]:
        return self._store

    def local_world_size_list(self) -> list[int]:
        return [n for n in self._store for _ in range(n)]

    def local_rank_list(self) -> list[int]:
        return [i for n in self._store for i in range(n)]

    def node_rank_list(self) -> list[int]:
        return [j for j, n in enumerate(self._store) for _ in range(n)]


def split_trainer_sampler_pools(num_nodes: int, gpus_per_node: int, ratio: int | float, hybrid: bool):
    """Hybrid: one pool with every GPU. Disaggregated: ``num_train = total // (ratio + 1)`` trainer GPUs,
    the rest go to the sampler (ratio = sampler GPUs per trainer GPU)."""
    total = num_nodes * gpus_per_node
    if hybrid:
        return {"global": ResourcePool([gpus_per_node] * num_nodes, n_gpus_per_node=gpus_per_node)}
    n_train = max(1, int(total // (ratio + 1)))
    n_samp = total - n_train
    assert n_samp > 0, "disaggregated mode needs at least one sampler GPU"

    def layout(n, offset):
        full, rem = divmod(n, gpus_per_node)
        return [gpus_per_node] * full + ([rem] if rem else []), offset

    tl, _ = layout(n_train, 0)
    sl, _ = layout(n_samp, 0)
    return {"trainer": ResourcePool(tl, n_gpus_per_node=gpus_per_node, name_prefix="trainer", device_offset=0),
            "sampler": ResourcePool(sl, n_gpus_per_node=gpus_per_node, name_prefix="sampler",
                                    device_offset=n_train % gpus_per_node if num_nodes == 1 else 0)}
