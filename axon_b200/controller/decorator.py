"""``@register``: marks a worker method as remotely callable through a worker group and says how the
controller splits its arguments over workers (dispatch), which workers run it (execute) and how the
results are merged (collect). Reference: axon/controller/decorator.py:36-407.

Dispatch modes
  RANK_ZERO                   args pass through; result comes from rank 0 only
  ONE_TO_ALL                  every worker receives the same args; results returned as a list
  ALL_TO_ALL                  caller supplies per-worker args already; results returned as a list
  DP_COMPUTE_PROTO_WITH_FUNC  DataProto args are chunked over workers; results concatenated
  DIRECT_SAMPLER_METHOD       not callable through the controller (used inside colocated workers)
  make_nd_compute_dataproto_dispatch_fn(mesh)
                              chunk over the mesh's DATA-PARALLEL ranks only (model-parallel peers get
                              the same chunk) and collect from the ranks the worker marked ``is_collect``
"""
from __future__ import annotations

import inspect
from functools import wraps

from ..protocol import DataProto, DataProtoFuture
from ..utils.py_utils import DynamicEnum
from ..utils.tensordict_lite import TensorDict
from ..utils.tensordict_lite import cat as _td_cat

MAGIC_ATTR = "_axon_register_info"


class Dispatch(DynamicEnum):
    _registry = {}
    _next_value = 0


class Execute(DynamicEnum):
    _registry = {}
    _next_value = 0


for _n in ("RANK_ZERO", "ONE_TO_ALL", "ALL_TO_ALL", "DP_COMPUTE_PROTO_WITH_FUNC", "DIRECT_SAMPLER_METHOD"):
    Dispatch.register(_n)
for _n in ("ALL", "RANK_ZERO"):
    Execute.register(_n)


def _chunk_item(item, chunks: int):
    if isinstance(item, TensorDict):
        parts = item.chunk(chunks)
    elif hasattr(item, "chunk"):
        parts = item.chunk(chunks=chunks)
    else:
        return [item] * chunks
    assert len(parts) == chunks, f"expected {chunks} chunks, got {len(parts)}"
    return parts


def dispatch(worker_group, *args, replicate: bool = True, split_first_arg: bool = False, rank_mapping=None, **kwargs):
    """Per-worker argument lists. ``rank_mapping[i]`` = data-parallel index of worker i."""
    ws = worker_group.world_size
    if rank_mapping is not None:
        dp = max(rank_mapping) + 1
        sa = [_chunk_item(a, dp) for a in args]
        sk = {k: _chunk_item(v, dp) for k, v in kwargs.items()}
        return (tuple([a[rank_mapping[i]] for i in range(ws)] for a in sa),
                {k: [v[rank_mapping[i]] for i in range(ws)] for k, v in sk.items()})
    if replicate:
        return tuple([a] * ws for a in args), {k: [v] * ws for k, v in kwargs.items()}
    if split_first_arg:
        return tuple(_chunk_item(a, ws) for a in args), {k: _chunk_item(v, ws) for k, v in kwargs.items()}
    return args, kwargs


def _concat_outputs(output: list):
    if not output:
        return output
    first = output[0]
    if isinstance(first, DataProto):
        return DataProto.concat(output)
    if isinstance(first, TensorDict):
        return _td_cat(output)
    if hasattr(first, "result") or isinstance(first, DataProtoFuture):
        return DataProtoFuture.concat(output)
    raise NotImplementedError(f"Cannot concat type {type(first)}")


def collect(worker_group, output, concat: bool = False, collect_mask=None):
    if collect_mask is not None:
        output = [o for o, keep in zip(output, collect_mask) if keep]
    return _concat_outputs(output) if concat else output


def _passthrough_dispatch(worker_group, *args, **kwargs):
    return args, kwargs


def _passthrough_collect(worker_group, output):
    return output


def _forbidden(*args, **kwargs):
    raise NotImplementedError("Direct sampler call is forbidden.")


def make_nd_compute_dataproto_dispatch_fn(mesh_name: str) -> dict:
    def dispatch_fn(worker_group, *args, **kwargs):
        if mesh_name not in worker_group._dispatch_info:
            info = worker_group._query_dispatch_info(mesh_name)
            assert len(info) == worker_group.world_size
            worker_group._dispatch_info[mesh_name] = info
        return dispatch(worker_group, *args, rank_mapping=worker_group._dispatch_info[mesh_name], **kwargs)

    def collect_fn(worker_group, output):
        if mesh_name not in worker_group._collect_info:
            info = worker_group._query_collect_info(mesh_name)
            assert len(info) == worker_group.world_size
            worker_group._collect_info[mesh_name] = info
        return collect(worker_group, output, collect_mask=worker_group._collect_info[mesh_name], concat=True)

    return {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn, "mesh_name": mesh_name}


def get_predefined_dispatch_fn(dispatch_mode) -> dict:
    table = {
        Dispatch.RANK_ZERO: (_passthrough_dispatch, _passthrough_collect),
        Dispatch.ONE_TO_ALL: (lambda wg, *a, **k: dispatch(wg, *a, replicate=True, **k),
                              lambda wg, out: collect(wg, out)),
        Dispatch.ALL_TO_ALL: (_passthrough_dispatch, lambda wg, out: collect(wg, out)),
        Dispatch.DP_COMPUTE_PROTO_WITH_FUNC: (lambda wg, *a, **k: dispatch(wg, *a, replicate=False, split_first_arg=True, **k),
                                              lambda wg, out: collect(wg, out, concat=True)),
        Dispatch.DIRECT_SAMPLER_METHOD: (_forbidden, _forbidden),
    }
    d, c = table[dispatch_mode]
    return {"dispatch_fn": d, "collect_fn": c}


def get_predefined_execute_fn(execute_mode) -> dict:
    return {Execute.ALL: {"execute_fn_name": "execute_all"},
            Execute.RANK_ZERO: {"execute_fn_name": "execute_rank_zero"}}[execute_mode]


def _materialize_futures(*args, **kwargs):
    conv = lambda v: v.get() if isinstance(v, DataProtoFuture) else v  # noqa: E731
    return tuple(conv(a) for a in args), {k: conv(v) for k, v in kwargs.items()}


def register(dispatch_mode=None, execute_mode=None, blocking: bool = True, materialize_futures: bool = True):
    """Attach dispatch metadata to a worker method. ``dispatch_mode`` is a ``Dispatch`` member or a dict
    with ``dispatch_fn`` / ``collect_fn`` (as produced by ``make_nd_compute_dataproto_dispatch_fn``)."""
    dispatch_mode = Dispatch.ALL_TO_ALL if dispatch_mode is None else dispatch_mode
    execute_mode = Execute.ALL if execute_mode is None else execute_mode
    if isinstance(dispatch_mode, dict):
        assert "dispatch_fn" in dispatch_mode and "collect_fn" in dispatch_mode
    elif not isinstance(dispatch_mode, Dispatch):
        raise ValueError(f"dispatch_mode must be Dispatch enum or dict, got {type(dispatch_mode)}")
    assert isinstance(execute_mode, Execute), f"execute_mode must be Execute. Got {execute_mode}"

    def decorator(func):
        if inspect.iscoroutinefunction(func):
            @wraps(func)
            async def wrapper(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                return await func(*args, **kwargs)
        else:
            @wraps(func)
            def wrapper(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                return func(*args, **kwargs)
        setattr(wrapper, MAGIC_ATTR, {"dispatch_mode": dispatch_mode, "execute_mode": execute_mode, "blocking": blocking})
        return wrapper
    return decorator
