"""Colocated roles: one worker process hosts several role objects (actor + sampler (+ ref / critic)).

``fuse_worker_cls(class_dict)`` builds a class whose instances create one inner object per role and
expose every registered method of role ``r`` as ``{r}_{method}`` — except methods registered with
``Dispatch.DIRECT_SAMPLER_METHOD``, which keep their own name so colocated workers can call each
other directly. ``RoleProxy`` gives the controller a per-role view with the original method names
and role-scoped mesh dispatch (reference: axon/controller/ray/fused_worker_group.py:31-261).
"""
from __future__ import annotations

from .decorator import MAGIC_ATTR, Dispatch, get_predefined_dispatch_fn, get_predefined_execute_fn, register
from .worker_group import ClassWithInitArgs, func_generator


def _registered_methods(cls):
    for name in dir(cls):
        try:
            m = getattr(cls, name)
        except Exception:  # noqa: BLE001
            continue
        info = getattr(m, MAGIC_ATTR, None)
        if callable(m) and info is not None:
            yield name, m, info


def fuse_worker_cls(class_dict: dict[str, ClassWithInitArgs]) -> ClassWithInitArgs:
    roles = list(class_dict)

    class FusedWorker:
        _role_classes = {r: class_dict[r].cls for r in roles}
        _fused_spec = class_dict          # how a worker process assembles this class again (``ClassWithInitArgs``)

        def __init__(self):
            self.role_objects = {r: class_dict[r]() for r in roles}
            for r, obj in self.role_objects.items():
                setattr(obj, "_fused_peers", self.role_objects)    # colocated roles reach each other directly

        @register(dispatch_mode=Dispatch.ONE_TO_ALL)
        def _query_dispatch_info(self, mesh_name: str):
            role, mesh = mesh_name.split("/", 1)
            return self.role_objects[role]._query_dispatch_info(mesh)

        @register(dispatch_mode=Dispatch.ONE_TO_ALL)
        def _query_collect_info(self, mesh_name: str):
            role, mesh = mesh_name.split("/", 1)
            return self.role_objects[role]._query_collect_info(mesh)

    def make_forward(role, name, info):
        def fwd(self, *args, **kwargs):
            return getattr(self.role_objects[role], name)(*args, **kwargs)
        fwd.__name__ = name
        setattr(fwd, MAGIC_ATTR, dict(info))
        return fwd

    for role in roles:
        for name, _, info in _registered_methods(class_dict[role].cls):
            if name in ("_query_dispatch_info", "_query_collect_info"):
                continue
            direct = info["dispatch_mode"] is Dispatch.DIRECT_SAMPLER_METHOD
            setattr(FusedWorker, name if direct else f"{role}_{name}", make_forward(role, name, info))
    FusedWorker.__name__ = "Fused_" + "_".join(roles)
    return ClassWithInitArgs(FusedWorker)


class RoleProxy:
    """Controller-side view of ONE role of a fused worker group."""

    def __init__(self, worker_group, role: str, role_cls):
        self._wg, self._role, self._cls = worker_group, role, role_cls
        self._dispatch_info: dict = {}
        self._collect_info: dict = {}
        for name, _, info in _registered_methods(role_cls):
            if name in ("_query_dispatch_info", "_query_collect_info"):
                continue
            mode = info["dispatch_mode"]
            if mode is Dispatch.DIRECT_SAMPLER_METHOD:
                continue
            fns = mode if isinstance(mode, dict) else get_predefined_dispatch_fn(mode)
            execute_fn = getattr(worker_group, get_predefined_execute_fn(info["execute_mode"])["execute_fn_name"])
            setattr(self, name, func_generator(self, f"{role}_{name}", fns["dispatch_fn"], fns["collect_fn"],
                                               execute_fn, info["blocking"]))

    @property
    def world_size(self) -> int:
        return self._wg.world_size

    @property
    def rpc_timeout(self):
        return self._wg.rpc_timeout

    @property
    def workers(self):
        return self._wg.workers

    def _query_dispatch_info(self, mesh_name: str):
        return self._wg._query_dispatch_info(f"{self._role}/{mesh_name}")

    def _query_collect_info(self, mesh_name: str):
        return self._wg._query_collect_info(f"{self._role}/{mesh_name}")

    def execute_all(self, method_name: str, *args, **kwargs):
        return self._wg.execute_all(method_name, *args, **kwargs)

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        return self._wg.execute_rank_zero(method_name, *args, **kwargs)

    def shutdown(self) -> None:
        self._wg.shutdown()
