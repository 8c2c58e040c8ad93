"""Sampler worker: one generation engine + server per GPU (reference: axon/sampler/sampler.py:35-164).

In the colocated ("hybrid") deployment the worker lives in the same process as the trainer role and
binds its engine to the trainer's flat parameter buffer, so a weight update needs no copy at all; in
the disaggregated deployment it owns its parameters and receives updates either as named tensors
(``update_weights``) or through the P2P push path. The server is reachable in-process (the object)
and, when ``serve_http`` is set, over an OpenAI-compatible HTTP endpoint.
"""
from __future__ import annotations

import datetime
import threading

import torch
import torch.distributed as dist

from ..controller.decorator import Dispatch, register
from ..core.worker import Worker
from ..utils.profiler import DistProfiler, DistProfilerExtension, ProfilerConfig
from .engine import GenerationEngine
from .server import SERVER_REGISTRY, SamplerMode, SamplerServer


def _get(cfg, key, default=None):
    cur = cfg
    for part in key.split("."):
        if isinstance(cur, dict) and part in cur:
            cur = cur[part]
        elif cur is not None and not isinstance(cur, dict) and hasattr(cur, part):
            cur = getattr(cur, part)
        else:
            return default
    return default if cur is None else cur


class SamplerWorker(Worker, DistProfilerExtension):
    def __init__(self, config, name: str = "sampler", **kwargs):
        Worker.__init__(self)
        self.config = config
        self.name = name
        scfg = _get(config, "sampler", config)
        self.scfg = scfg
        use_cuda = torch.cuda.is_available() and not _get(config, "force_cpu", False)
        if use_cuda:
            torch.cuda.set_device(self.local_rank % torch.cuda.device_count())
            self.device = torch.device("cuda", torch.cuda.current_device())
        else:
            self.device = torch.device("cpu")
        self.tp = int(_get(scfg, "tensor_model_parallel_size", 1))
        ep = int(_get(scfg, "expert_parallel_size", 1) or 1)
        if ep > 1 and self.tp == 1:
            # experts divided over a group of ranks: here that is the tensor-parallel group (which also divides the heads);
            # a layout with whole attention replicas around shared experts is not built
            self.tp = ep
        elif ep > 1 and ep != self.tp:
            raise NotImplementedError(f"sampler.expert_parallel_size ({ep}) must equal sampler.tensor_model_parallel_size ({self.tp}): "
                                      "a sampler group divides its experts over its own ranks")
        self.pp = int(_get(scfg, "pipeline_model_parallel_size", 1))
        assert self.world_size % (self.tp * self.pp) == 0
        self.dp_rank = self.rank // (self.tp * self.pp)
        self._register_dispatch_collect_info("sampler", dp_rank=self.dp_rank, is_collect=self.rank % (self.tp * self.pp) == 0)
        if self.world_size > 1 and self.tp * self.pp > 1 and not dist.is_initialized():
            dist.init_process_group(backend="nccl" if use_cuda else "gloo", rank=self.rank, world_size=self.world_size,
                                    init_method=f"tcp://{self._master_addr}:{self._master_port}",
                                    timeout=datetime.timedelta(seconds=600))
        DistProfilerExtension.__init__(self, DistProfiler(self.rank, ProfilerConfig.from_config(
            _get(scfg, "profiler", {}), _get(config, "global_profiler", None))))
        self.model = None
        self.engine: GenerationEngine | None = None
        self.server: SamplerServer | None = None
        self.tokenizer = None
        self._http_thread: threading.Thread | None = None
        self._http_server = None
        self.address: str | None = None
        self.shares_trainer_weights = False

    # ------------------------------------------------------------------ set-up
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        from ..utils.hf_model import build_model
        from ..utils.tokenizer import hf_tokenizer
        cfg, scfg = self.config, self.scfg
        peers = getattr(self, "_fused_peers", None) or {}
        trainer = next((p for r, p in peers.items() if r != self.name and getattr(p, "model", None) is not None
                        and hasattr(p, "engine") and not getattr(p, "_forward_only", False)), None)
        lockstep = None
        self.tp_group = None
        if self.tp * self.pp > 1:
            if self.pp > 1 and self.tp > 1:
                raise NotImplementedError("a sampler group is either tensor-parallel or cut into pipeline stages, not both")
            if self.pp > 1 and _get(cfg, "moe_replay", False):
                raise NotImplementedError("routed-experts capture is not gathered over the stages of a pipelined sampler group; "
                                          "use a tensor-parallel group with moe_replay")
            lockstep = self._make_tp_groups()
        shared = None
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        if trainer is not None and self.tp > 1:
            # colocated with a tensor- (and expert-) parallel trainer of the same group size: read its shards in place
            from ..models.tp_infer import Shard, share_trainer_shards
            shared = share_trainer_shards(trainer.model, Shard.create(self.tp_group, self.device))
        serves = trainer is not None and getattr(trainer.model, "serves_sampler", True) and hasattr(trainer.model, "prefill")
        if shared is not None:
            self.model = shared
            self.shares_trainer_weights = True
        elif trainer is not None and self.tp == 1 and self.pp == 1 and serves:
            self.model = trainer.model                  # zero-copy: generation reads the trainer's live parameters
            self.shares_trainer_weights = True
        elif trainer is not None:
            # the trainer's layout is not the sampler's (parameter shards, pipeline stages, another group size): this
            # sampler holds weights of its own - whole, or its part of a tensor-parallel group - and is refreshed from the
            # trainer's gathered tensors at every switch to rollout
            if self.tp > 1:
                from ..models.tp_infer import Shard, build_sharded_model
                self.model = build_sharded_model(_get(cfg, "model_path"), Shard.create(self.tp_group, self.device), device=self.device,
                                                 dtype=dtype, seed=int(_get(cfg, "seed", 42)), load_weights=False)
            elif self.pp > 1:
                from ..models.pp_infer import build_staged_model
                from ..models.tp_infer import Shard
                self.model = build_staged_model(_get(cfg, "model_path"), Shard.create(self.tp_group, self.device, reduce=False), device=self.device,
                                                dtype=dtype, seed=int(_get(cfg, "seed", 42)), load_weights=False)
            else:
                self.model = build_model(_get(cfg, "model_path"), device=self.device, dtype=dtype, seed=int(_get(cfg, "seed", 42)),
                                         load_weights=False)
        elif self.tp > 1:
            from ..models.tp_infer import Shard, build_sharded_model
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.model = build_sharded_model(_get(cfg, "model_path"), Shard.create(self.tp_group, self.device), device=self.device,
                                             dtype=dtype, seed=int(_get(cfg, "seed", 42)), load_weights=True)
        elif self.pp > 1:
            from ..models.pp_infer import build_staged_model
            from ..models.tp_infer import Shard
            self.model = build_staged_model(_get(cfg, "model_path"), Shard.create(self.tp_group, self.device, reduce=False), device=self.device,
                                            dtype=dtype, seed=int(_get(cfg, "seed", 42)), load_weights=True)
        else:
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.model = build_model(_get(cfg, "model_path"), device=self.device, dtype=dtype, seed=int(_get(cfg, "seed", 42)),
                                     load_weights=True)
        try:
            self.tokenizer = hf_tokenizer(_get(cfg, "model_path"))
        except Exception:
            self.tokenizer = None
        kv_bytes = None
        if self.device.type == "cuda":
            free, total = torch.cuda.mem_get_info()
            util = float(_get(scfg, "gpu_memory_utilization", 0.85))
            kv_bytes = max(1 << 28, int(free - (1.0 - util) * total))
            if self.shares_trainer_weights:
                kv_bytes = self._kv_bytes_beside_optimizer(trainer, kv_bytes)
        num_pages = _get(scfg, "num_kv_pages", None)
        if lockstep is not None and num_pages is None:
            # the engines of a group must make the same scheduling decisions: they take the smallest pool any rank can hold
            from .kv_cache import PagedKVCache
            fit = (kv_bytes if kv_bytes is not None else 4 << 30) // PagedKVCache.bytes_per_page(self.model.cfg, self.model.params.flat.element_size())
            agreed = torch.tensor([max(8, int(fit))], dtype=torch.int64)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=lockstep.group)
            num_pages = int(agreed.item())
        self.engine = GenerationEngine(self.model, num_pages=num_pages, max_num_seqs=int(_get(scfg, "max_num_seqs", 256)),
                                       max_num_batched_tokens=int(_get(scfg, "max_num_batched_tokens", 32768)),
                                       kv_memory_bytes=kv_bytes, seed=int(_get(cfg, "seed", 42)) + self.dp_rank)
        if _get(scfg, "enforce_eager", False):
            self.engine.use_cuda_graph = False
        self.engine.logprobs_mode = str(_get(scfg, "logprobs_mode", "processed"))
        self.engine.enable_prefix_caching = bool(_get(scfg, "enable_prefix_caching", False))
        self.engine.enable_chunked_prefill = bool(_get(scfg, "enable_chunked_prefill", True))
        spec = _get(scfg, "speculative_config", None) or {}
        spec = spec.to_dict() if hasattr(spec, "to_dict") else dict(spec)
        if spec:
            method = str(spec.get("method", "ngram"))
            if method != "ngram":
                raise ValueError(f"speculative_config.method={method!r}: only 'ngram' (prompt lookup) drafts are built")
            self.engine.speculative_ngram = int(spec.get("num_speculative_tokens", 4))
            self.engine.speculative_ngram_match = int(spec.get("prompt_lookup_max", 3))
        if _get(cfg, "moe_replay", False) and getattr(self.model.cfg, "num_experts", 0) > 0:
            self.engine.enable_routing_capture(True)      # outputs carry the routed experts for the trainer to replay
        max_len = _get(scfg, "max_model_len", None)
        if max_len:
            self.engine.set_max_model_len(int(max_len))
        mode = SamplerMode.HYBRID if self.shares_trainer_weights else SamplerMode.STANDALONE
        server_cls = SERVER_REGISTRY.get(str(_get(scfg, "name", "native")), SamplerServer)
        self.server = server_cls(self.engine, tokenizer=self.tokenizer, name=f"{self.name}-{self.rank}", mode=mode,
                                 lockstep=lockstep).start()
        if _get(scfg, "serve_http", False) and (lockstep is None or lockstep.leader):
            self._start_http()                          # a group is reached through its first rank
        if self.shares_trainer_weights and _get(scfg, "offload_sampler", True):
            self.server.sleep()                          # training starts with the KV pool released
        return {"address": self.address, "shares_trainer_weights": self.shares_trainer_weights,
                "kv_pages": self.engine._num_pages}

    def _make_tp_groups(self):
        """Process groups of this rank's tensor-parallel group: one for the activations (NCCL on GPUs) and a CPU one
        for the lockstep control messages. Every rank creates every group, in the same order."""
        from .server import Lockstep
        assert dist.is_initialized(), "a tensor-parallel sampler needs the worker group's process group"
        mine_data = mine_ctl = None
        size = self.tp * self.pp              # one of the two is 1
        for g in range(self.world_size // size):
            ranks = list(range(g * size, (g + 1) * size))
            data = dist.new_group(ranks)
            ctl = dist.new_group(ranks, backend="gloo", timeout=datetime.timedelta(hours=6))
            if g == self.dp_rank:
                mine_data, mine_ctl = data, ctl
        self.tp_group = mine_data
        return Lockstep(mine_ctl)

    def _start_http(self) -> None:
        import socket
        import time

        import uvicorn
        # the listening socket is opened HERE and handed to the server: a port that was only probed could be taken by
        # another worker process before the server binds it
        sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
        cfg = uvicorn.Config(self.server.build_app(), host="127.0.0.1", port=port, log_level="warning")
        self._http_server = uvicorn.Server(cfg)
        self._http_thread = threading.Thread(target=self._http_server.run, kwargs={"sockets": [sock]}, daemon=True, name="sampler-http")
        self._http_thread.start()
        deadline = time.monotonic() + 30.0
        while not self._http_server.started and self._http_thread.is_alive() and time.monotonic() < deadline:
            time.sleep(0.01)
        if not self._http_server.started:
            raise RuntimeError("the sampler's HTTP server did not start")
        self.address = f"http://127.0.0.1:{port}"

    def _kv_bytes_beside_optimizer(self, trainer, kv_bytes: int) -> int:
        """Colocated mode: the trainer's optimizer state (12 bytes per parameter of its shard, allocated at its first
        step) can stay on the device during rollout if the KV pool leaves room for it. When the pool that remains
        still covers the expected demand - ``kv_expected_fill`` (0.4) of the worst case of every sequence at full
        length at once - take the smaller pool; a pool that turns out too small only costs preemptions. Otherwise keep
        the large pool and let the optimizer state move to the host around every rollout."""
        from .kv_cache import PagedKVCache
        cfg, scfg = self.config, self.scfg
        eng = getattr(trainer, "engine", None)
        if eng is None or getattr(trainer, "_forward_only", False) or getattr(eng, "master", None) is not None:
            return kv_bytes                      # no optimizer, or its state is already counted in the free memory
        opt_bytes = 12 * int(self.model.params.numel) // max(1, int(getattr(eng, "opt_world", 1)))
        fill = _get(scfg, "kv_expected_fill", 0.4)
        if fill is None:
            return kv_bytes
        seq_len = int(_get(scfg, "max_model_len", None) or _get(cfg, "max_seq_length", 0) or 0)
        if seq_len <= 0:
            return kv_bytes
        per_token = PagedKVCache.bytes_per_page(self.model.cfg, self.model.params.flat.element_size()) / 128
        want = float(fill) * int(_get(scfg, "max_num_seqs", 256)) * seq_len * per_token
        fit = kv_bytes - opt_bytes
        return int(fit) if fit >= max(want, 4 << 30) else kv_bytes

    # ------------------------------------------------------------------ direct methods
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_server_address(self):
        """HTTP address when serving over HTTP, else None (callers in the same process use ``get_server``)."""
        return self.address

    get_zeromq_address = get_server_address      # name used by the reference's executor-facing API

    def get_server(self) -> SamplerServer:
        return self.server

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def wake_up(self):
        self.server.wake_up()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def sleep(self):
        self.server.sleep()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def pause_generation(self, strategy: str = "drain"):
        self.server.pause_generation(strategy)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def continue_generation(self):
        self.server.continue_generation()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def update_weights(self, named_tensors=None):
        """Hybrid deployment: nothing to move (shared buffer) — only cached state that depends on the
        old weights is dropped. Otherwise copy the given (name, tensor) pairs in."""
        self.server.reset_prefix_cache()              # cached keys / values were computed with the old weights
        if self.shares_trainer_weights or named_tensors is None:
            return 0
        return self.server.update_weights(named_tensors)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def param_sums(self) -> dict:
        """name -> (fp64 sum, shape, position-weighted fp64 sum) of every parameter tensor this rank holds (weight-sync
        checks compare them; the weighted sum also notices rows that arrived in the wrong place)."""
        from ..utils.state.utils import tensor_digest
        return {n: tensor_digest(v) for n, v in self.model.params.views.items()}

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def params_checksum(self) -> float:
        return float(self.model.params.flat.double().sum().item())

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def engine_stats(self) -> dict:
        return dict(self.engine.stats)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def shutdown(self):
        if self._http_server is not None:
            self._http_server.should_exit = True
        if self.server is not None:
            self.server.stop()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_profile(self, **kw):
        DistProfilerExtension.start_profile(self, role=self.name, **kw)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def stop_profile(self):
        DistProfilerExtension.stop_profile(self)
