"""Model-parallel trainer worker (the reference's Megatron personality:
axon/trainer/megatron_trainer.py:120-932, model functions axon/models/megatron_models.py).

World layout: ``world = dp x tp`` with tensor-parallel groups of consecutive ranks (one NVLink domain)
and data-parallel groups strided across them, as ``mpu.initialize_model_parallel`` lays them out.
Tensor parallelism uses sequence-parallel activations with the fused all-gather->GEMM and
GEMM->reduce-scatter kernels (``parallel/tp.py``); the optimizer is the sharded (distributed)
AdamW of the policy engine over the data-parallel group. Data is dispatched per data-parallel rank
and collected from tensor-parallel rank 0.

Expert parallelism (``expert_model_parallel_size``, with tp = 1): ``world = edp x ep``; expert-parallel
groups are consecutive ranks, every rank is a data-parallel rank of its own (different rows), tokens
reach their experts through peer memory (``parallel/ep.py``). Non-expert gradients are summed over the
expert-parallel group and then reduced with the expert gradients over the strided "expert data
parallel" group, which is also the group the optimizer state is sharded over.

Pipeline parallelism (``pipeline_model_parallel_size``, alone): stage groups of consecutive ranks,
``models/pp_dense.py`` (send / recv between stages, micro-batches one after another).

Tensor x pipeline (``world = dp x pp x tp``): ``models/tp_pp_dense.py`` - tensor-parallel shards inside pipeline
stages, the sequence-parallel local stream travels between stages. Other combinations of two model-parallel
dimensions (with expert or context parallelism) are refused with an explicit error.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .fsdp_trainer import CausalLM, RewardModel, TrainerWorker as _Base, ValueModel, _get  # noqa: F401


class TrainerWorker(_Base):
    def __init__(self, config, model=None, name: str = "trainer", **kwargs):
        m = _get(config, "megatron", {}) or {}
        self.tp_size = int(_get(m, "tensor_model_parallel_size", 1) or 1)
        self.ep_size = int(_get(m, "expert_model_parallel_size", 1) or 1)
        self.etp_size = int(_get(m, "expert_tensor_parallel_size", 1) or 1)
        if self.etp_size > 1 and (self.etp_size != self.tp_size or self.ep_size > 1):
            raise NotImplementedError("expert tensor parallelism divides every expert over the tensor-parallel group: set "
                                      "expert_tensor_parallel_size == tensor_model_parallel_size with expert_model_parallel_size = 1 "
                                      f"(got etp={self.etp_size}, tp={self.tp_size}, ep={self.ep_size})")
        if self.ep_size > 1 and self.tp_size > 1 and self.ep_size != self.tp_size:
            raise NotImplementedError("tensor and expert parallelism together divide the experts over the tensor-parallel group's own "
                                      f"ranks: set expert_model_parallel_size == tensor_model_parallel_size (got ep={self.ep_size}, tp={self.tp_size})")
        self.pp_size = int(_get(m, "pipeline_model_parallel_size", 1) or 1)
        self.vpp_size = int(_get(m, "virtual_pipeline_model_parallel_size", 1) or 1)
        if self.vpp_size > 1 and self.pp_size < 2:
            raise NotImplementedError("virtual pipeline stages interleave the chunks of a pipeline: pipeline_model_parallel_size >= 2")
        if self.pp_size > 1 and self.ep_size > 1 and self.tp_size != self.ep_size:
            raise NotImplementedError("pipeline stages of a sparse model divide their experts over the stage's tensor-parallel "
                                      "group: set expert_model_parallel_size == tensor_model_parallel_size > 1")
        self.cp_size = int(_get(m, "context_parallel_size", 1) or 1)
        if self.cp_size > 1 and (self.ep_size > 1 or self.pp_size > 1):
            raise NotImplementedError("context parallelism combines with tensor parallelism (world = dp x cp x tp); together with "
                                      "expert or pipeline parallelism it is not available in this trainer")
        self._pending_dispatch = True
        super().__init__(config, model=model, name=name, **kwargs)
        # ranks that work on the same rows (expert-parallel ranks do not): the asynchronous driver hands one shard of a batch to each such block
        self.rows_group_size = self.tp_size * self.pp_size * self.cp_size
        if self.cp_size > 1:
            assert self.ulysses_sequence_parallel_size == 1, "choose one of Ulysses and context parallelism"
            self.ulysses_sequence_parallel_size = self.cp_size      # the token caps count per group, as with Ulysses
            self.rows_group_size = self.tp_size * self.pp_size      # ... and the row shards per (context-parallel x this) block

    # the base class registers dp_rank = rank // sp; with TP the data shard is rank // tp
    def _register_dispatch_collect_info(self, mesh_name: str, dp_rank: int, is_collect: bool) -> None:
        if mesh_name == "trainer" and getattr(self, "_pending_dispatch", False):
            self._pending_dispatch = False
            # ranks of one tensor- / pipeline- / context-parallel group (or tensor x pipeline block) see the same rows
            mp = self.tp_size * self.pp_size if (self.tp_size > 1 and self.pp_size > 1) else max(self.tp_size, self.pp_size, self.cp_size)
            if self.tp_size > 1 and self.cp_size > 1:
                mp = self.tp_size * self.cp_size          # a context-parallel rank is a whole tensor-parallel group
            assert self.world_size % mp == 0, f"world size {self.world_size} not divisible by the model-parallel size {mp}"
            return super()._register_dispatch_collect_info(mesh_name, self.rank // mp, self.rank % mp == 0)
        return super()._register_dispatch_collect_info(mesh_name, dp_rank, is_collect)

    def _make_groups(self, tp: int | None = None):
        """(model-parallel group of ``tp`` consecutive ranks, strided data-parallel group) of this rank;
        every rank creates every group (collective contract)."""
        tp, world = tp or self.tp_size, self.world_size
        tp_group = dp_group = None
        if world == 1:
            return None, None
        for i in range(world // tp):
            ranks = list(range(i * tp, (i + 1) * tp))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                tp_group = g
        for j in range(tp):
            ranks = list(range(j, world, tp))
            g = dist.new_group(ranks)          # also for a single rank: the optimizer needs a group of its own
            if self.rank in ranks:
                dp_group = g
        return tp_group, dp_group

    def _build_pipeline_parallel(self, model_path, dtype, seed):
        import os
        from ..models.config import get_config
        from ..models.params import FlatParams
        from ..models.pp_dense import PipelineContext, PPDenseModel
        from ..utils.hf_model import has_hf_weights, iter_hf_weights
        mcfg = get_config(model_path)
        assert self.world_size % self.pp_size == 0, f"world size {self.world_size} not divisible by pp {self.pp_size}"
        assert not self.model_kind.value_head, "value-head models are not pipeline-parallel yet; run the critic with pp=1"
        pp_group, dp_group = self._make_groups(self.pp_size)
        self.pg, self._mp_group = dp_group, pp_group
        ends_group = None
        if (mcfg.tie_word_embeddings or mcfg.num_nextn_predict_layers > 0) and self.pp_size > 2:      # first and last stage of every pipeline share the embedding
            for i in range(self.world_size // self.pp_size):
                ranks = [i * self.pp_size, (i + 1) * self.pp_size - 1]
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    ends_group = g
        model = PPDenseModel(mcfg, PipelineContext(pp_group, self.device, ends_group), device=self.device, dtype=dtype,
                             virtual=self.vpp_size)
        ref = FlatParams(mcfg, "cpu", dtype)                 # full model on the host, cut down to this stage
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            ref.load_hf_state_dict(dict(iter_hf_weights(model_path)))
        else:
            ref.init_random(seed=seed)
        model.load_full_state(ref.views)
        model.recompute = str(_get(self.config, "recompute", "selective"))
        return model

    def _make_state_manager(self):
        both = self.tp_size > 1 and self.pp_size > 1
        mp = self.tp_size * self.pp_size if both else max(self.tp_size, self.ep_size, self.pp_size)
        if mp == 1:
            return super()._make_state_manager()
        from ..utils.state.megatron_state_manager import MegatronStateManager
        return MegatronStateManager(self.model, self.engine, mp_group=getattr(self, "_mp_group", None), tp=self.tp_size, ep=self.ep_size,
                                    etp=self.etp_size, pp=self.pp_size, dp_rank=self.rank // mp, tp_rank=(self.rank % self.tp_size) if both else None,
                                    processing_class=self.tokenizer, rank=self.rank, world_size=self.world_size, process_group=self.pg)

    def _build_tensor_pipeline_parallel(self, model_path, dtype, seed):
        """world = dp x pp x tp: tensor-parallel groups are consecutive ranks, the stages of one replica are tp ranks
        apart, replicas are pp x tp ranks apart (the order megatron's ``initialize_model_parallel`` uses)."""
        import os
        from ..models.config import get_config
        from ..models.params import FlatParams
        from ..models.pp_dense import PipelineContext
        from ..models.tp_pp_dense import TPPPDenseModel, TPPPMoEModel
        from ..parallel.tp import TPContext
        from ..utils.hf_model import has_hf_weights, iter_hf_weights
        mcfg = get_config(model_path)
        tp, pp, world = self.tp_size, self.pp_size, self.world_size
        block = tp * pp
        assert world % block == 0, f"world size {world} not divisible by tp x pp = {block}"
        assert not self.model_kind.value_head, "value-head models are not model-parallel yet; run the critic with tp = pp = 1"

        def make(groups):
            mine = None
            for ranks in groups:
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    mine = g
            return mine
        n_rep = world // block
        tp_group = make([list(range(b * block + s * tp, b * block + (s + 1) * tp)) for b in range(n_rep) for s in range(pp)])
        pp_group = make([[b * block + s * tp + t for s in range(pp)] for b in range(n_rep) for t in range(tp)])
        dp_group = make([[b * block + j for b in range(n_rep)] for j in range(block)])
        block_group = make([list(range(b * block, (b + 1) * block)) for b in range(n_rep)])
        ends_group = None
        if (mcfg.tie_word_embeddings or mcfg.num_nextn_predict_layers > 0) and pp > 2:
            ends_group = make([[b * block + t, b * block + (pp - 1) * tp + t] for b in range(n_rep) for t in range(tp)])
        self.pg, self._mp_group = dp_group, block_group
        rows = int(_get(self.config, "max_token_len_per_gpu", 16384))
        rows = (rows // tp + 127) // 128 * 128 + 128
        sparse = mcfg.num_experts > 0
        assert sparse == (self.ep_size > 1 or self.etp_size > 1), \
            "expert_model_parallel_size / expert_tensor_parallel_size go with a mixture-of-experts model (and only with one)"
        width = max(mcfg.qkv_size, mcfg.hidden_size) if sparse else max(mcfg.qkv_size, 2 * mcfg.intermediate_size, mcfg.hidden_size)
        ctx = TPContext(tp_group, self.device, max_rows_per_rank=rows, max_width=width)
        stage_ctx = PipelineContext(pp_group, self.device, ends_group=ends_group)
        if sparse:
            ep = None                 # expert TENSOR parallelism: a slice of every expert per rank of the stage
            if self.ep_size > 1:
                from ..parallel.ep import EPContext
                ep = EPContext(tp_group, self.device, mcfg.num_experts, mcfg.hidden_size, mcfg.moe_intermediate_size, max_tokens=rows,
                               top_k=mcfg.num_experts_per_tok)
            model = TPPPMoEModel(mcfg, ctx, ep, stage_ctx, block_group, device=self.device, dtype=dtype, virtual=self.vpp_size)
        else:
            model = TPPPDenseModel(mcfg, ctx, stage_ctx, block_group, device=self.device, dtype=dtype, virtual=self.vpp_size)
        ref = FlatParams(mcfg, "cpu", dtype)
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            ref.load_hf_state_dict(dict(iter_hf_weights(model_path)))
        else:
            ref.init_random(seed=seed)
        model.load_full_state(ref.views)
        model.recompute = str(_get(self.config, "recompute", "selective"))
        return model

    def _build_expert_parallel(self, model_path, dtype, seed):
        import os
        from ..models.config import get_config
        from ..models.moe import MoEModel
        from ..parallel.ep import EPContext
        from ..utils.hf_model import has_hf_weights, iter_hf_weights
        mcfg = get_config(model_path)
        assert mcfg.num_experts > 0, f"expert_model_parallel_size={self.ep_size} needs a mixture-of-experts model"
        assert self.world_size % self.ep_size == 0, f"world size {self.world_size} not divisible by ep {self.ep_size}"
        ep_group, edp_group = self._make_groups(self.ep_size)
        self.pg = edp_group
        self._mp_group = ep_group
        cap = int(_get(self.config, "max_token_len_per_gpu", 16384))
        ctx = EPContext(ep_group, self.device, mcfg.num_experts, mcfg.hidden_size, mcfg.moe_intermediate_size,
                        max_tokens=(cap + 127) // 128 * 128, top_k=mcfg.num_experts_per_tok)
        model = MoEModel(mcfg, device=self.device, dtype=dtype, ep=ctx)
        from ..models.params import FlatParams
        ref = FlatParams(mcfg, "cpu", dtype)                 # full model on the host, cut down to this rank's experts
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            ref.load_hf_state_dict(dict(iter_hf_weights(model_path)))
        else:
            ref.init_random(seed=seed)
        model.load_full_state(ref.views)
        model.recompute = str(_get(self.config, "recompute", "selective"))
        return model

    def _build_tensor_expert_parallel(self, model_path, dtype, seed):
        """tp == ep: consecutive ranks form one group that divides the attention heads (sequence-parallel activations)
        AND the experts; the ranks of a group see the same rows, groups are data-parallel replicas."""
        import os
        from ..models.config import get_config
        from ..models.params import FlatParams
        from ..models.tp_dense import TPModelAdapter
        from ..models.tp_moe import TPMoEModel
        from ..parallel.ep import EPContext
        from ..parallel.tp import TPContext
        from ..utils.hf_model import has_hf_weights, iter_hf_weights
        if self.model_kind.value_head:
            raise NotImplementedError("value-head models are not tensor-parallel yet; run the critic with tp=1")
        mcfg = get_config(model_path)
        assert mcfg.num_experts > 0, "expert_model_parallel_size / expert_tensor_parallel_size need a mixture-of-experts model"
        tp_group, dp_group = self._make_groups()
        self.pg = dp_group
        self._mp_group = tp_group
        rows = int(_get(self.config, "max_token_len_per_gpu", 16384))
        rows = (rows // self.tp_size + 127) // 128 * 128 + 128
        tp = TPContext(tp_group, self.device, max_rows_per_rank=rows, max_width=max(mcfg.qkv_size, mcfg.hidden_size))
        ep = None                     # expert TENSOR parallelism: a slice of every expert per rank, no token exchange
        if self.ep_size > 1:
            ep = EPContext(tp_group, self.device, mcfg.num_experts, mcfg.hidden_size, mcfg.moe_intermediate_size, max_tokens=rows,
                           top_k=mcfg.num_experts_per_tok)
        inner = TPMoEModel(mcfg, tp, ep, device=self.device, dtype=dtype)
        ref = FlatParams(mcfg, "cpu", dtype)                 # full model on the host, cut down to this rank's part
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            ref.load_hf_state_dict(dict(iter_hf_weights(model_path)))
        else:
            ref.init_random(seed=seed)
        inner.load_full_state(ref.views)
        return TPModelAdapter(inner)

    def _build_context_parallel(self, model_path, dtype, seed):
        """Consecutive ranks form a context-parallel group (same rows, two zigzag chunks of every sequence
        each); the optimizer keeps sharding over ALL ranks, so its reduce-scatter also completes the
        partial weight gradients of the group."""
        from ..models.config import get_config
        from ..models.cp import CPDenseModel, CPModelAdapter
        from ..parallel.cp import ContextParallel
        from ..utils.hf_model import has_hf_weights, load_hf_weights
        import os
        mcfg = get_config(model_path)
        assert mcfg.num_experts == 0 and not self.model_kind.value_head, "context parallelism is available on dense causal-LM models"
        assert self.world_size % self.cp_size == 0, f"world size {self.world_size} not divisible by cp {self.cp_size}"
        cp_group = None
        for i in range(self.world_size // self.cp_size):
            ranks = list(range(i * self.cp_size, (i + 1) * self.cp_size))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                cp_group = g
        cap = int(_get(self.config, "max_token_len_per_gpu", 16384))       # per-rank token cap; the group packs cp times that
        # per-sequence padding adds at most 2 cp - 1 tokens per sequence; leave room for a few hundred sequences
        ctx = ContextParallel(cp_group, self.device, max_local_tokens=(cap + 127) // 128 * 128 + 1024, kv_width=2 * mcfg.kv_size)
        inner = CPDenseModel(mcfg, ctx, device=self.device, dtype=dtype)
        inner.recompute = str(_get(self.config, "recompute", "selective"))
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            load_hf_weights(inner, model_path)
        else:
            inner.params.init_random(seed=seed)
        return CPModelAdapter(inner)

    def _build_tensor_context_parallel(self, model_path, dtype, seed):
        """world = dp x cp x tp, tensor-parallel ranks consecutive: the members with the same place in their tensor-parallel
        group form the context-parallel groups (and, over all replicas, the optimizer's group)."""
        import os
        from ..models.config import get_config
        from ..models.cp import CPModelAdapter
        from ..models.params import FlatParams
        from ..models.tp_cp_dense import TPCPDenseModel
        from ..models.tp_dense import TPModelAdapter
        from ..parallel.cp import ContextParallel
        from ..parallel.tp import TPContext
        from ..utils.hf_model import has_hf_weights, iter_hf_weights
        mcfg = get_config(model_path)
        tp, cp, world = self.tp_size, self.cp_size, self.world_size
        assert mcfg.num_experts == 0 and not self.model_kind.value_head, "tensor x context parallelism is available on dense causal-LM models"
        assert world % (tp * cp) == 0, f"world size {world} not divisible by cp x tp = {cp * tp}"
        tp_group, dp_group = self._make_groups()
        cp_group = None
        for b in range(world // (tp * cp)):
            for t in range(tp):
                ranks = [b * tp * cp + c * tp + t for c in range(cp)]
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    cp_group = g
        self.pg, self._mp_group = dp_group, tp_group
        cap = int(_get(self.config, "max_token_len_per_gpu", 16384))
        local = (cap + 127) // 128 * 128 + 1024 + 128 * tp           # the rank's tokens: padding per sequence and to 128 tp
        rows = (local // tp + 127) // 128 * 128 + 128
        ctx = TPContext(tp_group, self.device, max_rows_per_rank=rows, max_width=max(mcfg.qkv_size, 2 * mcfg.intermediate_size, mcfg.hidden_size))
        ring = ContextParallel(cp_group, self.device, max_local_tokens=local, kv_width=2 * mcfg.kv_size // tp)
        inner = TPCPDenseModel(mcfg, ctx, ring, device=self.device, dtype=dtype)
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            ref = FlatParams(mcfg, "cpu", dtype)
            ref.load_hf_state_dict(dict(iter_hf_weights(model_path)))
            inner.load_full_state(ref.views)
        else:
            inner.init_random(seed=seed)
        mid = TPModelAdapter(inner)
        mid.cp = ring
        return CPModelAdapter(mid, token_multiple=128 * tp)

    def _build(self, model_path, dtype, seed):
        if self.cp_size > 1 and self.tp_size > 1:
            return self._build_tensor_context_parallel(model_path, dtype, seed)
        if self.cp_size > 1:
            return self._build_context_parallel(model_path, dtype, seed)
        if self.pp_size > 1 and self.tp_size > 1:
            return self._build_tensor_pipeline_parallel(model_path, dtype, seed)
        if self.pp_size > 1:
            return self._build_pipeline_parallel(model_path, dtype, seed)
        if (self.ep_size > 1 or self.etp_size > 1) and self.tp_size > 1 and self.pp_size == 1:
            return self._build_tensor_expert_parallel(model_path, dtype, seed)
        if self.ep_size > 1:
            return self._build_expert_parallel(model_path, dtype, seed)
        if self.tp_size == 1:
            return super()._build(model_path, dtype, seed)
        from ..models.config import get_config
        from ..models.tp_dense import TPDenseModel, TPModelAdapter
        from ..parallel.tp import TPContext
        mcfg = get_config(model_path)
        if self.model_kind.value_head:           # critic / reward model: a scalar head, whole on every rank
            mcfg.extra = {**mcfg.extra, "value_head": True}
        tp_group, dp_group = self._make_groups()
        self.pg = dp_group                          # the optimizer shards over the data-parallel group
        self._mp_group = tp_group
        rows = int(_get(self.config, "max_token_len_per_gpu", 16384))
        rows = (rows // self.tp_size + 127) // 128 * 128 + 128
        width = max(mcfg.qkv_size, 2 * mcfg.intermediate_size, mcfg.hidden_size) // 1
        ctx = TPContext(tp_group, self.device, max_rows_per_rank=rows, max_width=width)
        inner = TPDenseModel(mcfg, ctx, device=self.device, dtype=dtype)
        import os
        from ..utils.hf_model import has_hf_weights, iter_hf_weights
        if os.path.isdir(str(model_path)) and has_hf_weights(model_path):
            from ..models.params import FlatParams
            ref = FlatParams(mcfg, "cpu", dtype)
            ref.load_hf_state_dict(dict(iter_hf_weights(model_path)), strict=not self.model_kind.value_head)
            if self.model_kind.value_head:           # the checkpoint of a language model has no value head: the same draw on every rank
                torch.nn.init.normal_(ref["v_head.weight"], std=0.02, generator=torch.Generator().manual_seed(seed))
            inner.load_full_state(ref.views)
        else:
            inner.init_random(seed=seed)
        return TPModelAdapter(inner)
