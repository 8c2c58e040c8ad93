#!/usr/bin/env bash
# Math RL, Qwen3-235B-A22B (sparse, 94 layers, 128 experts), colocated on eight 8-GPU nodes with the model-parallel trainer:
# pipeline 16 x (tensor = expert parallel 4) - a pipeline stage fills half a node, so its fused tensor- and expert-parallel
# kernels stay on NVLink while the stage boundaries cross nodes. 180 GB per GPU hold a sampler copy in groups of 8 ranks
# (one node each; key / value heads are replicated where the group is larger than their number), refreshed from the
# trainer's gathered tensors before every rollout; the experts the sampler routed to are replayed in training.
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
[ -f "${ROOT}/data/math/train.parquet" ] || python "${ROOT}/recipes/math/data.py" --out "${ROOT}/data/math/train.parquet"
[ -f "${ROOT}/data/math/test.parquet" ] || python "${ROOT}/recipes/math/data.py" --split test --synthetic_size 64 --out "${ROOT}/data/math/test.parquet"
axon train --fg -- \
    strategy=megatron advantage=loop train_files="${ROOT}/data/math/train.parquet" val_files="${ROOT}/data/math/test.parquet" \
    train_batch_size=64 mini_batch_size=64 max_prompt_length=2048 max_seq_length=16384 model_path=Qwen/Qwen3-235B-A22B \
    hybrid_engine=true moe_replay=true loss=ppo loss_args.clip_ratio_low=0.2 loss_args.clip_ratio_high=0.28 loss_args.kl_coef=0.0 \
    loss_args.entropy_coef=0 loss_args.token_reduce=mean-norm loss_args.batch_reduce=step-mean \
    actor.use_dynamic_bsz=true actor.max_token_len_per_gpu=18432 actor.grad_clip=1.0 actor.optimizer_args.lr=1e-6 \
    actor.optimizer_args.weight_decay=0.1 actor.lr_scheduler_args.lr_warmup_steps=0 \
    actor.megatron.pipeline_model_parallel_size=16 \
    actor.megatron.tensor_model_parallel_size=4 actor.megatron.expert_model_parallel_size=4 \
    actor.megatron.expert_tensor_parallel_size=1 actor.megatron.context_parallel_size=1 \
    sampler.tensor_model_parallel_size=8 sampler.name=native sampler.gpu_memory_utilization=0.75 sampler.enable_prefix_caching=false \
    decoding.temperature=1.0 decoding.n=8 validation.before_train=false validation.steps=10 validation.decoding.n=4 \
    "logger=[console]" project_name=math-agent experiment_name=math-qwen3-235b-a22b num_gpus_per_node=8 num_nodes=8 \
    save_steps=20 total_epochs=100 stepwise_advantage_mode=broadcast program.name=react \
    +program.env_name="${ROOT}/recipes/math/env.py:MathEnvironment" +program.env_args.max_turns=1 \
    +program.agent_name="${ROOT}/recipes/math/agent.py:MathAgent" "$@"
