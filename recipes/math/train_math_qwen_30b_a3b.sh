#!/usr/bin/env bash
# Math RL, Qwen3-30B-A3B (sparse), colocated on one 8-GPU node with the model-parallel trainer: pipeline 2 x (tensor =
# expert parallel 4) for training, sampler groups of 4 ranks (they divide heads and experts) whose weights are refreshed
# from the trainer's gathered tensors before every rollout; the experts the sampler routed to are replayed in training.
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
[ -f "${ROOT}/data/math/train.parquet" ] || python "${ROOT}/recipes/math/data.py" --out "${ROOT}/data/math/train.parquet"
[ -f "${ROOT}/data/math/test.parquet" ] || python "${ROOT}/recipes/math/data.py" --split test --synthetic_size 64 --out "${ROOT}/data/math/test.parquet"
axon train --fg -- \
    strategy=megatron advantage=rloo train_files="${ROOT}/data/math/train.parquet" val_files="${ROOT}/data/math/test.parquet" \
    train_batch_size=64 mini_batch_size=64 max_prompt_length=2048 max_seq_length=16384 model_path=Qwen/Qwen3-30B-A3B \
    hybrid_engine=true moe_replay=true loss=ppo loss_args.clip_ratio_low=0.2 loss_args.clip_ratio_high=0.28 loss_args.kl_coef=0.0 \
    actor.use_dynamic_bsz=true actor.max_token_len_per_gpu=34816 actor.grad_clip=1.0 actor.optimizer_args.lr=1e-6 \
    actor.optimizer_args.weight_decay=0.1 actor.megatron.pipeline_model_parallel_size=2 \
    actor.megatron.tensor_model_parallel_size=4 actor.megatron.expert_model_parallel_size=4 \
    actor.megatron.expert_tensor_parallel_size=1 actor.megatron.context_parallel_size=1 \
    sampler.tensor_model_parallel_size=4 sampler.name=native sampler.gpu_memory_utilization=0.7 sampler.enable_prefix_caching=false \
    decoding.temperature=1.0 decoding.n=8 validation.before_train=false validation.steps=10 validation.decoding.n=4 \
    "logger=[console]" project_name=math-agent experiment_name=math-qwen3-30b-a3b num_gpus_per_node=8 num_nodes=1 \
    save_steps=20 total_epochs=100 stepwise_advantage_mode=broadcast program.name=react \
    +program.env_name="${ROOT}/recipes/math/env.py:MathEnvironment" +program.env_args.max_turns=1 \
    +program.agent_name="${ROOT}/recipes/math/agent.py:MathAgent" "$@"
