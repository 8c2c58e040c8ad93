#!/usr/bin/env bash
# Math RL, Qwen3-8B, colocated FSDP-style trainer + sampler on one 8-GPU node (GRPO, 64 prompts x 4 samples,
# 24k-token packed micro-batches, temperature 0.6).
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
[ -f "${ROOT}/data/math/train.parquet" ] || python "${ROOT}/recipes/math/data.py" --out "${ROOT}/data/math/train.parquet"
[ -f "${ROOT}/data/math/test.parquet" ] || python "${ROOT}/recipes/math/data.py" --split test --synthetic_size 64 --out "${ROOT}/data/math/test.parquet"
axon train --fg -- \
    advantage=grpo train_files="${ROOT}/data/math/train.parquet" val_files="${ROOT}/data/math/test.parquet" \
    train_batch_size=64 max_prompt_length=2048 max_seq_length=4096 model_path=Qwen/Qwen3-8B hybrid_engine=true \
    actor.optimizer_args.lr=1e-6 actor.fsdp.use_remove_padding=true mini_batch_size=16 actor.use_dynamic_bsz=true \
    actor.max_token_len_per_gpu=24000 loss=ppo loss_args.kl_coef=0.0 loss_args.kl_type=low_var_kl \
    actor.fsdp.ulysses_sequence_parallel_size=1 actor.fsdp.enable_gradient_checkpointing=true \
    actor.param_offload=false actor.optimizer_offload=false sampler.tensor_model_parallel_size=1 sampler.name=native \
    decoding.temperature=0.6 decoding.n=4 sampler.gpu_memory_utilization=0.85 sampler.enforce_eager=false \
    validation.before_train=false validation.steps=10 validation.decoding.n=1 validation.decoding.temperature=0.6 \
    validation.decoding.top_p=0.95 critic_warmup=0 "logger=[console]" project_name=math-agent experiment_name=math-qwen3-8b \
    num_gpus_per_node=8 num_nodes=1 save_steps=10 total_epochs=1000 stepwise_advantage_mode=broadcast program.name=react \
    +program.env_name="${ROOT}/recipes/math/env.py:MathEnvironment" +program.env_args.max_turns=1 \
    +program.agent_name="${ROOT}/recipes/math/agent.py:MathAgent" "$@"
