#!/usr/bin/env bash
# FrozenLake, Qwen3-30B-A3B, disaggregated on one 8-GPU node: 4 trainer GPUs (expert parallel 4) and 4 sampler
# GPUs; the sampler generates step N+1 while the trainer works on step N, weights travel through the
# trainer -> sampler push after every step.
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
python "${ROOT}/recipes/frozenlake/data.py" --out "${ROOT}/data/frozenlake"
axon train --fg -- \
    model_path=Qwen/Qwen3-30B-A3B strategy=megatron hybrid_engine=false enable_one_off_pipeline=true driver_mode=sync \
    sampler_trainer_gpu_ratio=1 num_gpus_per_node=8 moe_replay=true \
    train_files="${ROOT}/data/frozenlake/train.parquet" val_files="${ROOT}/data/frozenlake/test.parquet" \
    train_batch_size=128 mini_batch_size=128 decoding.n=16 decoding.temperature=0.7 max_prompt_length=2048 max_seq_length=10240 \
    advantage=grpo loss=ppo actor.megatron.tensor_model_parallel_size=1 actor.megatron.expert_model_parallel_size=4 \
    actor.use_dynamic_bsz=true actor.max_token_len_per_gpu=32768 sampler.tensor_model_parallel_size=1 \
    sampler.expert_parallel_size=4 program.name=react \
    +program.env_name="${ROOT}/recipes/frozenlake/env.py:FrozenLakeEnv" +program.agent_name="${ROOT}/recipes/frozenlake/agent.py:FrozenLakeAgent" \
    "$@"
