#!/bin/bash
# Smoke test: CPU unit tests, then (on a GPU machine) the GPU tests and nine two-step training
# runs covering the block types, attention types and optimizer families.  Unlike the reference's
# scripts/smoke_test.sh (every step `|| true`, always exit 0) a failing step fails the script.
set -euo pipefail
cd "$(dirname "$0")"
export WANDB_MODE=${WANDB_MODE:-disabled}
python -m pytest tests -q -m "not gpu" -x
if ! python -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  echo "no GPU: CPU tier only"; exit 0
fi
python -m nsa_optim_b200.ops.build
python -m pytest tests -q -m gpu -x
NG=$(python -c "import torch; print(torch.cuda.device_count())")
LAUNCH="python"
if [ "$NG" -gt 1 ]; then LAUNCH="python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node $NG"; fi
COMMON="--model_size 100M --context_length 512 --batch_size 1 --gradient_accumulation_steps 2 --num_train_steps 2 --warmup_steps 0 --log_interval 1 --synthetic_data --vocab_size 4096 --dtype bfloat16 --output_dir /tmp/nsa_smoke"
run() { echo "== $*"; $LAUNCH train.py $COMMON "$@"; }
run --mamba_type none --attn_type dense --optimizer_type adamw8bit
run --mamba_type none --attn_type nsa --nsa_block_size 64 --nsa_window_size 64 --nsa_num_selected_blocks 4 --optimizer_type adamw8bit
run --block_pattern DD --optimizer_type adamw8bit
run --block_pattern MM --optimizer_type adamw8bit
run --block_pattern MDMA --optimizer_type adamw8bit
run --block_pattern MDMA --optimizer_type soap8bit
run --block_pattern MDMA --optimizer_type soap4bit
run --mamba_type none --attn_type dense --optimizer_type adamw
run --mamba_type none --attn_type dense --optimizer_type adamw --gradient_checkpointing
echo "smoke test passed"
