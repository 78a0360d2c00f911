#!/bin/bash
# The three headline runs: 1B MDMA hybrid, 64K context, on every GPU of the node, one run per
# optimizer.  Counterpart of the reference's run_experiments.sh:1-7 (same flags, working shell).
set -euo pipefail
NG=${NG:-$(python -c "import torch; print(max(torch.cuda.device_count(), 1))")}
for OPT in adamw8bit soap8bit soap4bit; do
  python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node "$NG" train.py \
    --model_size 1B --block_pattern MDMA --attn_type nsa --optimizer_type "$OPT" \
    --context_length 65536 --batch_size 1 --gradient_accumulation_steps 4 \
    -lr 1e-3 -wd 0.05 -clip 2.0 "$@"
done
