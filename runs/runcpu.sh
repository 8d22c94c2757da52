#!/bin/bash
# Small CPU-only walk through every stage (minutes to hours, toy quality): useful to check an installation.
set -e
export NANOCHAT_BASE_DIR="${NANOCHAT_BASE_DIR:-$HOME/.cache/nanochat}"
mkdir -p "$NANOCHAT_BASE_DIR"
WANDB_RUN="${WANDB_RUN:-dummy}"

python -c "from nanochat_b200.utils.build import build_tokenizer_extension as b; b()"
python -m nanochat_b200.dataset -n 8
python -m scripts.tok_train --max-chars=2000000000
python -m scripts.tok_eval
python -m scripts.base_train --depth=6 --head-dim=64 --window-pattern=L --max-seq-len=512 \
    --device-batch-size=32 --total-batch-size=16384 --eval-every=100 --eval-tokens=524288 \
    --core-metric-every=-1 --sample-every=100 --num-iterations=5000 --run=$WANDB_RUN
python -m scripts.base_eval --device-batch-size=1 --split-tokens=16384 --max-per-task=16
python -m scripts.chat_sft --eval-every=200 --eval-tokens=524288 --num-iterations=1500 --run=$WANDB_RUN
python -m scripts.chat_cli -p "hello"
