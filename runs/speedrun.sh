#!/bin/bash
# End-to-end pipeline on one 8-GPU node: data -> tokenizer -> pretrain (d24, fp8) -> eval -> SFT -> chat eval.
# Usage: bash runs/speedrun.sh            (WANDB_RUN=name to log to wandb, NPROC_PER_NODE to change the GPU count)
set -e
export OMP_NUM_THREADS=1
export NANOCHAT_BASE_DIR="${NANOCHAT_BASE_DIR:-$HOME/.cache/nanochat}"
mkdir -p "$NANOCHAT_BASE_DIR"
WANDB_RUN="${WANDB_RUN:-dummy}"
NPROC="${NPROC_PER_NODE:-8}"
LAUNCH="python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=$NPROC"

python -m nanochat_b200.utils.build                # native extensions (sm_100a kernels, C++ tokenizer)

python -m nanochat_b200.dataset -n 8               # enough shards to train the tokenizer ...
python -m nanochat_b200.dataset -n 170 &           # ... while the pretraining shards download
DATASET_PID=$!
python -m scripts.tok_train
python -m scripts.tok_eval
echo "Waiting for dataset download to complete..."
wait $DATASET_PID

$LAUNCH -m scripts.base_train -- --depth=24 --target-param-data-ratio=8 --device-batch-size=16 --fp8 --run=$WANDB_RUN
$LAUNCH -m scripts.base_eval -- --device-batch-size=16
$LAUNCH -m scripts.chat_sft -- --run=$WANDB_RUN
$LAUNCH -m scripts.chat_eval -- -i sft
# chat with it:  python -m scripts.chat_cli -p "Why is the sky blue?"
