#!/bin/bash
# Train a series of depths at their compute-optimal horizon and collect one CSV row per model.
# Usage: bash runs/miniseries.sh [series_name]
set -e
export OMP_NUM_THREADS=1
export NANOCHAT_BASE_DIR="${NANOCHAT_BASE_DIR:-$HOME/.cache/nanochat}"
SERIES_NAME="${1:-${SERIES_NAME:-$(date +%b%d | tr '[:upper:]' '[:lower:]')}}"
DEPTHS=(${DEPTHS:-12 14 16 18 20 22 24 26})
NPROC="${NPROC_PER_NODE:-8}"
WANDB_RUN="${WANDB_RUN:-${SERIES_NAME}_miniseries}"
LAUNCH="python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=$NPROC"
RESULTS_DIR="$NANOCHAT_BASE_DIR/${SERIES_NAME}_miniseries_results"
RESULTS_FILE="$RESULTS_DIR/results.csv"
mkdir -p "$RESULTS_DIR"
[ -f "$RESULTS_FILE" ] || echo "depth,model_dim,num_params,num_scaling_params,num_iterations,tokens_trained,param_data_ratio,val_bpb,core_score,train_time_sec" > "$RESULTS_FILE"
log() { echo "[$(date '+%Y-%m-%d %H:%M:%S')] $1"; }

for d in "${DEPTHS[@]}"; do
    TAG="${SERIES_NAME}_miniseries_d${d}"
    LOG_FILE="$RESULTS_DIR/${TAG}_train.log"
    if [ "$d" -ge 28 ]; then BATCH=8; elif [ "$d" -ge 20 ]; then BATCH=16; else BATCH=32; fi
    log "Training d=$d (device batch $BATCH)..."
    START=$(date +%s)
    $LAUNCH -m scripts.base_train -- --depth=$d --run="${WANDB_RUN}_d${d}" --model-tag="$TAG" \
        --core-metric-every=999999 --core-metric-max-per-task=-1 --sample-every=-1 --save-every=-1 \
        --device-batch-size=$BATCH 2>&1 | tee "$LOG_FILE"
    TRAIN_TIME=$(( $(date +%s) - START ))
    # figures are scraped from the driver's log lines
    NUM_PARAMS=$(grep "^total " "$LOG_FILE" | tail -1 | grep -oP '[\d,]+$' | tr -d ',')
    MATRICES=$(grep "^transformer_matrices" "$LOG_FILE" | tail -1 | grep -oP '[\d,]+$' | tr -d ',')
    LM_HEAD=$(grep "^lm_head" "$LOG_FILE" | tail -1 | grep -oP '[\d,]+$' | tr -d ',')
    NUM_SCALING=$(( MATRICES + LM_HEAD ))
    NUM_ITERS=$(grep "Calculated number of iterations" "$LOG_FILE" | tail -1 | sed 's/.*: //' | tr -d ',')
    BATCH_TOKENS=$(grep "Total batch size" "$LOG_FILE" | tail -1 | grep -oP 'size [\d,]+' | grep -oP '[\d,]+' | tr -d ',')
    TOKENS=$(( NUM_ITERS * BATCH_TOKENS ))
    RATIO=$(python -c "print(f'{$TOKENS / $NUM_SCALING:.2f}')")
    VAL_BPB=$(grep "Validation bpb:" "$LOG_FILE" | tail -1 | grep -oP '[\d.]+$')
    CORE=$(grep "CORE metric:" "$LOG_FILE" | tail -1 | awk '{print $NF}')
    log "  d=$d: params=$NUM_PARAMS scaling=$NUM_SCALING ratio=$RATIO bpb=$VAL_BPB CORE=${CORE:-0.0} time=${TRAIN_TIME}s"
    echo "$d,$(( (d * 64 + 127) / 128 * 128 )),$NUM_PARAMS,$NUM_SCALING,$NUM_ITERS,$TOKENS,$RATIO,$VAL_BPB,${CORE:-0.0},$TRAIN_TIME" >> "$RESULTS_FILE"
done
log "Results saved to: $RESULTS_FILE"
column -t -s',' "$RESULTS_FILE"
