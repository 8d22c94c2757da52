#!/bin/bash
# IsoFLOP sweep: for every compute budget train every depth for exactly that many FLOPs and record the
# parameter breakdown, tokens seen and validation bpb. Finished (budget, depth) pairs are skipped on re-runs.
# Usage: bash runs/scaling_laws.sh   (FLOPS_BUDGETS="1e18 3e18" DEPTHS="8 10 12" to override)
set -e
export OMP_NUM_THREADS=1
export NANOCHAT_BASE_DIR="${NANOCHAT_BASE_DIR:-$HOME/.cache/nanochat}"
FLOPS_BUDGETS=(${FLOPS_BUDGETS:-1e18 2.15e18 4.64e18 1e19})
DEPTHS=(${DEPTHS:-8 10 12 14 16 18 20})
NPROC="${NPROC_PER_NODE:-8}"
WANDB_RUN="${WANDB_RUN:-scaling}"
EVAL_TOKENS="${EVAL_TOKENS:-$((100 * 524288))}"
LAUNCH="python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=$NPROC"
RESULTS_DIR="$NANOCHAT_BASE_DIR/scaling_laws_results"
RESULTS_FILE="$RESULTS_DIR/results.csv"
mkdir -p "$RESULTS_DIR"
[ -f "$RESULTS_FILE" ] || echo "flops_budget,depth,model_dim,params_wte,params_value_embeds,params_lm_head,params_transformer,params_scalars,params_total,num_iterations,tokens_trained,val_bpb,core_score,train_time_sec" > "$RESULTS_FILE"
log() { echo "[$(date '+%Y-%m-%d %H:%M:%S')] $1"; }
count() { grep "^$1 " "$2" | tail -1 | grep -oP '[\d,]+$' | tr -d ','; }

for flops in "${FLOPS_BUDGETS[@]}"; do
    log "Compute budget: $flops FLOPs"
    for d in "${DEPTHS[@]}"; do
        if grep -q "^${flops},${d}," "$RESULTS_FILE" 2>/dev/null; then
            log "Skipping d=$d at $flops FLOPs (already in results)"
            continue
        fi
        TAG="scaling_${flops}_d${d}"
        LOG_FILE="$RESULTS_DIR/${TAG}_train.log"
        if [ "$d" -ge 28 ]; then BATCH=8; elif [ "$d" -ge 20 ]; then BATCH=16; else BATCH=32; fi
        log "Training d=$d at $flops FLOPs..."
        START=$(date +%s)
        $LAUNCH -m scripts.base_train -- --depth=$d --target-flops=$flops --target-param-data-ratio=-1 \
            --run="${WANDB_RUN}_${TAG}" --model-tag="$TAG" --eval-tokens=$EVAL_TOKENS \
            --core-metric-every=999999 --core-metric-max-per-task=-1 --sample-every=-1 --save-every=-1 \
            --device-batch-size=$BATCH 2>&1 | tee "$LOG_FILE"
        TRAIN_TIME=$(( $(date +%s) - START ))
        NUM_ITERS=$(grep "Calculated number of iterations" "$LOG_FILE" | tail -1 | sed 's/.*: //' | tr -d ',')
        BATCH_TOKENS=$(grep "Total batch size" "$LOG_FILE" | tail -1 | grep -oP 'Total batch size \K[\d,]+' | tr -d ',')
        VAL_BPB=$(grep "Validation bpb:" "$LOG_FILE" | tail -1 | grep -oP '[\d.]+$')
        CORE=$(grep "CORE metric:" "$LOG_FILE" | tail -1 | awk '{print $NF}')
        echo "$flops,$d,$(( (d * 64 + 127) / 128 * 128 )),$(count wte "$LOG_FILE"),$(count value_embeds "$LOG_FILE"),$(count lm_head "$LOG_FILE"),$(count transformer_matrices "$LOG_FILE"),$(count scalars "$LOG_FILE"),$(count total "$LOG_FILE"),$NUM_ITERS,$(( NUM_ITERS * BATCH_TOKENS )),$VAL_BPB,${CORE:-0.0},$TRAIN_TIME" >> "$RESULTS_FILE"
    done
done
log "Results saved to: $RESULTS_FILE"
column -t -s',' "$RESULTS_FILE"
