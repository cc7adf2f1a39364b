#!/bin/bash
# Pre-training launcher for one 8xB200 node (counterpart of examples/pretrain/run_pretrain_{8,32,64,128}k.sh of the
# reference, which launch with mpirun across hosts).  Usage:
#   STAGE=8k   bash examples/pretrain/run_pretrain.sh            # from scratch
#   STAGE=128k CHECKPOINT_DIR=out/64k bash examples/pretrain/run_pretrain.sh   # length extension, weights-only resume
# RECOMPUTE=full|mlp chooses what the long-context stages recompute in the backward pass: whole layers (as the
# reference does) or only the feed-forward blocks (keeps attention and its projections; fits in 180 GB per GPU).
set -euo pipefail
STAGE=${STAGE:-8k}
NGPU=${NGPU:-8}
# several nodes: run this script on every node with NNODES, NODE_RANK (0..NNODES-1) and MASTER_ADDR (node 0) set.
# Context-parallel groups stay inside a node; across nodes FSDP runs over NCCL collectives.
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MODEL_CONFIG=${MODEL_CONFIG:-examples/pretrain/model_config/model_config_1b9_ksa_hybrid.json}
DATASET_CONFIG=${DATASET_CONFIG:-examples/pretrain/dataset_config/pretrain_kai_mmap_${STAGE}.json}
OUTPUT_DIR=${OUTPUT_DIR:-out/${STAGE}}
CHECKPOINT_DIR=${CHECKPOINT_DIR:-}
case "$STAGE" in
  8k)   CP=1; LR=4e-4; MIN_LR=4e-5; STEPS=127200; WARM=1000; DECAY=1000; GRAD_ACC=${GRAD_ACC:-30}; EXTRA="" ;;
  32k)  CP=2; LR=1e-5; MIN_LR=1e-6; STEPS=1600;   WARM=100;  DECAY=100;  GRAD_ACC=${GRAD_ACC:-60}; EXTRA="--enable-gradient-checkpointing --gradient-checkpointing-mode ${RECOMPUTE:-full}" ;;
  64k)  CP=4; LR=1e-5; MIN_LR=1e-6; STEPS=1600;   WARM=100;  DECAY=100;  GRAD_ACC=${GRAD_ACC:-120}; EXTRA="--enable-gradient-checkpointing --gradient-checkpointing-mode ${RECOMPUTE:-full}" ;;
  128k) CP=8; LR=1e-5; MIN_LR=1e-6; STEPS=1600;   WARM=100;  DECAY=100;  GRAD_ACC=${GRAD_ACC:-240}; EXTRA="--enable-gradient-checkpointing --gradient-checkpointing-mode ${RECOMPUTE:-full}" ;;
  *) echo "unknown STAGE $STAGE"; exit 1 ;;
esac
RESUME=""
if [ -n "$CHECKPOINT_DIR" ]; then RESUME="--checkpoint-dir $CHECKPOINT_DIR --resume-weights --resume-dataloader"; fi
mkdir -p "$OUTPUT_DIR"
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
python -m torch.distributed.run --nnodes="$NNODES" --node-rank="$NODE_RANK" --nproc-per-node "$NGPU" \
  --master-addr "$MASTER_ADDR" --master-port ${MASTER_PORT:-8499} \
  recipes/pretrain_ksa.py \
  --model-config "$MODEL_CONFIG" --dataset-config "$DATASET_CONFIG" --output-dir "$OUTPUT_DIR" $RESUME \
  --enable-dataset-checkpointing --context-parallel-size $CP --gradient-accumulation-steps $GRAD_ACC \
  --chunked-loss-minibatch-size 2048 --learning-rate $LR --min-lr $MIN_LR --weight-decay 0.01 --beta1 0.9 --beta2 0.95 \
  --fp32-weight --lr-scheduler-type wsd --num-warmup-steps $WARM --num-decay-steps $DECAY --num-training-steps $STEPS \
  --save-checkpoint-per-step 250 --logging-per-step 1 --clip-range 1.0 --seed 42 $EXTRA \
  --comment "${COMMENT:-ksa_b200}" --commit-id "$(git rev-parse --short HEAD 2>/dev/null || echo none)" \
  > "$OUTPUT_DIR/stdout.log" 2> "$OUTPUT_DIR/stderr.log"
