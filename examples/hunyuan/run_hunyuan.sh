#!/bin/bash
# HunyuanVideo-13B, 720P x 129 frames on one 8-GPU box: TP 2 x CP 4, sharded AdamW, full activation recompute.
# Synthetic latents by default; add --distributed-vae --distributed-vae-world-size N (and N more ranks) to feed
# the DiT from encoder ranks.
set -euo pipefail
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-6000}
cd "$(dirname "$0")/../.."

torchrun --nproc_per_node "$GPUS_PER_NODE" --nnodes 1 --master_addr "$MASTER_ADDR" --master_port "$MASTER_PORT" \
    examples/hunyuan/pretrain_hunyuan.py \
    --model ParallelHunyuanVideoModel --model-preset hunyuanvideo-13b-t2v \
    --tensor-model-parallel-size 2 --context-parallel-size 4 \
    --micro-batch-size 1 --global-batch-size 1 --train-iters 100 \
    --num-frames 129 --video-resolution 720 1280 --synthetic-latents \
    --bf16 --lr 1e-5 --weight-decay 1e-2 --clip-grad 1.0 \
    --use-distributed-optimizer --init-on-device \
    --recompute-granularity full --recompute-method block --recompute-num-layers 1000 \
    --log-interval 1 --seed 1234 "$@"
