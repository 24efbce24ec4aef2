#!/bin/bash
# Wan2.1 training launch on one 8-GPU B200 box, same flag set as the reference launcher
# (examples/wan/run_wan.sh): N_GPU_FOR_TRAIN DiT ranks + N_GPU_FOR_DATA encoder ranks.
export PYTHONUNBUFFERED=1
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True

TP=${TP:-1}
CP=${CP:-2}
MBS=${MBS:-1}
N_MOE=${N_MOE:-1}
N_LAYERS=${N_LAYERS:-40}
N_GPU_FOR_TRAIN=${N_GPU_FOR_TRAIN:-4}
N_GPU_FOR_DATA=${N_GPU_FOR_DATA:-1}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-11220}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
N_GPU=$((N_GPU_FOR_TRAIN + N_GPU_FOR_DATA))
GBS=$((N_GPU_FOR_TRAIN * MBS / CP / TP / N_MOE))

case $N_MOE in
  1) MOE_ARGS=(--moe-step-factor-list 0.0 --moe-step-factor-list 1.0) ;;
  2) MOE_ARGS=(--moe-step-factor-list 0.0 --moe-step-factor-list 0.833 --moe-step-factor-list 1.0) ;;
  4) MOE_ARGS=(--moe-step-factor-list 0.0 --moe-step-factor-list 0.625 --moe-step-factor-list 0.833
               --moe-step-factor-list 0.937 --moe-step-factor-list 1.0) ;;
  *) echo "N_MOE must be 1, 2 or 4"; exit 1 ;;
esac

DISTRIBUTED_ARGS=(--nproc_per_node $N_GPU --nnodes $NNODES --node_rank $NODE_RANK
                  --master_addr $MASTER_ADDR --master_port $MASTER_PORT)
MODEL_ARGS=(--num-layers $N_LAYERS --hidden-size 5120 --num-attention-heads 40 --seq-length 512
            --max-position-embeddings 4096 --tokenizer-type NullTokenizer --vocab-size 0)
TRAINING_ARGS=(--model ParallelWanModel --task-type wan_i2v_prone --micro-batch-size $MBS
               --global-batch-size $GBS --train-iters 10000 --weight-decay 1e-2 --init-method-std 0.006
               --clip-grad 0.0 --bf16 --lr 1e-5 --lr-decay-style constant --lr-warmup-fraction 0
               --recompute-granularity full --recompute-method block --recompute-num-layers $N_LAYERS
               --use-distributed-optimizer --no-rope-fusion --distributed-timeout-minutes 60
               --init-on-device)   # 7 B parameters at 20 layers: create them on the GPU, not in host memory
MODEL_PARALLEL_ARGS=(--tensor-model-parallel-size $TP --context-parallel-size $CP --distributed-vae
                     --distributed-vae-world-size $N_GPU_FOR_DATA --consumer-models-num $N_MOE)
DATA_ARGS=(--dataset-type FakeDataset --split 949,50,1 --dataloader-type single --num-workers 1 --num-frames 81)
LOGGING_ARGS=(--tensorboard-queue-size 10 --log-interval 1 --save-interval 10000 --eval-interval 10000
              --eval-iters 0)
if [ -n "$ENCODER_MODEL_PATH" ]; then
  LOGGING_ARGS+=(--encoder-model-path "$ENCODER_MODEL_PATH" --encoder-tokenizer-path "$ENCODER_TOKENIZER_PATH")
else
  LOGGING_ARGS+=(--encoder-name synthetic_wan_encoder)   # random-weight stand-in: no checkpoints needed
fi

torchrun "${DISTRIBUTED_ARGS[@]}" "$(dirname "$0")/pretrain_wan.py" \
  "${MODEL_ARGS[@]}" "${TRAINING_ARGS[@]}" "${MODEL_PARALLEL_ARGS[@]}" "${MOE_ARGS[@]}" \
  "${DATA_ARGS[@]}" "${LOGGING_ARGS[@]}" "$@" | tee wan.log
