#!/usr/bin/env bash
# Launch a training job: every argument is forwarded to `python -m flame_b200.train`.
#
#   NNODE=1 NGPU=8 LOG_RANK=0 bash train.sh --job.config_file flame_b200/models/fla.toml \
#       --job.dump_folder exp/transformer-340M --model.config configs/transformer_340M.json \
#       --model.tokenizer_path fla-hub/transformer-1.3B-100B --training.varlen ...
#
# Environment: NNODE, NGPU, LOG_RANK, MASTER_ADDR, MASTER_PORT (same knobs as the reference launcher).
# After training, the last checkpoint is exported as a Hugging Face style model directory.

params="$@"
echo "Launching training with: $params"

NNODE=${NNODE:-"1"}
NGPU=${NGPU:-"8"}
LOG_RANK=${LOG_RANK:-0}
if [[ -z "${MASTER_ADDR}" ]]; then export MASTER_ADDR="127.0.0.1"; fi
if [[ -z "${MASTER_PORT}" ]]; then export MASTER_PORT="29500"; fi

get_arg() { echo "$params" | grep -oP -- "--$1[ =]\K[^ ]+" | tail -1; }
path=$(get_arg "job.dump_folder"); path=${path:-exp}
steps=$(get_arg "training.steps")
config=$(get_arg "model.config")
tokenizer=$(get_arg "model.tokenizer_path")
model_type=$(python -c "import json,sys,os; p='$config'; p=os.path.join(p,'config.json') if os.path.isdir(p) else p; print(json.load(open(p)).get('model_type','model'))" 2>/dev/null || echo model)

mkdir -p "$path/logs"
cp -r configs "$path/" 2>/dev/null
cp -r flame_b200 "$path/" 2>/dev/null

date=$(date +%Y%m%d%H%M)
export WANDB_RESUME=${WANDB_RESUME:-allow}
export WANDB_PROJECT=${WANDB_PROJECT:-flame_b200}
export WANDB_NAME=${WANDB_NAME:-"$model_type-$(basename "$path")"}
export WANDB_RUN_ID=${WANDB_RUN_ID:-"$WANDB_NAME-$date"}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-"expandable_segments:True"}

set -x
python -m flame_b200.ops._build || exit 1
python -m torch.distributed.run --nnodes="${NNODE}" --nproc_per_node="${NGPU}" \
  --rdzv_backend c10d --rdzv_endpoint "${MASTER_ADDR}:${MASTER_PORT}" \
  --local-ranks-filter "${LOG_RANK}" --role rank --tee 3 --log-dir "$path/logs" \
  -m flame_b200.train $params
status=$?
set +x
if [[ $status -ne 0 ]]; then echo "training failed with status $status"; exit $status; fi

if [[ -n "$steps" && -n "$config" && -d "$path/checkpoint/step-$steps" ]]; then
  echo "Converting the step-$steps checkpoint under $path to a Hugging Face model directory"
  python -m flame_b200.utils.convert_dcp_to_hf --path "$path" --step "$steps" --config "$config" --tokenizer "$tokenizer"
fi
echo "Done"
