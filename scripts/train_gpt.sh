#!/usr/bin/env bash
# Validate an HPP GPT config on CPU, then launch one rank per GPU of this node with torch.distributed.run.
set -euo pipefail

usage() {
    cat <<'USAGE'
Usage: scripts/train_gpt.sh \
  --config <gpt_config.json> --gpus-per-node <n> --num-nodes <n> --node-rank <r> \
  --master-addr <host> --master-port <port> \
  [--log-dir <dir>] [--train-iters <n>] [--precision <fp32|fp16|bf16>] [--loss-scale <value>] \
  [--attention-dropout <p>] [--hidden-dropout <p>] [--clip-grad <value>] \
  [--grad-sync-mode <tensor|block>] [--grad-sync-bucket-size-mb <size_mb>] \
  [--grad-sync-dump-plan <plan_json>] [--grad-sync-debug-replicated-check] \
  [--grad-sync-metadata-transport <auto|object|tensor>] \
  [--grad-sync-runtime-evidence-dir <runtime_evidence_dir>] [--evidence-dir <snapshot_dir>] \
  [--evidence-canonical-init] [--vocab-padding-multiple <value>] [--save <dir>] [--load <dir>] \
  [--save-interval <n>] [--python <python_path>] [--validate-only]
USAGE
}

declare -A OPT=([train-iters]=3 [precision]=fp16 [grad-sync-mode]=tensor [grad-sync-bucket-size-mb]=32
                [grad-sync-metadata-transport]=auto [python]=python3)
declare -A FLAG=()
while [ "$#" -gt 0 ]; do
    case "$1" in
        --config|--gpus-per-node|--num-nodes|--node-rank|--master-addr|--master-port|--log-dir|--train-iters|--precision|--loss-scale|--attention-dropout|--hidden-dropout|--clip-grad|--grad-sync-mode|--grad-sync-bucket-size-mb|--grad-sync-dump-plan|--grad-sync-metadata-transport|--grad-sync-runtime-evidence-dir|--evidence-dir|--vocab-padding-multiple|--save|--load|--save-interval|--python)
            [ "$#" -ge 2 ] || { echo "$1 requires a value" >&2; exit 1; }
            OPT[${1#--}]="$2"; shift 2 ;;
        --grad-sync-debug-replicated-check|--evidence-canonical-init|--validate-only)
            FLAG[${1#--}]=1; shift ;;
        -h|--help) usage; exit 0 ;;
        *) echo "Unknown argument: $1" >&2; usage >&2; exit 1 ;;
    esac
done
for key in config gpus-per-node num-nodes node-rank master-addr master-port; do
    [ -n "${OPT[$key]:-}" ] || { echo "Missing required argument --$key" >&2; usage >&2; exit 1; }
done
case "${OPT[precision]}" in fp32|fp16|bf16) ;; *) echo "PRECISION must be fp32, fp16, or bf16" >&2; exit 1 ;; esac
case "${OPT[grad-sync-mode]}" in tensor|block) ;; *) echo "GRAD_SYNC_MODE must be tensor or block" >&2; exit 1 ;; esac
case "${OPT[grad-sync-metadata-transport]}" in auto|object|tensor) ;; *) echo "GRAD_SYNC_METADATA_TRANSPORT must be auto, object, or tensor" >&2; exit 1 ;; esac
for key in gpus-per-node num-nodes node-rank master-port train-iters; do
    [[ "${OPT[$key]}" =~ ^[0-9]+$ ]] || { echo "${key} must be an integer" >&2; exit 1; }
done
[ "${OPT[gpus-per-node]}" -gt 0 ] || { echo "GPUS_PER_NODE must be positive" >&2; exit 1; }
[ "${OPT[num-nodes]}" -gt 0 ] || { echo "NUM_NODES must be positive" >&2; exit 1; }
[ "${OPT[node-rank]}" -lt "${OPT[num-nodes]}" ] || { echo "NODE_RANK must be smaller than NUM_NODES" >&2; exit 1; }
[ "${OPT[master-port]}" -gt 0 ] && [ "${OPT[master-port]}" -le 65535 ] || { echo "MASTER_PORT must be between 1 and 65535" >&2; exit 1; }
[ "${OPT[train-iters]}" -gt 0 ] || { echo "TRAIN_ITERS must be positive" >&2; exit 1; }
[[ "${OPT[grad-sync-bucket-size-mb]}" =~ ^[0-9]+$ ]] && [ "${OPT[grad-sync-bucket-size-mb]}" -gt 0 ] || \
    { echo "GRAD_SYNC_BUCKET_SIZE_MB must be a positive integer" >&2; exit 1; }

ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
abs() { case "$1" in /*) printf '%s\n' "$1" ;; *) printf '%s/%s\n' "$PWD" "$1" ;; esac; }
CONFIG="$(abs "${OPT[config]}")"
export PYTHONPATH="${ROOT}${PYTHONPATH:+:${PYTHONPATH}}"
[ -f "$CONFIG" ] || { echo "Config file not found: $CONFIG" >&2; exit 1; }
PY=${OPT[python]}
command -v "$PY" >/dev/null 2>&1 || { echo "Python interpreter not found: $PY" >&2; exit 1; }
WORLD=$((OPT[gpus-per-node] * OPT[num-nodes]))
"$PY" "${ROOT}/tools/validation/validate_train_config.py" --config "$CONFIG" --world-size "$WORLD" \
    --grad-sync-mode "${OPT[grad-sync-mode]}"

if [ -n "${FLAG[validate-only]:-}" ]; then
    echo "Training inputs validated; distributed launch skipped."
    exit 0
fi

LOG_DIR="${OPT[log-dir]:-${ROOT}/logs/eth_b200_gpt_$(date '+%Y-%m-%d-%H-%M-%S')}"
LOG_DIR="$(abs "$LOG_DIR")"
mkdir -p "${LOG_DIR}/csv"
NVCC="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
command -v nvcc >/dev/null 2>&1 && NVCC="$(command -v nvcc)"
"$PY" "${ROOT}/tools/validation/validate_cuda_toolchain.py" --nvcc "$NVCC"
"$PY" -m eth_b200.build_ext >/dev/null

echo "Launching GPT training"
echo "  config: ${CONFIG}"
echo "  distributed: ${OPT[num-nodes]} node(s), ${OPT[gpus-per-node]} GPU(s)/node, rank ${OPT[node-rank]}"
echo "  master: ${OPT[master-addr]}:${OPT[master-port]}"
echo "  log_dir: ${LOG_DIR}"
echo "  train_iters: ${OPT[train-iters]}"
echo "  precision: ${OPT[precision]}"
echo "  grad_sync: ${OPT[grad-sync-mode]}, ${OPT[grad-sync-bucket-size-mb]} MiB, ${OPT[grad-sync-metadata-transport]} metadata"

ARGS=(--flexpipe-config "$CONFIG" --train-iters "${OPT[train-iters]}" --eval-iters 0 --lr-decay-iters 320000
      --distributed-backend nccl --lr 0.00015 --lr-decay-style cosine --min-lr 1.0e-5 --weight-decay 1e-2
      --clip-grad 1.0 --lr-warmup-fraction .01 --log-interval 1 --DDP-impl local
      --grad-sync-mode "${OPT[grad-sync-mode]}" --grad-sync-bucket-size-mb "${OPT[grad-sync-bucket-size-mb]}"
      --grad-sync-metadata-transport "${OPT[grad-sync-metadata-transport]}" --log-path "${LOG_DIR%/}/")
case "${OPT[precision]}" in fp16) ARGS+=(--fp16) ;; bf16) ARGS+=(--bf16) ;; esac
[ -z "${OPT[loss-scale]:-}" ] || ARGS+=(--loss-scale "${OPT[loss-scale]}")
[ -z "${OPT[attention-dropout]:-}" ] || ARGS+=(--attention-dropout "${OPT[attention-dropout]}")
[ -z "${OPT[hidden-dropout]:-}" ] || ARGS+=(--hidden-dropout "${OPT[hidden-dropout]}")
[ -z "${OPT[clip-grad]:-}" ] || ARGS+=(--clip-grad "${OPT[clip-grad]}")
[ -z "${OPT[grad-sync-dump-plan]:-}" ] || ARGS+=(--grad-sync-dump-plan "$(abs "${OPT[grad-sync-dump-plan]}")")
[ -z "${FLAG[grad-sync-debug-replicated-check]:-}" ] || ARGS+=(--grad-sync-debug-replicated-check)
[ -z "${OPT[grad-sync-runtime-evidence-dir]:-}" ] || ARGS+=(--grad-sync-runtime-evidence-dir "$(abs "${OPT[grad-sync-runtime-evidence-dir]}")")
[ -z "${OPT[evidence-dir]:-}" ] || ARGS+=(--grad-sync-evidence-dir "$(abs "${OPT[evidence-dir]}")")
[ -z "${FLAG[evidence-canonical-init]:-}" ] || ARGS+=(--grad-sync-evidence-canonical-init)
[ -z "${OPT[vocab-padding-multiple]:-}" ] || ARGS+=(--make-vocab-size-divisible-by "${OPT[vocab-padding-multiple]}")
[ -z "${OPT[save]:-}" ] || ARGS+=(--save "$(abs "${OPT[save]}")")
[ -z "${OPT[load]:-}" ] || ARGS+=(--load "$(abs "${OPT[load]}")")
[ -z "${OPT[save-interval]:-}" ] || ARGS+=(--save-interval "${OPT[save-interval]}")

cd "$ROOT"
"$PY" -m torch.distributed.run --nproc-per-node "${OPT[gpus-per-node]}" --nnodes "${OPT[num-nodes]}" \
    --node-rank "${OPT[node-rank]}" --master-addr "${OPT[master-addr]}" --master-port "${OPT[master-port]}" \
    -m eth_b200.runtime.pretrain_gpt "${ARGS[@]}" 2>&1 | tee "${LOG_DIR}/gpt_train_rank${OPT[node-rank]}.log"
