#!/usr/bin/env bash
# Profile GPT ops, collectives and P2P bandwidth on this node's B200s and write a self-contained
# profile directory (op CSVs per micro-batch / TP / algo, collective CSVs, P2P CSV, metadata).
set -euo pipefail

usage() {
    cat <<'USAGE'
Usage: scripts/profile_gpt.sh [options]

Required:
  --model gpt                 Supported model family.
  --model-size SIZE           350M | 1_3B | 2_6B | 6_7B | 13B | scale-layer.
  --hardware LABEL            Stable hardware label used by search.
  --tp-sizes LIST             Comma-separated TP sizes, for example 1,2,4.
  --num-nodes N               Number of participating nodes.
  --gpus-per-node N           Visible GPUs on each node.
  --node-rank N               Zero-based rank of this node.
  --master-addr HOST          Distributed rendezvous host or address.
  --master-port PORT          Distributed rendezvous port.
  --output DIR                Self-contained profile output directory.

Optional:
  --python PATH               Python interpreter (default: python3).
  --reference-profile FILE   Reference op cache required for multi-node task splitting.
  --dry-run                  Validate inputs and write metadata plus the command plan only.
  -h, --help                 Show this help.
USAGE
}

fail() { echo "profile_gpt.sh: $*" >&2; exit 2; }

declare -A OPT=([python]=python3)
DRY_RUN=0
while [ "$#" -gt 0 ]; do
    case "$1" in
        --model|--model-size|--hardware|--tp-sizes|--num-nodes|--gpus-per-node|--node-rank|--master-addr|--master-port|--output|--python|--reference-profile)
            [ "$#" -ge 2 ] && [ -n "${2:-}" ] || fail "$1 requires a value"
            OPT[${1#--}]="$2"; shift 2 ;;
        --dry-run) DRY_RUN=1; shift ;;
        -h|--help) usage; exit 0 ;;
        *) usage >&2; fail "unknown argument: $1" ;;
    esac
done
for key in model model-size hardware tp-sizes num-nodes gpus-per-node node-rank master-addr master-port output; do
    [ -n "${OPT[$key]:-}" ] || { usage >&2; fail "missing required arguments"; }
done
PY=${OPT[python]}
[ "${OPT[model]}" = "gpt" ] || fail "--model must be gpt"
case "${OPT[model-size]}" in 350M|1_3B|2_6B|6_7B|13B|scale-layer) ;; *) fail "unsupported --model-size: ${OPT[model-size]}" ;; esac
for key in num-nodes gpus-per-node node-rank master-port; do
    [[ "${OPT[$key]}" =~ ^[0-9]+$ ]] || fail "--$key must be an integer"
done
[ "${OPT[num-nodes]}" -ge 1 ] || fail "--num-nodes must be positive"
[ "${OPT[gpus-per-node]}" -ge 1 ] || fail "--gpus-per-node must be positive"
[ "${OPT[node-rank]}" -lt "${OPT[num-nodes]}" ] || fail "--node-rank must be smaller than --num-nodes"
[ "${OPT[master-port]}" -ge 1 ] && [ "${OPT[master-port]}" -le 65535 ] || fail "--master-port must be between 1 and 65535"
IFS=',' read -r -a TPS <<< "${OPT[tp-sizes]}"
[ "${#TPS[@]}" -gt 0 ] || fail "--tp-sizes cannot be empty"
for tp in "${TPS[@]}"; do
    [[ "$tp" =~ ^[0-9]+$ ]] || fail "each TP size must be an integer"
    [ "$tp" -ge 1 ] || fail "each TP size must be positive"
    [ $((tp & (tp - 1))) -eq 0 ] || fail "each TP size must be a power of two"
    [ "$tp" -le "${OPT[gpus-per-node]}" ] || fail "TP size $tp exceeds --gpus-per-node ${OPT[gpus-per-node]}"
done
command -v "$PY" >/dev/null 2>&1 || fail "Python interpreter not found: $PY"
[ "$DRY_RUN" -eq 1 ] || [ "${OPT[num-nodes]}" -eq 1 ] || [ -f "${OPT[reference-profile]:-}" ] || \
    fail "--reference-profile is required for multi-node profiling"
if [ "$DRY_RUN" -eq 0 ]; then
    "$PY" -c 'import sys, torch; n = int(sys.argv[1]); sys.exit(0 if torch.cuda.is_available() and torch.cuda.device_count() >= n else 1)' \
        "${OPT[gpus-per-node]}" || fail "CUDA is unavailable or fewer than ${OPT[gpus-per-node]} devices are visible"
fi

ROOT=$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)
export PYTHONPATH="${ROOT}${PYTHONPATH:+:${PYTHONPATH}}"
mkdir -p "${OPT[output]}"
OUT=$(cd "${OPT[output]}" && pwd)
PLAN="${OUT}/profile_plan.txt"
RDZV="--nnodes ${OPT[num-nodes]} --node-rank ${OPT[node-rank]} --master-addr ${OPT[master-addr]} --master-port ${OPT[master-port]}"
{
    for tp in "${TPS[@]}"; do
        echo "$PY -m torch.distributed.run --nproc-per-node $tp $RDZV -m eth_b200.profiler.op_profiler --prof-tp-size $tp --prof-path <output>/ --prof-cache-file <output>/gpt_op_profile.pkl --prof-model-name gpt --prof-model-size ${OPT[model-size]}"
        echo "$PY -m eth_b200.profiler.comm_profiler --prof-path <output>/ --prof-cache-file <output>/gpt_comm_profile.pkl --prof-op-time-path <output>/ --prof-tp-size $tp --prof-model-name gpt --prof-model-size ${OPT[model-size]}"
    done
    echo "$PY -m eth_b200.profiler.p2p_band_profiler # writes <output>/p2p_intra_node.csv or p2p_inter_node.csv"
} > "$PLAN"

metadata() {
    "$PY" -m eth_b200.profiler.profile_metadata --output "$OUT" --status "$1" --model "${OPT[model]}" \
        --model-size "${OPT[model-size]}" --hardware "${OPT[hardware]}" --tp-sizes "${OPT[tp-sizes]}" \
        --num-nodes "${OPT[num-nodes]}" --gpus-per-node "${OPT[gpus-per-node]}" --node-rank "${OPT[node-rank]}"
}
if [ "$DRY_RUN" -eq 1 ]; then
    metadata planned
    echo "Validated profiling plan: $PLAN"
    exit 0
fi

cd "$ROOT"
for tp in "${TPS[@]}"; do
    ARGS=(--prof-tp-size "$tp" --prof-path "${OUT}/" --prof-cache-file "${OUT}/gpt_op_profile.pkl" --prof-model-name gpt
          --prof-model-size "${OPT[model-size]}" --prof-warmup-times 10 --prof-repeat-times 40)
    if [ "${OPT[num-nodes]}" -gt 1 ]; then
        ARGS+=(--prof-num-nodes "${OPT[num-nodes]}" --prof-node-rank "${OPT[node-rank]}" --prof-ref-data "${OPT[reference-profile]}")
    fi
    # shellcheck disable=SC2086
    "$PY" -m torch.distributed.run --nproc-per-node "$tp" $RDZV -m eth_b200.profiler.op_profiler "${ARGS[@]}" \
        2>&1 | tee "${OUT}/op_tp${tp}_rank${OPT[node-rank]}.log"
    if [ "${OPT[node-rank]}" -eq 0 ] && [ "$tp" -gt 1 ]; then
        MASTER_ADDR="${OPT[master-addr]}" MASTER_PORT="${OPT[master-port]}" "$PY" -m eth_b200.profiler.comm_profiler \
            --prof-path "${OUT}/" --prof-cache-file "${OUT}/gpt_comm_profile.pkl" --prof-op-time-path "${OUT}/" \
            --prof-tp-size "$tp" --prof-model-name gpt --prof-model-size "${OPT[model-size]}" \
            --prof-warmup-times 5 --prof-repeat-times 20 --max-data-size 4096 2>&1 | tee "${OUT}/comm_tp${tp}.log"
    fi
done
if [ "${OPT[node-rank]}" -eq 0 ] && [ "${OPT[gpus-per-node]}" -ge 2 ]; then
    MASTER_ADDR="${OPT[master-addr]}" MASTER_PORT="${OPT[master-port]}" NNODES=1 GPUS_PER_NODE=2 NODE_RANK=0 \
        FILE_NAME="${OUT}/p2p_intra_node.csv" "$PY" -m eth_b200.profiler.p2p_band_profiler 2>&1 | tee "${OUT}/p2p_intra_node.log"
fi
if [ "${OPT[num-nodes]}" -eq 2 ]; then
    MASTER_ADDR="${OPT[master-addr]}" MASTER_PORT="${OPT[master-port]}" NNODES=2 GPUS_PER_NODE=1 NODE_RANK="${OPT[node-rank]}" \
        FILE_NAME="${OUT}/p2p_inter_node.csv" "$PY" -m eth_b200.profiler.p2p_band_profiler 2>&1 | tee "${OUT}/p2p_inter_node_rank${OPT[node-rank]}.log"
fi
metadata complete
echo "Profiling complete: $OUT"
