#!/usr/bin/env bash
# Validate a profile + node description, run the HPP search, and publish <output>/gpt_config.json.
set -euo pipefail

usage() {
    cat <<'USAGE'
Usage: scripts/search_gpt.sh [options]

Required:
  --profile-dir DIR           Completed profile directory (from profile_gpt.sh).
  --model-size SIZE           350M | 1_3B | 2_6B | 6_7B | 13B.
  --search-budget SECONDS     Search time budget.
  --global-batch-size N       Total samples per iteration.
  --node-description FILE     JSON with node_info and device_info.
  --output DIR                Output directory (gpt_config.json, logs/, configs/).

Optional:
  --python PATH               Python interpreter (default: python3).
  --dry-run                   Validate inputs and write search_plan.txt only.
  -h, --help                  Show this help.
USAGE
}

fail() { echo "search_gpt.sh: $*" >&2; exit 2; }

declare -A OPT=([python]=python3)
DRY_RUN=0
while [ "$#" -gt 0 ]; do
    case "$1" in
        --profile-dir|--model-size|--search-budget|--global-batch-size|--node-description|--output|--python)
            [ "$#" -ge 2 ] && [ -n "${2:-}" ] || fail "$1 requires a value"
            OPT[${1#--}]="$2"; shift 2 ;;
        --dry-run) DRY_RUN=1; shift ;;
        -h|--help) usage; exit 0 ;;
        *) usage >&2; fail "unknown argument: $1" ;;
    esac
done
for key in profile-dir model-size search-budget global-batch-size node-description output; do
    [ -n "${OPT[$key]:-}" ] || { usage >&2; fail "missing required arguments"; }
done
PY=${OPT[python]}
case "${OPT[model-size]}" in 350M|1_3B|2_6B|6_7B|13B) ;; *) fail "unsupported --model-size: ${OPT[model-size]}" ;; esac
[[ "${OPT[search-budget]}" =~ ^[0-9]+$ ]] && [ "${OPT[search-budget]}" -gt 0 ] || fail "--search-budget must be a positive integer"
[[ "${OPT[global-batch-size]}" =~ ^[0-9]+$ ]] && [ "${OPT[global-batch-size]}" -gt 0 ] || fail "--global-batch-size must be a positive integer"
command -v "$PY" >/dev/null 2>&1 || fail "Python interpreter not found: $PY"

ROOT=$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)
export PYTHONPATH="${ROOT}${PYTHONPATH:+:${PYTHONPATH}}"
PROFILE=$(cd "${OPT[profile-dir]}" 2>/dev/null && pwd) || fail "profile directory does not exist: ${OPT[profile-dir]}"
NODE_DESC=$(cd "$(dirname "${OPT[node-description]}")" 2>/dev/null && pwd)/$(basename "${OPT[node-description]}")
SIZE=${OPT[model-size]}

mapfile -t CONTRACT < <("$PY" -m eth_b200.search.profile_validation --profile-dir "$PROFILE" --model-size "$SIZE" \
    --node-description "$NODE_DESC" --output "${OPT[output]}")
[ "${#CONTRACT[@]}" -eq 4 ] || fail "profile validator returned an incomplete contract"
HARDWARE=${CONTRACT[0]}; MAX_TP=${CONTRACT[1]}; TOTAL_GPUS=${CONTRACT[2]}; NODE_INFO=${CONTRACT[3]}
OUT=$(cd "${OPT[output]}" && pwd)

VIEW="${OUT}/profile_view"
mkdir -p "${VIEW}/${HARDWARE}"
ln -sfn "$PROFILE" "${VIEW}/${HARDWARE}/gpt_${SIZE}"
ln -sfn "${PROFILE}/p2p_intra_node.csv" "${VIEW}/${HARDWARE}/p2p_intra_node.csv"
[ ! -f "${PROFILE}/p2p_inter_node.csv" ] || ln -sfn "${PROFILE}/p2p_inter_node.csv" "${VIEW}/p2p_inter_node.csv"

START=2; END=$TOTAL_GPUS
[ "$END" -le 8 ] || END=8
[ "$END" -ge "$START" ] || fail "search requires at least two GPUs"
mkdir -p "${OUT}/logs" "${OUT}/configs/top_configs" "${OUT}/configs/csv"
cat > "${OUT}/search_plan.txt" <<PLAN
$PY -m eth_b200.search.search --model-name gpt --model-size $SIZE --global-batch-size ${OPT[global-batch-size]} --node-info '$NODE_INFO' --device-json-path <output>/device_info.json --profiled-time-path <output>/profile_view/ --config-save-path <output>/configs/ --max-tp $MAX_TP --time-budget-total ${OPT[search-budget]}
PLAN
if [ "$DRY_RUN" -eq 1 ]; then
    echo "Validated search plan: ${OUT}/search_plan.txt"
    exit 0
fi

STAMP=$(date -u '+%Y-%m-%d-%H-%M-%S')
rm -f "${OUT}/configs/top_configs/"*.json
cd "$ROOT"
"$PY" -m eth_b200.search.search --model-name gpt --model-size "$SIZE" --global-batch-size "${OPT[global-batch-size]}" \
    --micro-batch-size 1 2 4 8 --node-info "$NODE_INFO" --device-json-path "${OUT}/device_info.json" \
    --log-path "${OUT}/logs/" --profiled-time-path "${VIEW}/" --config-save-path "${OUT}/configs/" \
    --config-suffix "$STAMP" --max-num-hops 7 --time-budget-total "${OPT[search-budget]}" --initial-point balance_v1 \
    --num-of-saved-configs 1 --support-comm-predict --comm-revised --op-grain layer \
    --save-prefix "eth_gpt_${SIZE}_budget${OPT[search-budget]}" --max-tp "$MAX_TP" --start-num-stages "$START" \
    --end-num-stages "$END" --min-num-pipeline 1 --max-num-pipeline 100 --reduce-output --add-action-tp-dp-exchange \
    --no-add-action-tp-dp --use-cache --optimal-prune --sort-pipeline --dp-find-pipeline --homo-stage --elastic-time \
    2>&1 | tee "${OUT}/logs/search.log"

mapfile -t TOP < <(find "${OUT}/configs/top_configs" -maxdepth 1 -type f -name '*.json' -print)
[ "${#TOP[@]}" -eq 1 ] || fail "search must produce exactly one top config, found ${#TOP[@]}"
"$PY" -m eth_b200.search.config_adapter --input "${TOP[0]}" --output "${OUT}/gpt_config.json"
echo "Generated GPT config: ${OUT}/gpt_config.json"
