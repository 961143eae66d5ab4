#!/usr/bin/env bash
# Run the benchmark matrix and write the summary table.
#
#   bash fms_acceleration_b200/benchmarks/run_benchmarks.sh "1 2" "4 8" benchmark_results [SCENARIOS_YAML] [FILTER...]
#
# Arguments: numbers of GPUs, effective batch sizes, result directory, scenario file (default scenarios.yaml),
# then optional scenario names to restrict the run to.
# Environment switches (same meaning as in the reference's scripts/run_benchmarks.sh:38-48):
#   DRY_RUN=true             write command.sh for every experiment and run nothing
#   NO_DATA_PROCESSING=true  keep an existing tokenised cache
#   NO_OVERWRITE=true        keep finished experiments of an earlier run
#   MEMORY_LOGGING=nvidia|huggingface|all   record nvidia-smi memory and/or the allocator's peak
#   DATA_RECORDS=path        JSON/JSONL instruct records to tokenise (otherwise synthetic packed documents)
set -euo pipefail

NUM_GPUS_MATRIX=${1:-"1"}
EFFECTIVE_BS_MATRIX=${2:-"4"}
RESULT_DIR=${3:-"benchmark_results"}
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
SCENARIOS_CONFIG=${4:-"$HERE/scenarios.yaml"}
# a bare file name means one of the scenario files that sit beside this script
if [ ! -f "$SCENARIOS_CONFIG" ] && [ -f "$HERE/$SCENARIOS_CONFIG" ]; then SCENARIOS_CONFIG="$HERE/$SCENARIOS_CONFIG"; fi
shift $(( $# > 4 ? 4 : $# )) || true
SCENARIOS_FILTER=("$@")

DRY_RUN=${DRY_RUN:-false}
NO_DATA_PROCESSING=${NO_DATA_PROCESSING:-false}
NO_OVERWRITE=${NO_OVERWRITE:-false}
MEMORY_LOGGING=${MEMORY_LOGGING:-none}
DATA_CACHE="$RESULT_DIR/data"

if [ -d "$RESULT_DIR" ] && [ "$NO_OVERWRITE" != "true" ] && [ "$DRY_RUN" != "true" ]; then
  echo "result directory $RESULT_DIR exists; set NO_OVERWRITE=true to continue it or remove it first" >&2
  exit 1
fi
mkdir -p "$RESULT_DIR"
export PYTHONPATH="$ROOT${PYTHONPATH:+:$PYTHONPATH}"
python -m pip freeze > "$RESULT_DIR/requirements.txt" 2>/dev/null || true

EXTRA=()
[ "$DRY_RUN" = "true" ] && EXTRA+=(--dry_run)
[ "$NO_OVERWRITE" = "true" ] && EXTRA+=(--no_overwrite)
case "$MEMORY_LOGGING" in nvidia|all) EXTRA+=(--log_nvidia_smi);; esac
[ ${#SCENARIOS_FILTER[@]} -gt 0 ] && EXTRA+=(--run_only_scenarios "${SCENARIOS_FILTER[@]}")

if [ -n "${DATA_RECORDS:-}" ]; then
  OVER=(--overwrite)
  [ "$NO_DATA_PROCESSING" = "true" ] && OVER=()
  DATA_PATH=$(python -m fms_acceleration_b200.benchmarks.data_processing "$DATA_RECORDS" "$DATA_CACHE" --name bench "${OVER[@]}")
  EXTRA+=(--training_data_path "$DATA_PATH")
fi

# shellcheck disable=SC2086
python -m fms_acceleration_b200.benchmarks.benchmark \
  --num_gpus $NUM_GPUS_MATRIX \
  --effective_batch_size_matrix $EFFECTIVE_BS_MATRIX \
  --scenarios_config_path "$SCENARIOS_CONFIG" \
  --defaults_config_path "$HERE/defaults.yaml" \
  --results_output_path "$RESULT_DIR" "${EXTRA[@]}"

if [ "$DRY_RUN" != "true" ]; then
  python -m fms_acceleration_b200.benchmarks.display_bench_results "$RESULT_DIR" \
    --result_file "$RESULT_DIR/benchmarks.csv" \
    --keep_columns torch_dtype framework_config peft_method model_name_or_path num_gpus per_device_train_batch_size \
    --remove_columns training_data_path error_messages acceleration_framework_config_file wall_clock_s
fi
