#!/usr/bin/env bash
# Launches training with one process per GPU:
#   bash run.sh experiment=cosmos3/bidirectional [overrides...]
# Environment: NNODES NODE_RANK MASTER_ADDR MASTER_PORT NPROC_PER_NODE WM_PYTHON
# WM_RUNTIME_CACHE_ROOT.  A .env file beside the repository root supplies machine-local
# settings without overriding variables that are already exported.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"

if [[ -f .env ]]; then
  while IFS='=' read -r key value; do
    [[ -z "${key}" || "${key}" == \#* ]] && continue
    key="${key#export }"
    if [[ -z "${!key+x}" ]]; then export "${key}=${value}"; fi
  done < .env
fi

PYTHON="${WM_PYTHON:-python}"
NNODES="${NNODES:-1}"
NPROC="${NPROC_PER_NODE:-gpu}"
CACHE_ROOT="${WM_RUNTIME_CACHE_ROOT:-${TMPDIR:-/tmp}/agentgarten_b200-${USER:-user}}"
mkdir -p "${CACHE_ROOT}/nccl"

# flight recorder / desync diagnostics of the process-group watchdog
export TORCH_FR_BUFFER_SIZE="${TORCH_FR_BUFFER_SIZE:-20000}"
export TORCH_NCCL_DUMP_ON_TIMEOUT="${TORCH_NCCL_DUMP_ON_TIMEOUT:-1}"
export TORCH_NCCL_ENABLE_MONITORING="${TORCH_NCCL_ENABLE_MONITORING:-1}"
export TORCH_NCCL_DESYNC_DEBUG="${TORCH_NCCL_DESYNC_DEBUG:-1}"
export TORCH_NCCL_DEBUG_INFO_TEMP_FILE="${TORCH_NCCL_DEBUG_INFO_TEMP_FILE:-${CACHE_ROOT}/nccl/trace_rank_}"

"${PYTHON}" -m agentgarten_b200.build >/dev/null

if [[ "${NNODES}" == "1" && -z "${MASTER_ADDR:-}" ]]; then
  RENDEZVOUS=(--standalone --local-addr 127.0.0.1)
else
  RENDEZVOUS=(--nnodes "${NNODES}" --node-rank "${NODE_RANK:-0}"
              --master-addr "${MASTER_ADDR:-127.0.0.1}" --master-port "${MASTER_PORT:-29500}")
fi
exec "${PYTHON}" -m torch.distributed.run "${RENDEZVOUS[@]}" --nproc-per-node "${NPROC}" \
  -m agentgarten_b200.train "$@"
