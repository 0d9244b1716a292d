#!/usr/bin/env bash
# One node, one process per GPU: bash examples/run.sh examples/load_from_pretrained_example.yaml [key=value ...]
set -euo pipefail
CONFIG=${1:-examples/load_from_pretrained_example.yaml}
shift || true
python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPU:-8}" --master-addr 127.0.0.1 --master-port "${PORT:-12355}" \
  -m lmms_engine.launch.cli config_yaml="$CONFIG" "$@"
