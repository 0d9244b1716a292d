#!/usr/bin/env bash
# One node, one process per GPU.
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "${PORT:-29500}" \
  -m lmms_engine.launch.cli config_yaml=examples/qwen2_5_llm/example_config.yaml "$@"
