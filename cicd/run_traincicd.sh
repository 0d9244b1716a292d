#!/bin/bash
# Training smoke suite: a few optimizer steps of every model family (or of --model-name) on --gpu-count GPUs, tiny random-init
# models, synthetic data.  Arguments are those of tests/train/run_cicd.py (--model-name, --gpu-count, --cpu, --no-verbose).
set -e
cd "$(dirname "${BASH_SOURCE[0]}")/.."
exec python tests/train/run_cicd.py "$@"
