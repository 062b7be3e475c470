#!/usr/bin/env bash
# One HTTP server in front of an 8-GPU tensor-parallel group (rank 0 serves, the other ranks follow), with the
# checkpoint's NextN block as the speculative drafter and the hot-vocabulary draft head.
set -euo pipefail
MODEL=${1:?path of the GGUF file}
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \
    -m hipengine_b200.server --model "$MODEL" --tensor-parallel 8 --port 8000 \
    --max-active-requests 64 --max-context-tokens 32768 --prefix-cache radix \
    --speculative-mtp-serving auto --speculative-candidate-budget 3 --mtp-hot-vocab auto \
    --metrics prometheus --eager-load
