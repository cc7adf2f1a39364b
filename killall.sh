#!/bin/bash
# Stop a training job started by examples/pretrain/run_pretrain.sh: kills the launcher's process group only
# (the reference's killall.sh pkills every process whose command line mentions recipes/, on every host).
#   bash killall.sh <pid of the torch.distributed.run launcher>
set -euo pipefail
kill -- -"$(ps -o pgid= -p "$1" | tr -d ' ')"
