#!/bin/bash
# DCP checkpoint -> HF directory (counterpart of examples/pretrain/convert/convert_muse_to_hf.sh).
#   bash examples/pretrain/convert_to_hf.sh out/8k global_step5000
set -euo pipefail
python -m ksa_b200.tools.convert --dcp_path "$1" --step "$2" --base_model_path ksa_b200/hf --dtype bf16 --remap muse2hf
