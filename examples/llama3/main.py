"""LLaMA-3 trainer (reference: example/llama3/main.cc).  Example:

    infinitrain_b200/bin/infini_run --nproc_per_node=8 -- python examples/llama3/main.py \
        --model llama3-8b --tensor_parallel 8 --sequence_parallel --dtype bfloat16 \
        --batch_size 1 --sequence_length 2048 --total_batch_size 2048
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common.trainer import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main("llama3"))
