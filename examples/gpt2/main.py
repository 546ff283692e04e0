"""GPT-2 trainer (reference: example/gpt2/main.cc).  Example:

    python examples/gpt2/main.py --dtype bfloat16 --batch_size 16 --sequence_length 1024 \
        --total_batch_size 16384 --num_iteration 10 --optimizer adamw
    infinitrain_b200/bin/infini_run --nproc_per_node=8 -- python examples/gpt2/main.py --zero_stage 2 ...
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from common.trainer import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main("gpt2"))
