#!/usr/bin/env python
"""Entry point kept at the repository root, like the reference's ``train.py``:

    torchrun --nproc_per_node=8 train.py --parallel_mode odysseus --seq-length 65536 --model-config llama2-7b
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from odysseus_transformer_b200.train import build_parser, main  # noqa: E402

if __name__ == "__main__":
    main(build_parser().parse_args())
