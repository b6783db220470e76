#!/usr/bin/env python
"""Train a model: ``./deepy.py train.py <configs>`` (worker entry point, ``train.py:22-31`` of the reference)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(input_args=None, overwrite_values=None):
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.training import pretrain
    neox_args = NeoXArgs.consume_neox_args(input_args=input_args, overwrite_values=overwrite_values)
    neox_args.configure_distributed_args()
    neox_args.build_tokenizer()          # also fixes padded_vocab_size
    neox_args.initialize_tensorboard_writer()
    neox_args.initialize_comet()
    pretrain(neox_args=neox_args)


if __name__ == "__main__":
    main()
