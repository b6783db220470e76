#!/usr/bin/env python
"""Launcher: ``./deepy.py <script.py> [-d confdir] cfg1.yml cfg2.yml ...``

Parses the YAML configs once, then starts one worker process per GPU (this host) or hands the same
command line to ``pdsh`` / ``mpirun`` / ``srun`` for every host of the hostfile.  Every worker receives the
resolved configuration as a base64 JSON blob (``--megatron_config``), so ranks cannot disagree.
Same command-line surface as the reference's ``deepy.py:21-37`` (which delegates to DeepSpeed's runner).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(input_args=None):
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.launcher import launch
    neox_args = NeoXArgs.consume_deepy_args(input_args)
    return launch(neox_args)


if __name__ == "__main__":
    sys.exit(main())
