#!/bin/bash
# Online REINFORCE on one 8-GPU node: GPUs 0-3 train (TP 4), GPUs 4 and 5 run one sampler / data server each.
# The trainer serves its live weights over CUDA IPC (serve_model_weights), the samplers pull them before every batch.
set -euo pipefail
CUDA_VISIBLE_DEVICES=4 python post-training/online_data_example_llama3.py --port 10000 --weight-port 6000 &
CUDA_VISIBLE_DEVICES=5 python post-training/online_data_example_llama3.py --port 10001 --weight-port 6000 &
CUDA_VISIBLE_DEVICES=0,1,2,3 python deepy.py train.py post-training/configs/llama3-8b-reinforce.yml
kill %1 %2
