# Training image for B200 (sm_100a) nodes.  The CUDA libraries are compiled ahead of time for sm_100a only, so the
# image starts training without a JIT step (python -m gpt_neox_b200.ops.build is what __graft_entry__.build() runs).
FROM nvcr.io/nvidia/pytorch:25.03-py3

ENV DEBIAN_FRONTEND=noninteractive
RUN apt-get update -y && apt-get install -y --no-install-recommends git pdsh openssh-server openssh-client sudo tmux && \
    rm -rf /var/lib/apt/lists/* && mkdir -p /run/sshd && \
    echo 'export PDSH_RCMD_TYPE=ssh' >> /etc/bash.bashrc

WORKDIR /workspace/gpt-neox-b200
COPY requirements/ requirements/
RUN python -m pip install --no-cache-dir -r requirements/requirements.txt
COPY . .
# C ABI kernels (nvcc -gencode arch=compute_100a,code=sm_100a) and the host C++ helpers
RUN python -m gpt_neox_b200.ops.build

ENV PYTHONPATH=/workspace/gpt-neox-b200
CMD ["bash"]
