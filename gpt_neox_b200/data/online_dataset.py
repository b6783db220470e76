"""Dataset fed by an online sampling server (REINFORCE-style training,
``megatron/data/online_dataset.py:29-128``): each request returns a pickled
``{"prefix": [...], "completions": [[...], ...], "rewards": [...]}`` batch; rewards are centred with a
leave-one-out baseline or a moving average, and every completion becomes one sample with the prompt positions
labelled -100."""
from __future__ import annotations

import pickle
import socket
import time
from collections import deque

import numpy as np
import torch


class OnlineDataset(torch.utils.data.Dataset):
    def __init__(self, num_samples, seq_length, leave_one_out=False, data_split="train", dataserver_ips="localhost",
                 dataserver_ports=10000):
        self.num_samples, self.seq_length, self.leave_one_out = num_samples, seq_length, leave_one_out
        self.data_split = data_split
        self.ips = dataserver_ips if isinstance(dataserver_ips, (list, tuple)) else [dataserver_ips]
        self.ports = dataserver_ports if isinstance(dataserver_ports, (list, tuple)) else [dataserver_ports]
        self.queue = deque()
        self.reward_window = deque(maxlen=100)
        self._rr = 0

    def __len__(self):
        return self.num_samples

    def _fetch(self):
        ip = self.ips[self._rr % len(self.ips)]
        port = self.ports[self._rr % len(self.ports)]
        self._rr += 1
        while True:
            try:
                with socket.create_connection((ip, port), timeout=60) as s:
                    s.sendall(self.data_split.encode())
                    buf = b""
                    while True:
                        chunk = s.recv(1 << 20)
                        if not chunk:
                            break
                        buf += chunk
                return pickle.loads(buf)
            except (ConnectionRefusedError, socket.timeout):
                time.sleep(1.0)

    def _fill(self):
        batch = self._fetch()
        rewards = np.asarray(batch["rewards"], dtype=np.float32)
        if self.leave_one_out and len(rewards) > 1:
            baseline = (rewards.sum() - rewards) / (len(rewards) - 1)
        else:
            self.reward_window.extend(rewards.tolist())
            baseline = np.full_like(rewards, float(np.mean(self.reward_window)))
        centred = rewards - baseline
        prefix = list(batch["prefix"])
        for comp, rw, raw in zip(batch["completions"], centred, rewards):
            toks = (prefix + list(comp))[: self.seq_length + 1]
            n = len(toks)
            text = np.zeros(self.seq_length + 1, dtype=np.int64)
            text[:n] = toks
            label = np.full(self.seq_length + 1, -100, dtype=np.int64)
            label[len(prefix):n] = toks[len(prefix):n]
            self.queue.append({"text": text, "label": label, "reward": np.full(self.seq_length + 1, rw, np.float32),
                               "raw_reward": np.float32(raw)})

    def __getitem__(self, idx):
        while not self.queue:
            self._fill()
        return self.queue.popleft()
