"""Serve the live model weights of a training rank to a co-located sampler process over CUDA IPC
(``megatron/weight_server.py:1-64`` of the reference): a daemon thread listens on ``weight_server_port + rank``
on localhost and answers every connection with a pickled ``{name: (storage IPC handle, dtype, shape, stride,
offset)}`` map, so an inference engine on the same GPU can alias the parameters without a copy."""
from __future__ import annotations

import pickle
import socket
import threading

import torch


def _handles(state_dict):
    out = {}
    for k, v in state_dict.items():
        if not torch.is_tensor(v) or not v.is_cuda:
            continue
        storage = v.untyped_storage()
        out[k] = {"handle": storage._share_cuda_(), "dtype": v.dtype, "shape": tuple(v.shape),
                  "stride": tuple(v.stride()), "offset": v.storage_offset()}
    return out


def _serve(model, port):
    sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    sock.bind(("localhost", port))
    sock.listen(5)
    while True:
        conn, _ = sock.accept()
        try:
            payload = pickle.dumps(_handles(model.module.state_dict()))
            conn.sendall(len(payload).to_bytes(8, "little"))
            conn.sendall(payload)
        finally:
            conn.close()


def start_server(model, ports=6000):
    import torch.distributed as dist
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    port = ports[rank] if isinstance(ports, (list, tuple)) else ports + rank
    t = threading.Thread(target=_serve, args=(model, port), daemon=True)
    t.start()
    return t
