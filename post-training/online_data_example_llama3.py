"""Data server for online REINFORCE training: samples completions from the model being trained and scores them.

    python post-training/online_data_example_llama3.py --port 10000 --weight-port 6000 --tokenizer <hf tokenizer>

Protocol (the client is ``gpt_neox_b200.data.online_dataset.OnlineDataset``): the trainer connects to ``--port``,
sends the split name (``train`` / ``valid`` / ``test``) and reads until EOF one pickled dict

    {"prefix": [token ids], "completions": [[token ids], ...], "rewards": [float, ...]}

with ``--num-completions`` sampled continuations of one prompt.  The sampler keeps its weights current by asking the
trainer's weight server (``gpt_neox_b200.weight_server``, port ``--weight-port`` + rank) for the CUDA IPC handles of
the live parameters and re-binding them before every batch, so no checkpoint ever touches disk.

This example uses a Hugging Face model on the same GPU as the sampler and a toy reward (negative length penalty plus
a bonus for ending with the EOS token); swap ``reward_fn`` for a reward model or a verifier.  With an inference engine
such as vLLM the structure is the same: only ``Sampler.generate`` changes.
"""
import argparse
import pickle
import random
import socket


def fetch_ipc_weights(port):
    """{name: tensor aliasing the trainer's parameter} from the weight server on localhost:port."""
    import torch
    with socket.create_connection(("localhost", port), timeout=60) as s:
        n = int.from_bytes(s.recv(8), "little")
        buf = b""
        while len(buf) < n:
            buf += s.recv(min(1 << 20, n - len(buf)))
    out = {}
    for name, d in pickle.loads(buf).items():
        storage = torch.UntypedStorage._new_shared_cuda(*d["handle"])
        t = torch.empty(0, dtype=d["dtype"], device=storage.device)
        t.set_(storage, d["offset"], d["shape"], d["stride"])
        out[name] = t
    return out


class Sampler:
    def __init__(self, model_name, weight_port=None, name_map=None):
        import torch
        from transformers import AutoModelForCausalLM, AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(model_name)
        self.model = AutoModelForCausalLM.from_pretrained(model_name, torch_dtype=torch.bfloat16).cuda().eval()
        self.weight_port, self.name_map = weight_port, name_map or {}

    def refresh(self):
        """Copy the trainer's current parameters (aliased over IPC) into the sampler; ``name_map`` translates
        trainer parameter names to this model's names (e.g. produced by tools/ckpts/convert_neox_to_hf)."""
        if self.weight_port is None:
            return
        live = fetch_ipc_weights(self.weight_port)
        sd = self.model.state_dict()
        for src, dst in self.name_map.items():
            if src in live and dst in sd and sd[dst].shape == live[src].shape:
                sd[dst].copy_(live[src])

    def generate(self, prompt_ids, n, max_new_tokens):
        import torch
        ids = torch.tensor([prompt_ids], device="cuda")
        with torch.no_grad():
            out = self.model.generate(ids, do_sample=True, temperature=1.0, top_p=0.95, num_return_sequences=n,
                                      max_new_tokens=max_new_tokens, pad_token_id=self.tok.eos_token_id)
        return [o[len(prompt_ids):].tolist() for o in out]


def reward_fn(tok, completion):
    ends = len(completion) > 0 and completion[-1] == tok.eos_token_id
    return (1.0 if ends else 0.0) - 0.001 * len(completion)


def serve(args):
    sampler = Sampler(args.tokenizer, args.weight_port)
    prompts = [l.strip() for l in open(args.prompts)] if args.prompts else ["Write a haiku about GPUs.", "Explain NVLink briefly."]
    srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind(("0.0.0.0", args.port))
    srv.listen(8)
    print(f"online data server on :{args.port}", flush=True)
    while True:
        conn, _ = srv.accept()
        try:
            conn.recv(64)                                    # split name; this example serves the same prompts for all
            sampler.refresh()
            text = random.choice(prompts)
            prefix = sampler.tok.apply_chat_template([{"role": "user", "content": text}], add_generation_prompt=True)
            comps = sampler.generate(prefix, args.num_completions, args.max_new_tokens)
            payload = {"prefix": prefix, "completions": comps, "rewards": [reward_fn(sampler.tok, c) for c in comps]}
            conn.sendall(pickle.dumps(payload))
        finally:
            conn.close()


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--port", type=int, default=10000)
    ap.add_argument("--weight-port", type=int, default=None, help="trainer weight-server port (omit to keep static weights)")
    ap.add_argument("--tokenizer", default="meta-llama/Meta-Llama-3-8B-Instruct", help="HF model / tokenizer id")
    ap.add_argument("--prompts", default=None, help="text file with one prompt per line")
    ap.add_argument("--num-completions", type=int, default=4)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    serve(ap.parse_args())
