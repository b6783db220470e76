"""Autoregressive text generation (role of ``megatron/text_generation_utils.py``).

``stream_tokens`` is a generator that adds one token per iteration to every unfinished row of the
batch: prompts are right-padded to a common length (NOT to ``seq_length``: the kernels need no
fixed-size mask), the first forward consumes the shortest prompt prefix and fills the per-layer
key/value caches, later forwards feed one token.  Sampling: greedy when ``temperature == top_k == top_p ==
0``, otherwise temperature scaling, top-k / nucleus filtering (vectorised over the batch) and a
multinomial draw.  With pipeline parallelism the last stage samples and broadcasts the token to the
other stages; prompts are broadcast from tensor-parallel rank 0.
"""
from __future__ import annotations

import copy
import json
import time
from typing import List, Union

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F

from .parallel import mpu
from .utils import get_ltor_masks_and_position_ids, is_mp_rank_0, print_rank_0


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def _dist_on():
    return dist.is_available() and dist.is_initialized()


def get_batch(neox_args, context_tokens: torch.Tensor):
    tokens = context_tokens.contiguous().to(_dev())
    attention_mask, _, position_ids = get_ltor_masks_and_position_ids(
        data=tokens, eod_token=neox_args.tokenizer.eod, eod_mask_loss=neox_args.eod_mask_loss)
    return tokens, attention_mask, position_ids


def pad_batch(context_tokens: List[List[int]], pad_id: int, pad_len: int, truncate: bool = False):
    lengths = []
    for i, tokens in enumerate(context_tokens):
        n = len(tokens)
        if n < pad_len:
            tokens.extend([pad_id] * (pad_len - n))
        elif n > pad_len:
            if not truncate:
                raise ValueError("context_length is bigger than to be padded length")
            context_tokens[i] = tokens[:pad_len]
            n = pad_len
        lengths.append(n)
    return context_tokens, lengths


def filter_logits(logits, top_k=0, top_p=0.0, filter_value=-float("Inf")):
    """Top-k then nucleus filtering, all rows at once (the reference loops over the batch in Python,
    ``text_generation_utils.py:120-122``).  On the GPU one kernel does both filters without sorting."""
    if logits.is_cuda and logits.dim() == 2 and filter_value == -float("Inf") and (top_k > 0 or 0.0 < top_p < 1.0) \
            and logits.shape[-1] * 4 <= 224 * 1024:
        import ctypes
        from .ops import native
        if native.available() and native.lib().has("neox_sample_filter"):
            x = logits.float().contiguous()
            out = torch.empty_like(x)
            rc = native.lib().neox_sample_filter(native.ptr(x), native.ptr(out), x.shape[0], x.shape[1], int(top_k),
                                                 ctypes.c_float(top_p), ctypes.c_void_p(native.stream_ptr()))
            native.check(rc, "neox_sample_filter")
            return out.to(logits.dtype)
    if top_k > 0:
        kth = torch.topk(logits, top_k)[0][..., -1, None]
        logits = logits.masked_fill(logits < kth, filter_value)
    if top_p > 0.0:
        sorted_logits, sorted_idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(sorted_logits, dim=-1), dim=-1)
        remove = cum > top_p
        remove[..., 1:] = remove[..., :-1].clone()      # keep the first token that crosses the threshold
        remove[..., 0] = False
        mask = torch.zeros_like(remove).scatter(-1, sorted_idx, remove)
        logits = logits.masked_fill(mask, filter_value)
    return logits


def switch(val1, val2, boolean):
    boolean = boolean.type_as(val1)
    return (1 - boolean) * val1 + boolean * val2


def forward_model(model, model_inputs, is_pipe_parallel=False, pipe_parallel_size=0, timers=None):
    """Logits ``[b, s, V]`` for one forward (``None`` on pipeline stages other than the last)."""
    if not is_pipe_parallel:
        out = model.module(model_inputs)
        return out[0] if isinstance(out, tuple) else out
    # the pipeline engine wants a (inputs, labels) pair per micro-batch; message shapes change with the
    # sequence length, so the cached shapes are dropped before every call
    tokens, position_ids, attention_mask = model_inputs
    model.reset_activation_shape()
    batch_fn, model.batch_fn = model.batch_fn, None
    try:
        _, logits = model.eval_batch(iter([((tokens, position_ids, attention_mask), None)]), return_logits=True,
                                     num_micro_batches=1)
    finally:
        model.batch_fn = batch_fn
    return logits


def broadcast_terminate_signal(terminate_runs: int):
    t = torch.tensor([terminate_runs], dtype=torch.long, device=_dev())
    if _dist_on() and mpu.get_model_parallel_world_size() > 1:
        dist.broadcast(t, mpu.get_model_parallel_src_rank(), group=mpu.get_model_parallel_group())
    return int(t[0].item())


def stop_tokens_in_completion(stop_tokens, context_tokens, batch_index, current_index):
    if stop_tokens is None:
        return False
    for seq in stop_tokens:
        n = len(seq)
        if current_index + 1 >= n and bool((context_tokens[batch_index, current_index + 1 - n:current_index + 1]
                                            == seq).all()):
            return True
    return False


class GraphDecoder:
    """Token-by-token decoding with a fixed-capacity key/value cache, replayed from a CUDA graph.

    A decoding step of the ordinary cached path launches a few dozen small kernels per layer whose shapes change with
    the position (the cache grows), so it is bound by launch overhead and cannot be captured.  Here every attention
    layer owns a ``[2, capacity, batch, heads, d]`` buffer and reads the current position from a device scalar: the
    step's launch sequence is identical for every token, is captured once after the prompt pass and replayed.  On a
    machine without CUDA (or with ``capture=False``) the same static-cache step runs eagerly, which is how its
    numerics are tested.  The reference decodes with ``torch.cat`` caches and eager launches
    (``megatron/text_generation_utils.py:198-405``)."""

    def __init__(self, neox_args, model, batch_size, capacity, capture=None):
        self.model = model
        dev = _dev()
        self.attn = [m for m in model.module.modules() if hasattr(m, "static_kv") and hasattr(m, "static_cache_supported")]
        self.supported = bool(self.attn) and all(m.static_cache_supported() and m.use_cache for m in self.attn)
        self.capture = (torch.cuda.is_available() if capture is None else capture) and self.supported
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.tokens = torch.zeros(batch_size, 1, dtype=torch.long, device=dev)
        self.position_ids = torch.zeros(batch_size, 1, dtype=torch.long, device=dev)
        self.graph, self.logits, self.steps = None, None, 0
        self.caches = []
        if self.supported:
            dt = neox_args.params_dtype
            self.caches = [torch.zeros(2, capacity, batch_size, m.num_kv_heads_per_partition,
                                       m.hidden_size_per_attention_head, dtype=dt, device=dev) for m in self.attn]

    @classmethod
    def for_model(cls, neox_args, model, batch_size):
        """The decoder of ``model`` for this batch size, kept on the model between generation calls so the captured
        graph (which holds the addresses of the caches and of the static inputs) is reused.  Capacity is the model's
        sequence length: every request fits."""
        pool = model.__dict__.setdefault("_graph_decoders", {})
        dec = pool.get(batch_size)
        if dec is None:
            dec = pool[batch_size] = cls(neox_args, model, batch_size, neox_args.seq_length)
        return dec

    def attach(self):
        """Hand the caches to the attention layers for one generation call (an empty cache: the prompt pass fills it)."""
        for m, buf in zip(self.attn, self.caches):
            m.static_kv, m.static_pos, m.static_filled = buf, self.pos, False

    def close(self):
        """Take the caches back (the layers return to the growing-cache path); the graph stays valid for the next call."""
        for m in self.attn:
            m.static_kv, m.static_pos, m.static_filled = None, None, False

    def prefill(self, tokens, position_ids):
        """The prompt pass (eager): fills the caches; returns the logits of the prompt."""
        out = self.model.module((tokens, position_ids, None))
        return out[0] if isinstance(out, tuple) else out

    def _forward(self):
        out = self.model.module((self.tokens, self.position_ids, None))
        return out[0] if isinstance(out, tuple) else out

    def step(self, tokens, position_ids, index):
        """Logits ``[b, 1, V]`` for the token at sequence position ``index`` given everything before it."""
        self.tokens.copy_(tokens)
        self.position_ids.copy_(position_ids)
        self.pos.fill_(index)
        self.steps += 1
        if not self.capture:
            return self._forward()
        if self.graph is None:
            # warm up on a side stream (lazy allocations, descriptor caches), then capture the very same step:
            # re-running a step is harmless, it rewrites the same cache slot with the same values
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._forward()
            torch.cuda.current_stream().wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.logits = self._forward()
        self.graph.replay()
        return self.logits


def stream_tokens(neox_args, model, context_tokens: List[List[int]], eos_token_id: int = None,
                  maximum_tokens: int = None, recompute: bool = False, temperature: float = 0.0, top_k: int = 0,
                  top_p: float = 0.0, stop_tokens=None):
    """Yields ``(tokens, generation_start_index, generation_end_index, logits, is_done)`` after every new token."""
    model.eval()
    longest = max(len(c) for c in context_tokens)
    budget = maximum_tokens or (neox_args.seq_length - longest - 1)
    total_len = min(neox_args.seq_length, longest + budget)
    context_tokens, context_lengths = pad_batch(copy.deepcopy(context_tokens), pad_id=neox_args.tokenizer.eod,
                                                pad_len=total_len, truncate=True)
    dev = _dev()
    context_tokens = torch.tensor(context_tokens, dtype=torch.long, device=dev)
    if stop_tokens:
        if len(stop_tokens) > 0 and not isinstance(stop_tokens[0], (list, tuple)):
            stop_tokens = [stop_tokens]
        stop_tokens = [torch.tensor(s, dtype=torch.long, device=dev) for s in stop_tokens]
    start_index = torch.tensor(context_lengths, dtype=torch.long, device=dev)
    if _dist_on() and mpu.get_model_parallel_world_size() > 1:
        dist.broadcast(context_tokens, mpu.get_model_parallel_src_rank(), group=mpu.get_model_parallel_group())
        dist.broadcast(start_index, mpu.get_model_parallel_src_rank(), group=mpu.get_model_parallel_group())
    context_tokens, attention_mask, position_ids = get_batch(neox_args, context_tokens)
    eos_token_id = eos_token_id if eos_token_id is not None else neox_args.tokenizer.eod
    batch_size = context_tokens.size(0)
    index = int(start_index.min().item())
    first_index = index
    last_index = min(total_len - 1, index + budget - 1)
    if hasattr(model.module, "clear_cache"):
        model.module.clear_cache()
    decoder = None
    if (getattr(neox_args, "cuda_graph_decode", False) and not recompute and not neox_args.is_pipe_parallel
            and mpu.get_model_parallel_world_size() == 1):
        decoder = GraphDecoder.for_model(neox_args, model, batch_size)
        if decoder.supported:
            decoder.attach()
        else:
            decoder = None
    try:
        yield from _decode_loop(neox_args, model, decoder, context_tokens, position_ids, attention_mask, start_index,
                                index, first_index, last_index, budget, batch_size, eos_token_id, stop_tokens,
                                recompute, temperature, top_k, top_p, dev)
    finally:
        if decoder is not None:
            decoder.close()
            if hasattr(model.module, "clear_cache"):
                model.module.clear_cache()


def _decode_loop(neox_args, model, decoder, context_tokens, position_ids, attention_mask, start_index, index,
                 first_index, last_index, budget, batch_size, eos_token_id, stop_tokens, recompute, temperature, top_k,
                 top_p, dev):
    with torch.no_grad():
        is_done = torch.zeros(batch_size, dtype=torch.bool, device=dev)
        end_index = torch.full((batch_size,), -1, dtype=torch.long, device=dev)
        gen_logits = torch.empty(max(budget, 1), neox_args.padded_vocab_size, dtype=torch.float, device=dev) \
            if neox_args.return_logits else None
        while index <= last_index:
            if recompute:
                logits = forward_model(model, (context_tokens[:, :index], position_ids[:, :index], attention_mask),
                                       neox_args.is_pipe_parallel)
                tok_logits = logits[:, index - 1, :] if logits is not None else None
            else:
                if index == first_index:
                    use_t, use_p = context_tokens[:, :index], position_ids[:, :index]
                else:
                    use_t = context_tokens[:, index - 1].view(batch_size, -1)
                    use_p = position_ids[:, index - 1].view(batch_size, -1)
                if decoder is not None:
                    logits = decoder.prefill(use_t, use_p) if index == first_index else \
                        decoder.step(use_t, use_p, index - 1)
                else:
                    logits = forward_model(model, (use_t, use_p, attention_mask), neox_args.is_pipe_parallel)
                tok_logits = logits[:, -1].view(batch_size, -1).contiguous() if logits is not None else None
            if tok_logits is not None:
                tok_logits = tok_logits[:, : neox_args.padded_vocab_size]
                if temperature == 0.0 and top_k == 0 and top_p == 0.0:
                    new_tokens = torch.argmax(tok_logits, dim=-1).view(-1)
                else:
                    tok_logits = tok_logits.float()
                    if temperature > 0.0:
                        tok_logits = tok_logits / temperature
                    tok_logits = filter_logits(tok_logits, top_k=top_k, top_p=top_p)
                    new_tokens = torch.multinomial(F.softmax(tok_logits, dim=-1), num_samples=1).view(-1)
                if gen_logits is not None:
                    gen_logits[index - first_index] = tok_logits[0].float()
            if neox_args.is_pipe_parallel and mpu.get_pipe_parallel_world_size() > 1:
                src = mpu.get_pipe_parallel_ranks()[-1]
                new_tokens = new_tokens if tok_logits is not None else torch.zeros(batch_size, dtype=torch.long,
                                                                                 device=dev)
                dist.broadcast(new_tokens, src=src, group=mpu.get_pipe_parallel_group())
            started = start_index <= index
            context_tokens[:, index] = switch(context_tokens[:, index].view(-1), new_tokens, started)
            done_now = (new_tokens == eos_token_id) & started
            is_done = is_done | done_now
            if stop_tokens:
                hit = torch.tensor([stop_tokens_in_completion(stop_tokens, context_tokens, b, index)
                                    for b in range(batch_size)], dtype=torch.bool, device=dev)
                is_done = is_done | hit
            end_index[started & ~is_done] = index
            index += 1
            yield context_tokens, start_index, end_index, gen_logits, is_done
            if bool(is_done.all()):
                break


def generate_samples_from_prompt(neox_args, model, text: Union[List[str], str], eos_token_id: int = None,
                                 maximum_tokens: int = 64, recompute: bool = False, temperature: float = 0.0,
                                 top_k: int = 0, top_p: float = 0.0, stop_tokens=None):
    """One dict per prompt: ``context``, ``text``, ``length``, ``finished``, ``message``, ``duration_seconds``."""
    eos_token_id = eos_token_id if eos_token_id is not None else neox_args.tokenizer.eod
    texts = [text] if isinstance(text, str) else list(text)
    results = []
    for idx in range(len(texts) + 1):
        terminate = 0
        raw = ""
        tokens = []
        if is_mp_rank_0():
            if idx == len(texts):
                terminate = 1
            else:
                raw = texts[idx]
                tokens = neox_args.tokenizer.tokenize(raw) if raw != "" else [eos_token_id]
                if len(tokens) == 0:
                    tokens = [eos_token_id]
                if len(tokens) >= neox_args.seq_length // 2:
                    print_rank_0(f"\nWarning! Context length {len(tokens)} is long; please give smaller context "
                                 "(half of the sequence length or less)!")
        elif idx == len(texts):
            terminate = 1
        if not is_mp_rank_0():
            tokens = neox_args.tokenizer.tokenize("EMPTY TEXT")
        if broadcast_terminate_signal(terminate) == 1:
            return results
        t0 = time.time()
        last = None
        for last in stream_tokens(neox_args=neox_args, model=model, context_tokens=[tokens], eos_token_id=eos_token_id,
                                  maximum_tokens=maximum_tokens, recompute=recompute, temperature=temperature,
                                  top_k=top_k, top_p=top_p, stop_tokens=stop_tokens):
            pass
        if last is None:
            continue
        batch_tokens, starts, ends, logits, done = last
        toks = batch_tokens.cpu().numpy().tolist()
        for t, s, e, d in zip(toks, starts.cpu().numpy().tolist(), ends.cpu().numpy().tolist(),
                              done.cpu().numpy().tolist()):
            if e >= s:
                gen = t[s:e + 1]
                try:
                    out_text, message = neox_args.tokenizer.detokenize(gen), None
                except KeyError:
                    out_text, message = None, "WARNING: generated token which doesn't exist."
            else:
                gen, out_text, message = [], None, "WARNING: text generation did not start; try different batching or adjust parameters"
            if is_mp_rank_0():
                item = {"context": raw, "text": out_text, "length": len(gen), "finished": bool(d), "message": message,
                        "duration_seconds": float(time.time() - t0)}
                if neox_args.return_logits and logits is not None:
                    item["logits"] = logits[: len(gen)].cpu().numpy().tolist()
                results.append(item)
    return results


def _write(results, output_file):
    if output_file is not None and is_mp_rank_0():
        with open(output_file, "w") as fh:
            for item in results:
                fh.write(json.dumps(item) + "\n")


def generate_samples_input_from_file(neox_args, model, input_file, output_file=None, eos_token_id: int = None,
                                     maximum_tokens: int = 64, prompt_end: str = "\n", recompute: bool = False,
                                     temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0):
    print_rank_0(f"generate_samples_input_from_file() loading input from {input_file}")
    with open(input_file, "r", encoding="utf-8") as fh:
        prompts = [p.strip() for p in fh.read().split(neox_args.prompt_end or prompt_end)]
    prompts = [p for p in prompts if p]
    assert len(prompts) > 0
    if is_mp_rank_0() and output_file is None:
        output_file = str(input_file) + ".output.jsonl"
        print_rank_0(f"generate_samples_input_from_file() setting default output file to {output_file}")
    results = generate_samples_from_prompt(neox_args=neox_args, model=model, text=prompts, eos_token_id=eos_token_id,
                                           maximum_tokens=maximum_tokens, recompute=recompute, temperature=temperature,
                                           top_k=top_k, top_p=top_p)
    _write(results, output_file)
    print_rank_0("generate_samples_input_from_file() done")
    return results


def generate_samples_unconditional(neox_args, model, number_of_samples: int = 10, output_file=None,
                                   eos_token_id: int = None, maximum_tokens: int = 64, recompute: bool = False,
                                   temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0):
    print_rank_0("generate_samples_unconditional() generating...")
    results = generate_samples_from_prompt(neox_args=neox_args, model=model, text=[""] * number_of_samples,
                                           eos_token_id=eos_token_id, maximum_tokens=maximum_tokens,
                                           recompute=recompute, temperature=temperature, top_k=top_k, top_p=top_p)
    _write(results, output_file)
    print_rank_0("generate_samples_unconditional() done")
    return results


def generate_samples_interactive(neox_args, model, maximum_tokens: int = 64, prompt_end: str = "\n",
                                 eos_token_id: int = None, recompute: bool = False, temperature: float = 0.0,
                                 top_k: int = 0, top_p: float = 0.0):
    while True:
        if _dist_on():
            dist.barrier(group=mpu.get_model_parallel_group())
        terminate, raw, tokens = 0, "", []
        if is_mp_rank_0():
            try:
                raw = input("Context prompt >>> ")
            except EOFError:
                terminate = 1
            tokens = neox_args.tokenizer.tokenize(raw) if raw else [neox_args.tokenizer.eod]
            if len(tokens) >= neox_args.seq_length // 2:
                print_rank_0("\nContext is too long; please give a shorter one")
                continue
        else:
            tokens = neox_args.tokenizer.tokenize("EMPTY TEXT")
        if broadcast_terminate_signal(terminate) == 1:
            return
        for batch_tokens, starts, ends, _, done in stream_tokens(
                neox_args=neox_args, model=model, context_tokens=[tokens], eos_token_id=eos_token_id,
                maximum_tokens=maximum_tokens, recompute=recompute, temperature=temperature, top_k=top_k, top_p=top_p):
            if is_mp_rank_0():
                gen = batch_tokens[0].cpu().numpy().tolist()[int(starts[0]):int(ends[0]) + 1]
                print_rank_0("Generated Text: " + neox_args.tokenizer.detokenize(gen))
        if is_mp_rank_0():
            input("\n<press enter to continue>")


def get_logp(logits, labels, force_fp32=False):
    if force_fp32:
        logits = logits.float()
    return torch.gather(logits.log_softmax(dim=-1), dim=2, index=labels.unsqueeze(2)).squeeze(2)


def precompute_logits(neox_args, model):
    """Write the reference model's per-token log-probabilities for every training document next to the
    dataset as ``<prefix>_<precompute_model_name>.bin/.idx`` (consumed by DPO / KTO as ``ref`` data)."""
    from .data.indexed_dataset import MMapIndexedDatasetBuilder, make_dataset
    assert not neox_args.is_pipe_parallel or mpu.get_pipe_parallel_world_size() == 1, \
        "precompute is only implemented for a single pipeline stage"
    model.eval()
    paths = list(neox_args.train_data_paths or []) + list(neox_args.pos_train_data_paths or []) \
        + list(neox_args.neg_train_data_paths or [])
    labels_paths = list(neox_args.train_label_data_paths or []) + list(neox_args.pos_train_label_data_paths or []) \
        + list(neox_args.neg_train_label_data_paths or [])
    dp_rank, dp_world = mpu.get_data_parallel_rank(), mpu.get_data_parallel_world_size()
    for pi, prefix in enumerate(paths):
        ds = make_dataset(prefix, neox_args.data_impl, True)
        out_prefix = f"{prefix}_{neox_args.precompute_model_name}"
        builder = None
        if dp_rank == 0 and is_mp_rank_0():
            builder = MMapIndexedDatasetBuilder(out_prefix + ".bin", dtype=np.float32)
        for i in range(len(ds)):
            owner = i % dp_world
            tokens = np.asarray(ds[i], dtype=np.int64)[: neox_args.seq_length + 1]
            t = torch.from_numpy(tokens.astype(np.int64)).unsqueeze(0).to(_dev())
            logp = torch.zeros(1, max(t.shape[1] - 1, 1), device=_dev())
            if owner == dp_rank and t.shape[1] > 1:
                inp, lab = t[:, :-1].contiguous(), t[:, 1:].contiguous()
                pos = torch.arange(inp.shape[1], device=_dev()).unsqueeze(0)
                with torch.no_grad():
                    out = model.module((inp, pos, None))
                    logits = out[0] if isinstance(out, tuple) else out
                    from .parallel import mappings as M
                    full = logits if getattr(model.module, "parallel_output", True) is False else \
                        M.gather_from_model_parallel_region(logits)
                    logp = get_logp(full[..., : neox_args.padded_vocab_size], lab, True)
            if _dist_on() and dp_world > 1:
                dist.broadcast(logp, src=mpu.get_data_parallel_ranks()[owner], group=mpu.get_data_parallel_group())
            if builder is not None:
                builder.add_item(np.concatenate([logp[0].float().cpu().numpy(), np.zeros(1, dtype=np.float32)]))
                builder.end_document()
        if builder is not None:
            builder.finalize(out_prefix + ".idx")
        if _dist_on():
            dist.barrier()
    print_rank_0("precompute_logits() done")
