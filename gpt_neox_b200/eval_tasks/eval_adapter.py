"""Adapter between a trained engine and lm-evaluation-harness (``eval_tasks/eval_adapter.py:36-538`` of the
reference).  The scoring logic is harness independent and usable on its own:

* ``loglikelihood(requests)``: for (context, continuation) string pairs returns (sum log-prob of the continuation,
  whether it is the greedy continuation); requests are length-sorted, batched, left-truncated to ``max_length``,
  sharded over data-parallel ranks and gathered back;
* ``loglikelihood_rolling(texts)``: whole-document log-likelihood in windows of ``max_length``;
* ``generate_until(requests)``: greedy generation until one of the stop strings.

``run_eval_harness`` wires it into ``lm_eval.evaluator`` when the package is installed.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel import mappings as M
from ..parallel import mpu
from ..text_generation import generate_samples_from_prompt
from ..utils import print_rank_0


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


class EvalHarnessAdapter:
    def __init__(self, model, forward_step_fn, neox_args, batch_size=None):
        self.model, self.neox_args, self.tokenizer = model, neox_args, neox_args.tokenizer
        self._forward_step_fn = forward_step_fn
        self.cache_hook = None
        self._device = _dev()
        self._eot_token_id = neox_args.tokenizer.eod_id if hasattr(neox_args.tokenizer, "eod_id") else neox_args.tokenizer.eod
        self._max_length = neox_args.max_position_embeddings // 2 if neox_args.seq_length is None else neox_args.seq_length
        self._max_gen_toks = 128
        self._vocab_size = neox_args.padded_vocab_size
        self.is_main = (neox_args.rank or 0) == 0
        self.is_local_main = (neox_args.local_rank or 0) == 0
        self.is_model_parallel = neox_args.model_parallel_size > 1
        self.is_pipe_parallel = bool(neox_args.is_pipe_parallel)
        self.is_data_parallel = mpu.get_data_parallel_world_size() > 1
        self.is_last_stage = True if not self.is_pipe_parallel else model.is_last_stage()
        self.dp_world_size, self.dp_rank = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
        self.dp_group = mpu.get_data_parallel_group()
        self._batch_size = batch_size or (neox_args.batch_size * self.dp_world_size)

    # ------------------------------------------------------------------ properties the harness reads
    @property
    def vocab_size(self):
        return self._vocab_size

    @property
    def eot_token_id(self):
        return self._eot_token_id

    @property
    def max_length(self):
        return self._max_length

    @property
    def max_gen_toks(self):
        return self._max_gen_toks

    @property
    def batch_size(self):
        return self._batch_size

    @property
    def device(self):
        return self._device

    def tok_encode(self, string, **kw):
        return self.tokenizer.tokenize(string)

    def tok_decode(self, tokens, **kw):
        return self.tokenizer.detokenize(list(tokens))

    # ------------------------------------------------------------------ model call
    def _model_call(self, inps):
        """inps: [batch, seq] token ids on this data-parallel rank -> logits [batch, seq, vocab] (None off the last stage)."""
        inps = inps.to(self._device)
        pos = torch.arange(inps.shape[1], device=self._device).unsqueeze(0).expand_as(inps)
        with torch.no_grad():
            if self.is_pipe_parallel:
                self.model.reset_activation_shape()
                bf, self.model.batch_fn = self.model.batch_fn, None
                try:
                    _, logits = self.model.eval_batch(iter([((inps, pos, None), None)]), return_logits=True,
                                                      num_micro_batches=1)
                finally:
                    self.model.batch_fn = bf
            else:
                out = self.model.module((inps, pos, None))
                logits = out[0] if isinstance(out, tuple) else out
                if getattr(self.model.module, "parallel_output", False) and self.is_model_parallel:
                    logits = M.gather_from_model_parallel_region(logits)
        return logits[..., : self._vocab_size] if logits is not None else None

    def _dp_scatter(self, inps):
        """Pad the batch to a multiple of the DP size and keep this rank's slice; returns (slice, padded rows)."""
        b = inps.shape[0]
        pad = (-b) % self.dp_world_size
        if pad:
            inps = torch.cat([inps] + [inps[:1]] * pad, dim=0)
        per = inps.shape[0] // self.dp_world_size
        return inps[self.dp_rank * per:(self.dp_rank + 1) * per], pad

    def _dp_gather(self, logits, pad):
        if logits is None or self.dp_world_size == 1:
            return logits
        parts = [torch.zeros_like(logits) for _ in range(self.dp_world_size)]
        dist.all_gather(parts, logits.contiguous(), group=self.dp_group)
        full = torch.cat(parts, dim=0)
        return full[: full.shape[0] - pad] if pad else full

    # ------------------------------------------------------------------ scoring
    def _loglikelihood_tokens(self, requests, disable_tqdm=True):
        """requests: list of ((context str, continuation str) | None, context ids, continuation ids)."""
        self.model.module.inference_mode(use_cache=False)
        self.model.module.clear_cache()          # key/value caches left by a generation request must not leak in
        order = sorted(range(len(requests)), key=lambda i: -(len(requests[i][1]) + len(requests[i][2])))
        results = [None] * len(requests)
        with torch.no_grad():
            for s in range(0, len(order), self.batch_size):
                chunk = [requests[i] for i in order[s:s + self.batch_size]]
                rows, lens, conts = [], [], []
                for _, ctx, cont in chunk:
                    ids = (list(ctx) + list(cont))[-(self.max_length + 1):][:-1]
                    lens.append(len(ids))
                    conts.append(list(cont))
                    rows.append(ids)
                width = max(lens)
                batch = torch.tensor([r + [0] * (width - len(r)) for r in rows], dtype=torch.long)
                mine, pad = self._dp_scatter(batch)
                logits = self._dp_gather(self._model_call(mine), pad)
                if logits is None:
                    continue
                logp = F.log_softmax(logits.float(), dim=-1).cpu()
                for j, (n, cont) in enumerate(zip(lens, conts)):
                    c = min(len(cont), n)
                    lp = logp[j, n - c:n]
                    target = torch.tensor(cont[-c:], dtype=torch.long)
                    greedy = bool((lp.argmax(-1) == target).all())
                    score = float(lp.gather(1, target[:, None]).sum())
                    results[order[s + j]] = (score, greedy)
        self.model.module.train_mode()
        return results

    def loglikelihood(self, requests):
        reqs = []
        for r in requests:
            ctx, cont = r.args if hasattr(r, "args") else r
            ctx_ids = [self.eot_token_id] if ctx == "" else self.tok_encode(ctx)
            reqs.append(((ctx, cont), ctx_ids, self.tok_encode(cont)))
        return self._loglikelihood_tokens(reqs)

    def loglikelihood_rolling(self, requests):
        out = []
        for r in requests:
            (text,) = r.args if hasattr(r, "args") else (r,)
            ids = self.tok_encode(text)
            total, prev = 0.0, [self.eot_token_id]
            for s in range(0, len(ids), self.max_length):
                window = ids[s:s + self.max_length]
                (score, _), = self._loglikelihood_tokens([(None, prev[-1:], window)])
                total += score
                prev = window
            out.append(total)
        return out

    def generate_until(self, requests):
        self.model.module.inference_mode(use_cache=True)
        res = []
        for r in requests:
            ctx, kw = r.args if hasattr(r, "args") else r
            until = kw.get("until", []) if isinstance(kw, dict) else kw
            until = [until] if isinstance(until, str) else list(until)
            stop = [self.tok_encode(u) for u in until if u]
            # prompt and continuation share the model's context: keep the tail of a long prompt, cap the continuation
            ids = self.tok_encode(ctx)
            room = max(1, min(self.max_gen_toks, self.max_length // 2))
            if len(ids) > self.max_length - room:
                ctx = self.tok_decode(ids[-(self.max_length - room):])
                ids = ids[-(self.max_length - room):]
            budget = max(1, min(self.max_gen_toks, self.max_length - len(ids)))
            out = generate_samples_from_prompt(self.neox_args, self.model, text=ctx, recompute=self.neox_args.recompute,
                                               temperature=0.0, maximum_tokens=budget, stop_tokens=stop or None)
            text = (out[0]["text"] if out else "") or ""
            for u in until:
                if u:
                    text = text.split(u)[0]
            res.append(text)
        self.model.module.clear_cache()
        self.model.module.train_mode()
        return res

    # ------------------------------------------------------------------ harness driver
    def run_eval(self, eval_tasks=None, num_fewshot=0, bootstrap_iters=2, use_cache=False, name="neox", limit=None):
        try:
            from lm_eval import evaluator, tasks
            from lm_eval.api.model import LM
        except ModuleNotFoundError as exc:
            raise ModuleNotFoundError("lm_eval (lm-evaluation-harness >= 0.4) is required for eval.py / `eval_tasks`") from exc
        adapter = self

        class _LM(LM):
            def loglikelihood(self, requests):
                return adapter.loglikelihood(requests)

            def loglikelihood_rolling(self, requests):
                return adapter.loglikelihood_rolling(requests)

            def generate_until(self, requests):
                return adapter.generate_until(requests)

        eval_tasks = eval_tasks or ["lambada_openai", "piqa", "hellaswag", "winogrande", "mathqa", "pubmedqa"]
        task_manager = tasks.TaskManager()
        task_dict = tasks.get_task_dict(eval_tasks, task_manager)
        results = evaluator.evaluate(lm=_LM(), task_dict=task_dict, limit=limit, bootstrap_iters=bootstrap_iters,
                                     log_samples=False)
        results["config"] = {"model": name, "num_fewshot": num_fewshot, "batch_size": self.batch_size,
                             "limit": limit, "bootstrap_iters": bootstrap_iters}
        return results


def run_eval_harness(model, forward_step_fn, neox_args, batch_size=None, eval_tasks=None, num_fewshot=0,
                     bootstrap_iters=2):
    print_rank_0("Running evaluation harness...")
    adapter = EvalHarnessAdapter(model, forward_step_fn, neox_args, batch_size)
    return adapter.run_eval(eval_tasks=eval_tasks, num_fewshot=num_fewshot, bootstrap_iters=bootstrap_iters)
