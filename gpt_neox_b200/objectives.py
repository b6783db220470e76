"""Training objectives beyond the plain LM loss: MoE load-balancing auxiliary loss, pairwise reward
model, DPO, KTO and REINFORCE with KL variants.

Definitions follow ``megatron/training.py:533-939`` of the reference; each objective is a function
of (sharded) logits so it can be unit-tested against a dense restatement.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .parallel import mappings as M
from .parallel.cross_entropy import vocab_parallel_cross_entropy


def get_logp(logits, labels, force_fp32=False):
    """Per-token log-probability of ``labels`` under vocab-parallel ``logits`` ([b, s, V/tp])."""
    if force_fp32:
        logits = logits.float()
    return -vocab_parallel_cross_entropy(logits, labels)


def get_pos_neg_logp(logits, labels, force_fp32=False):
    """Batch is [chosen ; rejected] stacked on dim 0."""
    return torch.chunk(get_logp(logits, labels, force_fp32), 2, 0)


def reward_model_loss(values, loss_mask, z_loss=0.0):
    """Pairwise Bradley-Terry loss.  ``values``: [2B, s, 1]; the i-th unmasked position of a chosen row
    is compared with the i-th unmasked position of the matching rejected row."""
    pos, neg = torch.chunk(values, 2, 0)
    pos_mask, neg_mask = torch.chunk(loss_mask, 2, 0)
    pos_idx = pos_mask.nonzero()[:, 1].unsqueeze(1)
    neg_idx = neg_mask.nonzero()[:, 1].unsqueeze(1)
    pos = torch.gather(pos.squeeze(-1), dim=1, index=pos_idx)
    neg = torch.gather(neg.squeeze(-1), dim=1, index=neg_idx)
    metrics = {"pos_values": pos.detach().mean(), "neg_values": neg.detach().mean(),
               "margin": (pos - neg).detach().mean(), "accuracy": ((pos - neg) > 0).float().mean()}
    loss = -F.logsigmoid(pos - neg).mean() + (z_loss * (pos ** 2 + neg ** 2)).mean()
    return loss, metrics


def dpo_loss(policy_logits, labels, loss_mask, beta, ref_logits=None, ref_logp=None, reference_free=False,
             fp32=True):
    pos_mask, neg_mask = torch.chunk(loss_mask, 2, 0)
    with torch.no_grad():
        if reference_free:
            ref_pos = ref_neg = 0.0
        else:
            if ref_logp is None:
                rp, rn = get_pos_neg_logp(ref_logits, labels, fp32)
            else:
                rp, rn = torch.chunk(ref_logp, 2, 0)
            ref_pos, ref_neg = (rp * pos_mask).sum(-1), (rn * neg_mask).sum(-1)
    cp, cn = get_pos_neg_logp(policy_logits, labels, fp32)
    chosen_pos, chosen_neg = (cp * pos_mask).sum(-1), (cn * neg_mask).sum(-1)
    metrics = {"chosen_neg": chosen_neg.detach().mean(), "chosen_pos": chosen_pos.detach().mean()}
    if not reference_free:
        cr = beta * (chosen_pos.detach() - ref_pos)
        rr = beta * (chosen_neg.detach() - ref_neg)
        metrics.update({"ref_neg": ref_neg.mean(), "ref_pos": ref_pos.mean(), "chosen_rewards": cr.mean(),
                        "rejected_rewards": rr.mean(), "reward_acc": (cr > rr).float().mean(),
                        "margins": (cr - rr).mean()})
    logits = (chosen_pos - chosen_neg) - (ref_pos - ref_neg)
    return -F.logsigmoid(beta * logits).mean(), metrics


def kto_loss(policy_logits, labels, loss_mask, rewards, beta, desirable_weight, undesirable_weight, ref_logits=None,
             ref_logp=None, fp32=True):
    """KTO with the batch split in halves, each half providing the KL baseline of the other."""
    lab = labels.clone()
    lab[lab == -100] = 0
    with torch.no_grad():
        if ref_logp is None:
            ref_logp = get_logp(ref_logits, lab, fp32)
        ref_logp = ref_logp * loss_mask
        scaling = (rewards.sum(-1) > 0.001).float() * desirable_weight \
            + (rewards.sum(-1) < -0.001).float() * undesirable_weight
        pos_mask, neg_mask = (rewards > 0.001).float(), (rewards < -0.001).float()
    pol = get_logp(policy_logits, lab, fp32) * loss_mask
    with torch.no_grad():
        d = pol.detach()
        metrics = {"ref_logp": ref_logp.sum(-1).mean(), "policy_logp": d.sum(-1).mean(),
                   "pos_ref_logp": (ref_logp * pos_mask).sum(-1).mean(),
                   "neg_ref_logp": (ref_logp * neg_mask).sum(-1).mean(),
                   "pos_policy_logp": (d * pos_mask).sum(-1).mean(), "neg_policy_logp": (d * neg_mask).sum(-1).mean(),
                   "kl": (d - ref_logp).sum() / loss_mask.sum()}
        pr = beta * rewards * (d - ref_logp)
        metrics["reward_acc"] = (pr.sum(-1) > 0.0).float().mean()
        metrics["policy_rewards"] = pr.sum()
    p1, p2 = torch.chunk(pol, 2, 0)
    r1, r2 = torch.chunk(ref_logp, 2, 0)
    w1, w2 = torch.chunk(rewards, 2, 0)
    s1, s2 = torch.chunk(scaling, 2, 0)
    kl1 = torch.clamp((p1 - r1).sum(-1), min=0).mean().detach()
    kl2 = torch.clamp((p2 - r2).sum(-1), min=0).mean().detach()
    l1 = 0.5 * s1 * (1 - torch.sigmoid(beta * w1.mean(-1) * ((p1 - r1).sum(-1) - kl2)))
    l2 = 0.5 * s2 * (1 - torch.sigmoid(beta * w2.mean(-1) * ((p2 - r2).sum(-1) - kl1)))
    return (l1 + l2).mean(), metrics


def reinforce_loss(policy_logits, labels, loss_mask, rewards, raw_rewards, kl_impl="mse", kl_beta=0.1,
                   ref_logits=None, fp32=True):
    metrics = {}
    full = kl_impl == "full"
    ref_tok = ref_full = None
    if ref_logits is not None:
        with torch.no_grad():
            if full:
                r = M.gather_from_model_parallel_region(ref_logits)
                ref_full = (r.float() if fp32 else r).log_softmax(dim=-1)
                ref_tok = torch.gather(ref_full, 2, labels.unsqueeze(2)).squeeze(2)
            else:
                ref_tok = get_logp(ref_logits, labels, fp32)
            metrics["ref_logp"] = ref_tok.mean()
    if full:
        o = M.gather_from_model_parallel_region(policy_logits)
        logp_full = (o.float() if fp32 else o).log_softmax(dim=-1)
        tok = torch.gather(logp_full, 2, labels.unsqueeze(2)).squeeze(2)
    else:
        tok = get_logp(policy_logits, labels, fp32)
    metrics.update({"logp": tok.detach().mean(), "reward": raw_rewards.detach().mean(),
                    "reward_std": raw_rewards.detach().std()})
    denom = loss_mask.sum()
    if ref_logits is not None:
        if full:
            kl = F.kl_div(ref_full, logp_full, log_target=True, reduction="none").sum(-1)
        else:
            kl = tok - ref_tok
            kl = kl.abs() if kl_impl == "abs" else 0.5 * kl.square() if kl_impl == "mse" else kl
        metrics["kl"] = kl.detach().mean()
        loss = -tok * rewards + kl_beta * kl
    else:
        loss = -(rewards * tok)
    return ((loss * loss_mask).sum(-1) / denom).mean(), metrics
