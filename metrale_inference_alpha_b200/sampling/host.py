"""Full-logits sampling path for requests the fused device selection cannot serve: logit
bias, grammar masks, top-n-sigma, top-k log-prob reporting, and repetition / presence /
frequency penalties. Order follows the reference host pipeline: penalties -> bias -> greedy
or (top-n-sigma -> temperature -> top-k -> min-p -> top-p -> multinomial)
(``crates/sampling/src/sample_impl.rs:26-178``, ``penalties.rs``). Penalties and the final
draw run as device kernels on the fp32 logits; only grammar masks and bias need the host.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Tuple

import torch

from .. import ops


def _penalty_tables(items, device):
    rows = []
    for it in items:
        p = it.seq.req.params
        if not p.has_penalties:
            rows.append(([], [], []))
            continue
        out = Counter(it.seq.output_ids)
        prompt = set(it.seq.tokens[:it.seq.prompt_len])
        toks = list(set(out) | prompt)
        rows.append((toks, [out.get(t, 0) for t in toks], [int(t in prompt) for t in toks]))
    width = max(1, max(len(r[0]) for r in rows))
    mk = lambda k, fill: torch.tensor([r[k] + [fill] * (width - len(r[k])) for r in rows], dtype=torch.int32,
                                      device=device)
    return mk(0, -1), mk(1, 0), mk(2, 0)


def sample_rows(runner, plan, logits: torch.Tensor) -> Tuple[List[List[int]], List[List[float]]]:
    """logits: fp32 [R, V], one row per sampled position in plan order."""
    items = [it for it in plan.items if it.sample]
    dev = logits.device
    # expand per-item parameters to per-row (verify items own several rows, all greedy)
    row_item = []
    for it in items:
        row_item += [it] * (it.verify + 1)
    R = len(row_item)
    assert logits.shape[0] == R
    P = [it.seq.req.params for it in row_item]
    if any(p.has_penalties for p in P):
        tok, cnt, inp = _penalty_tables(row_item, dev)
        f = lambda name: torch.tensor([getattr(p, name) for p in P], dtype=torch.float32, device=dev)
        ops.apply_penalties(logits, tok, cnt, inp, f("repetition_penalty"), f("presence_penalty"),
                            f("frequency_penalty"))
    for r, it in enumerate(row_item):
        p = it.seq.req.params
        if p.logit_bias:
            idx = torch.tensor(list(p.logit_bias.keys()), device=dev)
            logits[r, idx] += torch.tensor(list(p.logit_bias.values()), dtype=torch.float32, device=dev)
        if p.grammar is not None:
            mask = p.grammar.allowed_mask(logits.shape[1]).to(dev)
            logits[r].masked_fill_(~mask, float("-inf"))
        if runner.logit_processor is not None:
            logits[r] = runner.logit_processor(it.seq, logits[r])
        if p.top_n_sigma > 0 and p.temperature > 0:
            x = logits[r]
            fin = torch.isfinite(x)
            thr = x[fin].max() - p.top_n_sigma * x[fin].std()
            x.masked_fill_(x < thr, float("-inf"))
    t = lambda vals, dt: torch.tensor(vals, dtype=dt, device=dev)
    seeds = [(p.seed if p.seed is not None else it.seq.seq_id * 1000003) & ((1 << 62) - 1)
             for p, it in zip(P, row_item)]
    ids, lp = ops.sample(logits, t([p.temperature for p in P], torch.float32),
                         t([p.top_k for p in P], torch.int32), t([p.top_p for p in P], torch.float32),
                         t([p.min_p for p in P], torch.float32), t(seeds, torch.int64),
                         t([it.seq.sample_step for it in row_item], torch.int64))
    ids, lp = ids.tolist(), lp.tolist()
    toks, lps, r = [], [], 0
    for it in plan.items:
        if not it.sample:
            toks.append([]); lps.append([])
            continue
        k = it.verify + 1
        toks.append(ids[r:r + k]); lps.append(lp[r:r + k])
        if it.seq.req.params.grammar is not None:
            it.seq.req.params.grammar.advance(ids[r + k - 1])
        if it.seq.req.params.top_logprobs:
            top = torch.log_softmax(logits[r + k - 1], -1).topk(it.seq.req.params.top_logprobs)
            it.seq.top_logprobs = getattr(it.seq, "top_logprobs", []) + [
                list(zip(top.indices.tolist(), top.values.tolist()))]
        it.seq.sample_step += 1
        r += k
    return toks, lps
