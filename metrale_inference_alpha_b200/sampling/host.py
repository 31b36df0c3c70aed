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


def dry_penalties(tokens: List[int], multiplier: float, base: float, allowed: int, window: int) -> dict:
    """DRY: for every earlier occurrence of the last token, measure how long the text before it
    matches the text before the end; the token that followed that occurrence would extend a repeat
    of that length. Returns {token: penalty} (the largest repeat per token wins).
    Role of ``crates/sampling/src/penalties.rs`` (DRY)."""
    n = len(tokens)
    if n < 2 or multiplier <= 0:
        return {}
    lo = max(0, n - window)
    last = tokens[-1]
    out: dict = {}
    for i in range(n - 2, lo - 1, -1):
        if tokens[i] != last:
            continue
        k = 1
        while i - k >= lo and tokens[i - k] == tokens[n - 1 - k] and k < 64:
            k += 1
        if k >= allowed:
            nxt = tokens[i + 1]
            pen = multiplier * base ** (k - allowed)
            if pen > out.get(nxt, 0.0):
                out[nxt] = pen
    return out


def lz_penalty(tokens: List[int], strength: float, window: int = 2048) -> dict:
    """Loop guard: the longest earlier match of the current suffix (length L >= 4) predicts its
    continuation; that token is penalised by strength * L. Role of the LZ penalty of
    ``crates/sampling/src/penalties.rs``."""
    n = len(tokens)
    if strength <= 0 or n < 8:
        return {}
    lo = max(0, n - window)
    best_len, best_next = 0, None
    for i in range(n - 2, lo - 1, -1):
        if tokens[i] != tokens[-1]:
            continue
        k = 1
        while i - k >= lo and tokens[i - k] == tokens[n - 1 - k] and k < 256:
            k += 1
        if k > best_len:
            best_len, best_next = k, tokens[i + 1]
    return {best_next: strength * best_len} if best_len >= 4 else {}


def forced_think_close(out_tokens: List[int], budget: int, end_ids: List[int]):
    """Token to force so that the reasoning block closes, or None: nothing is forced before
    `budget` output tokens, nor once the closing marker has appeared; after the budget the
    marker is emitted token by token (resuming a partly written marker)."""
    n = len(end_ids)
    if budget <= 0 or n == 0 or len(out_tokens) < budget:
        return None
    for i in range(len(out_tokens) - n + 1):
        if out_tokens[i:i + n] == end_ids:
            return None
    k = min(n - 1, len(out_tokens) - budget)
    while k > 0 and out_tokens[-k:] != end_ids[:k]:
        k -= 1
    return end_ids[k]


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
    row_first = {}
    for r0, it0 in enumerate(row_item):
        row_first.setdefault(id(it0), r0)
    P = [it.seq.req.params for it in row_item]
    if any(p.has_penalties for p in P):
        tok, cnt, inp = _penalty_tables(row_item, dev)
        f = lambda name: torch.tensor([getattr(p, name) for p in P], dtype=torch.float32, device=dev)
        ops.apply_penalties(logits, tok, cnt, inp, f("repetition_penalty"), f("presence_penalty"),
                            f("frequency_penalty"))
    spec_ahead: dict = {}            # item -> draft tokens its grammar was advanced over while masking
    for r, it in enumerate(row_item):
        p = it.seq.req.params
        if p.logit_bias:
            idx = torch.tensor(list(p.logit_bias.keys()), device=dev)
            logits[r, idx] += torch.tensor(list(p.logit_bias.values()), dtype=torch.float32, device=dev)
        if p.dry_multiplier > 0 or p.lz_penalty > 0:
            # verify rows of one item see the sequence as of their own position
            upto = len(it.seq.tokens) - (it.verify - (r - row_first[id(it)]))
            hist = it.seq.tokens[:upto]
            pens = dry_penalties(hist, p.dry_multiplier, p.dry_base, p.dry_allowed_length, p.dry_window)
            for tkn, v in lz_penalty(hist, p.lz_penalty).items():
                pens[tkn] = pens.get(tkn, 0.0) + v
            if pens:
                idx = torch.tensor(list(pens.keys()), device=dev)
                logits[r, idx] -= torch.tensor(list(pens.values()), dtype=torch.float32, device=dev)
        if p.grammar is not None:
            # row j of a verify item is masked from the state after drafts 1..j; the matcher is
            # rewound to the accepted prefix once the targets are known
            j = r - row_first[id(it)]
            mask = p.grammar.allowed_mask(logits.shape[1])
            if j < it.verify and hasattr(p.grammar, "rollback"):
                d = it.tokens[1 + j]
                if spec_ahead.get(id(it), 0) == j and d < mask.shape[0] and bool(mask[d]):
                    p.grammar.advance(d)
                    spec_ahead[id(it)] = j + 1
            logits[r].masked_fill_(~mask.to(dev), float("-inf"))
        if p.thinking_budget > 0 and p.think_end_ids and it.verify == 0:
            force = forced_think_close(it.seq.tokens[it.seq.prompt_len:], p.thinking_budget, p.think_end_ids)
            if force is not None and force < logits.shape[1] and torch.isfinite(logits[r, force]):
                keep = logits[r, force].clone()
                logits[r].fill_(float("-inf"))
                logits[r, force] = keep
        if runner.logit_processor is not None:
            logits[r] = runner.logit_processor(it.seq, logits[r])
        if p.top_n_sigma > 0 and p.temperature > 0:
            x = logits[r]
            fin = torch.isfinite(x)
            thr = x[fin].max() - p.top_n_sigma * x[fin].std()
            x.masked_fill_(x < thr, float("-inf"))
    temps = [p.temperature for p in P]
    for r, it in enumerate(row_item):
        ad = it.seq.req.params.adaptive
        if ad is not None and it.verify == 0:
            temps[r] = ad.step(logits[r], it.seq.tokens[it.seq.prompt_len:], it.seq.req.params.grammar is not None)
    t = lambda vals, dt: torch.tensor(vals, dtype=dt, device=dev)
    seeds = [(p.seed if p.seed is not None else it.seq.seq_id * 1000003) & ((1 << 62) - 1)
             for p, it in zip(P, row_item)]
    ids, lp = ops.sample(logits, t(temps, torch.float32),
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
        gm = it.seq.req.params.grammar
        if gm is not None:
            if spec_ahead.get(id(it)):
                gm.rollback(spec_ahead[id(it)])
            n_acc = 0
            while n_acc < it.verify and it.tokens[1 + n_acc] == ids[r + n_acc]:
                n_acc += 1
            for tkn in list(it.tokens[1:1 + n_acc]) + [ids[r + n_acc]]:
                gm.advance(tkn)
        if it.seq.req.params.top_logprobs:
            top = torch.log_softmax(logits[r + k - 1], -1).topk(it.seq.req.params.top_logprobs)
            it.seq.top_logprobs = getattr(it.seq, "top_logprobs", []) + [
                list(zip(top.indices.tolist(), top.values.tolist()))]
        it.seq.sample_step += 1
        r += k
    return toks, lps
