"""Multi-token-prediction drafting on the model runner.

After a target step, each sequence's drafter context is caught up: the MTP layer consumes
(token t+1, target hidden of position t) pairs for every position the target just committed,
writing its own KV cache, and then drafts k tokens autoregressively, feeding its own hidden
state back (``crates/server/src/scheduler/mtp_step.rs``: catch-up then propose;
``crates/model-layers/src/layers/mtp_head/forward.rs``).
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..engine.batch import ForwardBatch


def mtp_propose(runner, plan, result, accepted: List[int], k: int) -> List[List[int]]:
    """`accepted[i]` = number of tokens sequence i committed in this step (>= 1 for sampled
    items). result.hidden holds the target hidden rows of every sampled row, in plan order."""
    dec, bs, dev = runner.decoder, runner.block_size, runner.device
    hidden_all = result.hidden
    seqs, first_tok, hid_rows = [], [], []
    r = 0
    for i, it in enumerate(plan.items):
        if not it.sample:
            continue
        rows = it.verify + 1
        if accepted[i] > 0 and not it.seq.is_finished():
            n_acc = accepted[i] - 1                     # accepted drafts; bonus token follows
            # hidden of the last committed target position predicts the newest token
            hid_rows.append(r + n_acc)
            seqs.append(it.seq)
            first_tok.append(it.seq.tokens[-1])
        r += rows
    drafts = {s.seq_id: [] for s in seqs}
    if not seqs:
        return [[] for _ in plan.items]
    if dev.type == "cuda" and runner.graphs_ready() and getattr(runner, "graph_propose", True):
        got = runner.propose_graphed(seqs, first_tok, hid_rows, hidden_all, k)
        if got is not None:
            for s, d in zip(seqs, got):
                drafts[s.seq_id] = d
            return _collect(plan, drafts)
    hidden = hidden_all.index_select(0, torch.tensor(hid_rows, device=dev))
    toks = torch.tensor(first_tok, dtype=torch.int32, device=dev)
    for j in range(k):
        items = []
        for s in seqs:
            # the drafter token at step j sits at position len(tokens) - 1 + j of the sequence
            pos = len(s.tokens) - 1 + j
            nb = (pos + bs) // bs
            if nb > len(s.blocks):
                return _collect(plan, drafts)          # no block headroom: stop drafting here
            items.append(dict(tokens=[0], start_pos=pos, blocks=s.blocks, state_slot=0))
        b = ForwardBatch.build(items, bs, device=dev, max_blocks=runner.max_blocks)
        b.token_ids = toks
        logits, hidden = dec.mtp_forward(toks, hidden, b, runner.caches)
        runner.tp.end_forward()
        toks = ops.argmax(logits)
        for s, t in zip(seqs, toks.tolist()):
            drafts[s.seq_id].append(int(t))
    return _collect(plan, drafts)


def _collect(plan, drafts):
    return [drafts.get(it.seq.seq_id, []) for it in plan.items]
