"""One forward step's device-side description (what the scheduler hands the model).

Rows are query tokens, grouped by sequence: sequence s owns rows
``q_start[s] .. q_start[s] + q_len[s]``; its KV context after this step is ``ctx_len[s]``
tokens, addressed through ``block_table[s]``. The same structure describes a decode step
(q_len 1), a speculative verify step (q_len k+1), a prefill chunk (q_len up to the chunk
budget) and any mix of them. Role of the reference's ``ForwardContext``
(``crates/model-layers/src/layer.rs:218-290``) and per-row metadata uploads
(``model-engine/src/model/trait_impl/decode_a2.rs``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


class SpecStash:
    """Inputs of every recurrent op of one speculative verify step. During such a step the
    recurrent layers read their state but do not advance it; once the scheduler knows how many
    tokens each sequence accepted, ``ModelRunner.commit_recurrent`` replays exactly that many
    rows of these inputs through the same ops, state-only (write-on-accept; role of the
    reference's GDN carry / verify kernels, ``crates/model-engine/src/model/gdn_carry.rs:1-25``,
    rollback invariants ``book/src/deep-dives/mtp.md:294-300``)."""

    def __init__(self, batch: "ForwardBatch"):
        self.batch = batch
        self.layers = {}                 # recurrent layer index -> tuple of retained tensors


@dataclass
class ForwardBatch:
    token_ids: torch.Tensor            # [T] int32
    positions: torch.Tensor            # [T] int32
    slot_mapping: torch.Tensor         # [T] int64 flat KV slot (-1 = do not write)
    q_start: torch.Tensor              # [S] int32
    q_len: torch.Tensor                # [S] int32
    ctx_len: torch.Tensor              # [S] int32
    block_table: torch.Tensor          # [S, max_blocks] int32
    logit_rows: torch.Tensor           # [R] int64 rows whose logits are needed
    max_q_len: int = 1
    max_ctx: int = 0
    state_slots: Optional[torch.Tensor] = None   # [S] int32 recurrent-state slot per sequence
    num_tokens: int = 0
    num_seqs: int = 0
    # host copies (CPU reference path and debugging)
    host_q_len: Optional[List[int]] = None
    # hidden rows to return for the MTP head (same indexing as logit_rows)
    want_hidden: bool = False
    # LoRA: adapter slot of every token row (-1 = base model); None when no row has an adapter
    adapter_rows: Optional[torch.Tensor] = None
    # multimodal rows: (row indices int64 [n], embeddings bf16 [n, hidden]) that replace token embeddings
    embed_override: Optional[tuple] = None
    # per-row rotary tables (cos, sin) [T, rot / 2] when some row's rotary position is not its sequence index
    rope_tables: Optional[tuple] = None
    rope_rows: Optional[torch.Tensor] = None     # arange(T) int32: row -> its rotary row
    # speculative verify over recurrent layers: state is left untouched and inputs are retained here
    spec_stash: Optional[SpecStash] = None

    @property
    def device(self):
        return self.token_ids.device

    @staticmethod
    def build(seqs, block_size: int, device="cpu", max_blocks: Optional[int] = None,
              pad_seqs: int = 0, pin: bool = False) -> "ForwardBatch":
        """seqs: list of dicts {tokens: [ids], start_pos: int, blocks: [ids], state_slot: int,
        logits: 'last' | 'all' | 'none'}. `pad_seqs` pads to a fixed sequence count with
        null rows (token 0, position 0, null block, q_len 1) for CUDA-graph rungs."""
        tok, pos, slot, qs, ql, cl, lrows, sslots = [], [], [], [], [], [], [], []
        nb = max_blocks or max(1, max((len(s["blocks"]) for s in seqs), default=1))
        bt = []
        row = 0
        for s in seqs:
            n = len(s["tokens"])
            st = s["start_pos"]
            tok += list(s["tokens"])
            pos += list(range(st, st + n))
            for p in range(st, st + n):
                slot.append(s["blocks"][p // block_size] * block_size + p % block_size)
            qs.append(row)
            ql.append(n)
            cl.append(st + n)
            bt.append(list(s["blocks"]) + [0] * (nb - len(s["blocks"])))
            sslots.append(s.get("state_slot", 0))
            want = s.get("logits", "last")
            if want == "last":
                lrows.append(row + n - 1)
            elif want == "all":
                lrows += list(range(row, row + n))
            row += n
        real_seqs = len(seqs)
        while len(qs) < pad_seqs:
            tok.append(0); pos.append(0); slot.append(-1)
            qs.append(row); ql.append(1); cl.append(1)
            bt.append([0] * nb); sslots.append(0)
            lrows.append(row)
            row += 1
        mk = lambda v, dt: torch.tensor(v, dtype=dt, device=device)
        b = ForwardBatch(
            token_ids=mk(tok, torch.int32), positions=mk(pos, torch.int32), slot_mapping=mk(slot, torch.int64),
            q_start=mk(qs, torch.int32), q_len=mk(ql, torch.int32), ctx_len=mk(cl, torch.int32),
            block_table=mk(bt, torch.int32).view(len(qs), nb), logit_rows=mk(lrows, torch.int64),
            max_q_len=max(ql) if ql else 1, max_ctx=max(cl) if cl else 0,
            state_slots=mk(sslots, torch.int32), num_tokens=row, num_seqs=len(qs), host_q_len=ql)
        b.real_seqs = real_seqs
        return b
