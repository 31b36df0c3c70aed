"""Block drafter ("DFlash" style): all drafts of a step come out of ONE forward.

A small stack of dense attention layers, conditioned on the target model's own hidden states:

* context: after every target forward the hidden states of a few chosen target layers are
  stacked per token, projected by ``fc`` and normalised (``hidden_norm``); every drafter layer's
  key / value projection of that feature is written into the drafter's paged KV cache at the
  token's own slot. The drafter cache is addressed by the *target's* block tables, so prefix
  reuse, preemption and rollback need no bookkeeping of their own: a slot that the target
  rewrites is rewritten here by the same forward.
* block: a proposal embeds ``[last token, MASK x gamma]`` at positions p + 1 .. p + 1 + gamma
  (with the target's embedding table), runs the drafter layers with every block row attending
  to the whole context and to the whole block (not causal inside the block), and reads the
  drafts off the mask rows through the drafter's final norm and the target's lm_head.

Inside this engine the block rows are expressed to the paged attention kernel as sequences of
one query row each that share the sequence's block table and context length, which gives the
bidirectional block mask without a new kernel. The drafter reuses ``Decoder`` with its own
configuration for the layer bodies.

Role of the reference's block-diffusion draft head (``crates/model-arch/src/dflash_head.rs``:
shared embedding / lm_head, ``fc`` + ``hidden_norm`` over ``target_layer_ids``;
``dflash_head/precompute_ctx_kv.rs``: context K/V of every layer from one feature;
``dflash_head/forward_block.rs``: anchor + mask rows, one forward per proposal;
``dflash_head/propose.rs``); the proposal width policy is ``speculative/ladder.py::DflashRung``.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..cache import PagedKvCache
from ..config.model_config import ModelConfig
from ..engine.batch import ForwardBatch
from ..models.decoder import Decoder, LayerCaches
from ..ops import QuantWeight
from ..weights.loader import Loader
from ..weights.source import SyntheticSource, TensorSource


@dataclass
class DflashConfig:
    num_layers: int = 2
    target_layer_ids: Sequence[int] = ()        # target layers whose output hidden states condition the drafter
    mask_token_id: int = 0
    gamma: int = 5                              # widest block: drafts per proposal
    num_heads: int = 0                          # 0 = the target's
    num_kv_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0

    def resolve(self, cfg: ModelConfig) -> "DflashConfig":
        ids = tuple(self.target_layer_ids) or tuple(sorted({cfg.num_layers // 2, cfg.num_layers - 1}))
        assert all(0 <= i < cfg.num_layers for i in ids), ids
        return dataclasses.replace(
            self, target_layer_ids=ids, num_heads=self.num_heads or cfg.num_heads,
            num_kv_heads=self.num_kv_heads or cfg.num_kv_heads, head_dim=self.head_dim or cfg.head_dim,
            intermediate_size=self.intermediate_size or cfg.intermediate_size)


@dataclass
class DflashW:
    fc: QuantWeight = None                      # [hidden, len(target_layer_ids) * hidden] bf16
    hidden_norm: torch.Tensor = None
    norm: torch.Tensor = None
    layers: List = field(default_factory=list)  # LayerW (attention + dense FFN)


def drafter_model_config(cfg: ModelConfig, dc: DflashConfig) -> ModelConfig:
    """The drafter's layer geometry as a plain dense GQA configuration (bf16 weights and KV)."""
    return ModelConfig(name=cfg.name + "-dflash", arch="dense_gqa", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                       num_layers=dc.num_layers, num_heads=dc.num_heads, num_kv_heads=dc.num_kv_heads,
                       head_dim=dc.head_dim, rope_theta=cfg.rope_theta, qk_norm=True, rms_eps=cfg.rms_eps,
                       intermediate_size=dc.intermediate_size, weight_format="bf16", kv_dtype="bf16",
                       max_position=cfg.max_position)


def load_dflash(cfg: ModelConfig, dc: DflashConfig, src: Optional[TensorSource] = None, device="cpu",
                seed: int = 1) -> DflashW:
    """Drafter weights from a checkpoint source in HF layout (``model.layers.N.*``, ``fc.weight``,
    ``hidden_norm.weight``, ``model.norm.weight``), or random ones when `src` is None (the
    drafter checkpoint carries no embedding and no lm_head: both are the target's;
    ``crates/model-arch/src/weight_loader/dflash_loader.rs``)."""
    dcfg = drafter_model_config(cfg, dc)
    synthetic = src is None
    if synthetic:
        src = SyntheticSource(dcfg, seed=seed, device=device)
    ld = Loader(dcfg, src, device)
    w = DflashW()
    for i in range(dc.num_layers):
        w.layers.append(ld.layer(f"model.layers.{i}", "attention", "dense"))
    H, n = cfg.hidden_size, len(dc.target_layer_ids)
    if synthetic:
        g = torch.Generator().manual_seed(seed + 17)
        w.fc = ops.make_weight(torch.randn(H, n * H, generator=g) * (0.5 / (n * H) ** 0.5), "bf16").to(device)
        w.hidden_norm = torch.ones(H, dtype=torch.bfloat16, device=device)
    else:
        w.fc = ld.lin("fc", quant=False)
        w.hidden_norm = ld.vec("hidden_norm.weight")
    w.norm = ld.vec("model.norm.weight")
    return w


class DflashDrafter:
    """Owns the drafter's weights, decoder and KV cache; hooks into the target's forward for the
    context and serves `propose`."""

    def __init__(self, runner, dc: DflashConfig, weights: Optional[DflashW] = None, seed: int = 1):
        cfg = runner.cfg
        self.runner, self.target = runner, runner.decoder
        self.dc = dc.resolve(cfg)
        self.dcfg = drafter_model_config(cfg, self.dc)
        self.device = runner.device
        self.w = weights or load_dflash(cfg, self.dc, None, self.device, seed)
        from ..engine.runner import kv_config
        from ..weights.loader import ModelW
        mw = ModelW()
        mw.layers, mw.embed, mw.final_norm, mw.lm_head = self.w.layers, runner.w.embed, self.w.norm, runner.w.lm_head
        self.dec = Decoder(self.dcfg, mw, None, self.device)            # replicated on every rank: no collectives
        self.kv = PagedKvCache(kv_config(self.dcfg, mw, runner.block_size), runner.kv.num_blocks, self.device)
        self.caches = LayerCaches(self.dcfg, kv=self.kv)
        self.capture_ids = {i: j for j, i in enumerate(self.dc.target_layer_ids)}
        self._feat: Optional[torch.Tensor] = None
        self.proposals = 0

    # ------------------------------------------------------------------ context (called by the target decoder)
    def begin(self, num_tokens: int) -> None:
        H, n = self.target.cfg.hidden_size, len(self.capture_ids)
        self._feat = torch.empty(num_tokens, n * H, dtype=torch.bfloat16, device=self.device)

    def capture(self, layer: int, x: torch.Tensor) -> None:
        j = self.capture_ids.get(layer)
        if j is not None:
            H = self.target.cfg.hidden_size
            self._feat[:, j * H:(j + 1) * H].copy_(x)

    def absorb(self, batch: ForwardBatch) -> None:
        """Write every drafter layer's context K/V of the forward's rows at the rows' own slots."""
        d, c = self.dec, self.dcfg
        f = ops.linear(d._as_act(self._feat, "bf16"), self.w.fc)
        a = d._norm_act(f, self.w.hidden_norm, "bf16")
        for li, lw in enumerate(self.w.layers):
            m = lw.mixer
            qkv = ops.linear(a, m.qkv)
            ops.qk_norm_rope_kvwrite(
                qkv, Hq=m.heads, Hkv=m.kv_heads, D=c.head_dim, positions=batch.positions, slots=batch.slot_mapping,
                k_cache=self.kv.k[li], v_cache=self.kv.v[li], q_norm_w=m.q_norm, k_norm_w=m.k_norm,
                plus_one=c.norm_plus_one, eps=c.rms_eps, cos=d.cos, sin=d.sin, q_head_stride=c.head_dim,
                k_scale=self.kv.k_scale[li], v_scale=self.kv.v_scale[li])
        self._feat = None

    # ------------------------------------------------------------------ proposal
    def propose(self, seqs, k: int) -> List[List[int]]:
        """`seqs`: running sequences whose newest token has no target hidden state yet. Returns
        up to `k` drafts per sequence (fewer when its KV blocks do not reach that far)."""
        bs = self.runner.block_size
        k = min(k, self.dc.gamma)
        items, widths = [], []
        for s in seqs:
            p1 = len(s.tokens) - 1                          # position of the newest token (the anchor row)
            room = len(s.blocks) * bs - 1 - p1              # positions available after the anchor
            g = max(0, min(k, room))
            widths.append(g)
            if g == 0:
                continue
            total = p1 + 1 + g                              # every block row sees the context and the whole block
            for j in range(g + 1):
                items.append(dict(tokens=[s.tokens[-1] if j == 0 else self.dc.mask_token_id], start_pos=p1 + j,
                                  blocks=s.blocks, state_slot=0, ctx=total))
        if not items:
            return [[] for _ in seqs]
        b = ForwardBatch.build(items, bs, device=self.device, max_blocks=self.runner.max_blocks)
        ctx = torch.tensor([it["ctx"] for it in items], dtype=torch.int32, device=self.device)
        b.ctx_len, b.max_ctx = ctx, max(it["ctx"] for it in items)
        d = self.dec
        x = self.target.embed(b.token_ids)
        for li, lw in enumerate(self.w.layers):
            x = d.layer(li, x, lw, b, self.caches)
        lg = self.target.logits(x, final_norm=self.w.norm)
        ids = ops.argmax(lg).tolist()
        self.proposals += 1
        out, r = [], 0
        for g in widths:
            if g == 0:
                out.append([])
                continue
            out.append([int(t) for t in ids[r + 1:r + 1 + g]])
            r += g + 1
        return out
