"""NLLB / M2M-100 encoder-decoder translation model with beam search.

Architecture (HF ``M2M100ForConditionalGeneration`` tensor names): shared token embedding scaled by
sqrt(d_model), sinusoidal positions (offset 2, the padding index keeps a zero row), pre-LayerNorm
encoder layers (self-attention with biases, ReLU feed-forward) with a final LayerNorm, decoder layers
with causal self-attention over a growing cache, cross-attention over the encoder output (its keys and
values are projected once per translation) and a feed-forward block, final LayerNorm, LM head tied to
the embedding.

Generation: the decoder starts from ``</s>``, the first generated token is forced to the target
language code, and beam search keeps ``num_beams`` hypotheses with the usual length-normalised score
(sum of log-probs / length ** length_penalty); finished hypotheses leave the beam, the search stops
when the best running beam can no longer beat the worst kept hypothesis or at ``max_new_tokens``. The
per-step candidate selection is one top-k over ``beams x vocab`` on the device.

The GEMMs go through ``ops.linear`` (tcgen05 bf16 kernel) on a GPU; attention over these short
sequences is ``scaled_dot_product_attention``. Reference: the NLLB encoder-decoder path of
``crates/model-engine`` and ``kernels/gb10/common/nllb_encoder.cu`` (23 kernels incl. the beam top-k).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F


@dataclass
class NllbConfig:
    vocab_size: int = 256206
    d_model: int = 1024
    encoder_layers: int = 12
    decoder_layers: int = 12
    encoder_attention_heads: int = 16
    decoder_attention_heads: int = 16
    encoder_ffn_dim: int = 4096
    decoder_ffn_dim: int = 4096
    max_position_embeddings: int = 1024
    scale_embedding: bool = True
    pad_token_id: int = 1
    eos_token_id: int = 2
    decoder_start_token_id: int = 2
    activation_function: str = "relu"

    @staticmethod
    def from_hf(d: dict) -> "NllbConfig":
        if d.get("model_type") not in ("m2m_100", "nllb", None):
            raise ValueError(f"not an M2M-100 / NLLB configuration: {d.get('model_type')!r}")
        keys = NllbConfig.__dataclass_fields__
        return NllbConfig(**{k: d[k] for k in keys if k in d})


def sinusoidal_table(n: int, dim: int, padding_idx: int) -> torch.Tensor:
    """fairseq-style table: [sin | cos] halves, row ``padding_idx`` zero."""
    half = dim // 2
    freq = torch.exp(torch.arange(half, dtype=torch.float32) * -(math.log(10000.0) / (half - 1)))
    ang = torch.arange(n, dtype=torch.float32)[:, None] * freq[None, :]
    tab = torch.cat([torch.sin(ang), torch.cos(ang)], 1)
    if dim % 2:
        tab = torch.cat([tab, torch.zeros(n, 1)], 1)
    tab[padding_idx] = 0
    return tab


class NllbModel:
    def __init__(self, cfg: NllbConfig, tensors: Dict[str, torch.Tensor], device="cpu"):
        from ..ops import QuantWeight
        self.cfg, self.device = cfg, torch.device(device)
        cuda = self.device.type == "cuda"
        t = {k[6:] if k.startswith("model.") else k: v for k, v in tensors.items()}
        emb = t.get("shared.weight", t.get("encoder.embed_tokens.weight"))
        if emb is None:
            raise KeyError("shared.weight")
        self.embed = emb.to(self.device).to(torch.bfloat16 if cuda else torch.float32)
        self.scale = math.sqrt(cfg.d_model) if cfg.scale_embedding else 1.0
        self.pos = sinusoidal_table(cfg.max_position_embeddings + 2, cfg.d_model, cfg.pad_token_id).to(self.device)

        def lin(name):
            w, b = t[name + ".weight"].to(self.device), t[name + ".bias"].to(self.device).float()
            return (QuantWeight("bf16", w.shape[0], w.shape[1], w.to(torch.bfloat16).contiguous()) if cuda else w.float()), b

        def ln(name):
            return t[name + ".weight"].to(self.device).float(), t[name + ".bias"].to(self.device).float()

        def attn(p):
            # q | k | v fused into one projection where the three read the same input
            ws = [t[f"{p}.{n}_proj.weight"] for n in "qkv"]
            bs = [t[f"{p}.{n}_proj.bias"] for n in "qkv"]
            return dict(q=lin(f"{p}.q_proj"), k=lin(f"{p}.k_proj"), v=lin(f"{p}.v_proj"), o=lin(f"{p}.out_proj"),
                        qkv=self._fuse(ws, bs, cuda), kv=self._fuse(ws[1:], bs[1:], cuda))

        self.enc = [dict(attn=attn(f"encoder.layers.{i}.self_attn"), ln1=ln(f"encoder.layers.{i}.self_attn_layer_norm"),
                         fc1=lin(f"encoder.layers.{i}.fc1"), fc2=lin(f"encoder.layers.{i}.fc2"),
                         ln2=ln(f"encoder.layers.{i}.final_layer_norm")) for i in range(cfg.encoder_layers)]
        self.enc_ln = ln("encoder.layer_norm")
        self.dec = [dict(attn=attn(f"decoder.layers.{i}.self_attn"), ln1=ln(f"decoder.layers.{i}.self_attn_layer_norm"),
                         cross=attn(f"decoder.layers.{i}.encoder_attn"), lnx=ln(f"decoder.layers.{i}.encoder_attn_layer_norm"),
                         fc1=lin(f"decoder.layers.{i}.fc1"), fc2=lin(f"decoder.layers.{i}.fc2"),
                         ln2=ln(f"decoder.layers.{i}.final_layer_norm")) for i in range(cfg.decoder_layers)]
        self.dec_ln = ln("decoder.layer_norm")
        head = t.get("lm_head.weight")
        hw = (head if head is not None else emb).to(self.device)
        self.head = (QuantWeight("bf16", hw.shape[0], hw.shape[1], hw.to(torch.bfloat16).contiguous()) if cuda else hw.float()), None

    def _fuse(self, ws, bs, cuda):
        from ..ops import QuantWeight
        w = torch.cat([x.to(self.device) for x in ws], 0)
        b = torch.cat([x.to(self.device).float() for x in bs], 0)
        return (QuantWeight("bf16", w.shape[0], w.shape[1], w.to(torch.bfloat16).contiguous()) if cuda else w.float()), b

    # ------------------------------------------------------------------ pieces
    def _linear(self, x, wb):
        w, b = wb
        shp = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if self.device.type == "cuda":
            from .. import ops
            xa = x2.to(torch.bfloat16).contiguous()
            y = ops.linear(ops.Act("bf16", xa.shape[0], xa.shape[1], xa, bf16=xa), w, out_f32=True)
        else:
            y = x2.float() @ w.T
        if b is not None:
            y = y + b
        return y.view(*shp, -1)

    def _embed(self, ids: torch.Tensor, past: int = 0) -> torch.Tensor:
        """Token embedding * scale + sinusoidal position (positions count non-padding tokens from 2)."""
        c = self.cfg
        mask = (ids != c.pad_token_id).long()
        pos = (torch.cumsum(mask, 1) + past) * mask + c.pad_token_id
        return self.embed[ids].float() * self.scale + self.pos[pos]

    def _heads(self, x, H):
        B, T, E = x.shape
        return x.view(B, T, H, E // H).transpose(1, 2)

    def _ffn(self, x, L):
        act = F.relu if self.cfg.activation_function == "relu" else F.gelu
        return self._linear(act(self._linear(x, L["fc1"])), L["fc2"])

    def encode(self, src: torch.Tensor) -> dict:
        """``src`` [B, S] (padded with pad_token_id) -> encoder state for ``decode_step`` / ``translate``."""
        c = self.cfg
        H = c.encoder_attention_heads
        src = src.to(self.device)
        x = self._embed(src)
        key_mask = (src != c.pad_token_id)[:, None, None, :]                         # [B, 1, 1, S]
        for L in self.enc:
            h = F.layer_norm(x, (c.d_model,), *L["ln1"])
            q, k, v = self._linear(h, L["attn"]["qkv"]).chunk(3, -1)
            a = F.scaled_dot_product_attention(self._heads(q, H), self._heads(k, H), self._heads(v, H), attn_mask=key_mask)
            x = x + self._linear(a.transpose(1, 2).reshape(x.shape), L["attn"]["o"])
            x = x + self._ffn(F.layer_norm(x, (c.d_model,), *L["ln2"]), L)
        x = F.layer_norm(x, (c.d_model,), *self.enc_ln)
        Hd = c.decoder_attention_heads
        cross = []
        for L in self.dec:                                                          # cross-attention K / V once per translation
            k, v = self._linear(x, L["cross"]["kv"]).chunk(2, -1)
            cross.append((self._heads(k, Hd), self._heads(v, Hd)))
        return dict(hidden=x, mask=key_mask, cross=cross)

    def new_cache(self) -> list:
        return [None] * self.cfg.decoder_layers

    def decode_step(self, tokens: torch.Tensor, enc: dict, cache: list, past: int) -> torch.Tensor:
        """``tokens`` [B, n] continuing ``past`` cached positions -> logits [B, n, vocab] (fp32). The cache
        (per layer K / V [B, H, past, D]) is extended in place."""
        c = self.cfg
        H = c.decoder_attention_heads
        x = self._embed(tokens.to(self.device), past)
        n = tokens.shape[1]
        for i, L in enumerate(self.dec):
            h = F.layer_norm(x, (c.d_model,), *L["ln1"])
            q, k, v = (self._heads(z, H) for z in self._linear(h, L["attn"]["qkv"]).chunk(3, -1))
            if cache[i] is not None:
                k, v = torch.cat([cache[i][0], k], 2), torch.cat([cache[i][1], v], 2)
            cache[i] = (k, v)
            causal = None
            if n > 1:
                T = k.shape[2]
                causal = torch.ones(n, T, dtype=torch.bool, device=self.device).tril(T - n)
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=causal)
            x = x + self._linear(a.transpose(1, 2).reshape(x.shape), L["attn"]["o"])
            h = F.layer_norm(x, (c.d_model,), *L["lnx"])
            q = self._heads(self._linear(h, L["cross"]["q"]), H)
            ck, cv = enc["cross"][i]
            a = F.scaled_dot_product_attention(q, ck, cv, attn_mask=enc["mask"])
            x = x + self._linear(a.transpose(1, 2).reshape(x.shape), L["cross"]["o"])
            x = x + self._ffn(F.layer_norm(x, (c.d_model,), *L["ln2"]), L)
        x = F.layer_norm(x, (c.d_model,), *self.dec_ln)
        return self._linear(x, self.head).float()

    # ------------------------------------------------------------------ beam search
    @torch.no_grad()
    def translate(self, src_ids: Sequence[int], tgt_lang_id: int, *, num_beams: int = 4, max_new_tokens: int = 200,
                  length_penalty: float = 1.0) -> List[int]:
        """One sentence (token ids ending in ``</s>``, source language code first) -> the best hypothesis'
        token ids after the target language code, without the closing ``</s>``."""
        c = self.cfg
        dev = self.device
        B = num_beams
        enc = self.encode(torch.tensor([list(src_ids)], dtype=torch.long))
        enc = dict(hidden=enc["hidden"].expand(B, -1, -1), mask=enc["mask"].expand(B, -1, -1, -1),
                   cross=[(k.expand(B, -1, -1, -1), v.expand(B, -1, -1, -1)) for k, v in enc["cross"]])
        cache = self.new_cache()
        seqs = torch.full((B, 1), c.decoder_start_token_id, dtype=torch.long, device=dev)
        scores = torch.full((B,), float("-inf"), device=dev)
        scores[0] = 0.0                                               # all beams start identical: keep one alive
        done: List[tuple] = []                                        # (normalised score, ids)
        last = seqs
        for step in range(max_new_tokens + 1):
            logp = torch.log_softmax(self.decode_step(last, enc, cache, seqs.shape[1] - last.shape[1])[:, -1], -1)
            if step == 0:                                             # the target language code is forced
                forced = torch.full_like(logp, float("-inf"))
                forced[:, tgt_lang_id] = 0.0
                logp = forced
            if step == max_new_tokens:                                # out of budget: every beam must close
                forced = torch.full_like(logp, float("-inf"))
                forced[:, c.eos_token_id] = logp[:, c.eos_token_id]
                logp = forced
            cand = (scores[:, None] + logp).view(-1)
            top, idx = torch.topk(cand, 2 * B)                        # 2B candidates so that B survive the finished ones
            beam, tok = idx // logp.shape[1], idx % logp.shape[1]
            keep_b, keep_t, keep_s = [], [], []
            for s, b, t in zip(top.tolist(), beam.tolist(), tok.tolist()):
                if s == float("-inf"):
                    continue
                if t == c.eos_token_id:
                    length = seqs.shape[1] + 1
                    done.append((s / (length ** length_penalty), seqs[b].tolist() + [t]))
                elif len(keep_b) < B:
                    keep_b.append(b)
                    keep_t.append(t)
                    keep_s.append(s)
                if len(keep_b) == B:
                    break
            if not keep_b:
                break
            if len(done) >= B:
                done.sort(key=lambda x: -x[0])
                done = done[:B]
                # a running beam can at best keep its score: stop when none can reach the kept hypotheses
                best_running = keep_s[0] / ((seqs.shape[1] + 1) ** length_penalty)
                if best_running <= done[-1][0]:
                    break
            while len(keep_b) < B:                                    # dead slots (kept at -inf) so that shapes stay fixed
                keep_b.append(keep_b[0])
                keep_t.append(keep_t[0])
                keep_s.append(float("-inf"))
            bi = torch.tensor(keep_b, device=dev)
            seqs = torch.cat([seqs[bi], torch.tensor(keep_t, device=dev)[:, None]], 1)
            scores = torch.tensor(keep_s, device=dev)
            cache = [(k[bi], v[bi]) for k, v in cache]
            last = seqs[:, -1:]
        if not done:
            done = [(float(scores[0]), seqs[0].tolist() + [c.eos_token_id])]
        best = max(done, key=lambda x: x[0])[1]
        return best[2:-1] if len(best) > 2 and best[1] == tgt_lang_id else best[1:-1]
