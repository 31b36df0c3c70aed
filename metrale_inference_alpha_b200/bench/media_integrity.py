"""Media integrity: an image request's reply must be a function of its own text and its own image.

The driver sends one prompt with image A, the same prompt with image A again, the same prompt with image B, and
image A once more; ``judge`` (no I/O) then requires that

* the two replies with image A that frame the run are identical (nothing image B left behind changed them),
* the repeated image-A request was served from the prefix cache (the cache is keyed by the images' digest, so
  an identical request must hit),
* the image-B request reused no cached block at or behind the first image placeholder (keys and values computed
  with image A's embeddings must never serve image B; at most the text in front of the placeholder is shared),
* the reply with image B is not identical to image A's when the run asks for that (``expect_different``: a model
  that ignores its image passes the cache rules but fails this one).

Reference: ``crates/bench/src/benchmarks/media_integrity.rs`` and ``media_integrity_responses.rs``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

from ..sampling.params import SamplingParams
from .gate import GateRecord, kernel_closure_hash


def judge(records: Sequence[dict], placeholder_index: int, block_size: int, expect_different: bool = True) -> dict:
    """``records``: [A first, A repeated, B, A last], each {"tokens", "cached_tokens"}."""
    if len(records) != 4:
        return {"pass": False, "why": f"{len(records)} of 4 requests"}
    a1, a2, b, a3 = records
    why: List[str] = []
    if a2["tokens"] != a1["tokens"] or a3["tokens"] != a1["tokens"]:
        why.append("the replies with the same image differ")
    if a2["cached_tokens"] <= 0:
        why.append("the repeated request did not hit the prefix cache")
    shared_limit = (placeholder_index // block_size) * block_size      # whole blocks of text in front of the image
    if b["cached_tokens"] > shared_limit:
        why.append(f"the other image reused {b['cached_tokens']} cached tokens, more than the {shared_limit} in front of its placeholder")
    if expect_different and b["tokens"] == a1["tokens"]:
        why.append("the reply does not depend on the image")
    return {"pass": not why, "why": "; ".join(why)}


def media_integrity(engine, prompt: Sequence[int], image_a, image_b, max_tokens: int = 8, expect_different: bool = True,
                    device: str = "") -> GateRecord:
    ph = engine.cfg.image_token_id
    if ph is None or ph not in prompt:
        raise ValueError("the prompt needs the model's image placeholder token")
    sp = SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True)
    recs = []
    for img in (image_a, image_a, image_b, image_a):
        out = engine.generate([list(prompt)], sp, images=[[img]])[0]
        recs.append({"tokens": list(out.output_ids), "cached_tokens": out.cached_tokens})
    res = judge(recs, list(prompt).index(ph), engine.args.block_size, expect_different)
    return GateRecord("media-integrity", "replies follow their own image; the cache never crosses images", 1.0 if res["pass"] else 0.0,
                      "pass", config={**res, "cached": [r["cached_tokens"] for r in recs], "model": engine.cfg.name},
                      closure=kernel_closure_hash(), device=device)
