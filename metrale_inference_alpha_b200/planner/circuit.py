"""Declarative op graphs ("circuits") of a model family: load, instantiate for a configuration, fuse by
rule, plan activation buffers, and check checkpoint bindings.

A circuit file (TOML, ``planner/circuits/*.toml``) names blocks; a block is a list of nodes, each an op
with input edges, output edges (format + symbolic ``rows x cols`` shape over the configuration's
dimensions) and the checkpoint modules it binds (``{L}`` = the layer's module path), plus the per-sequence
state it touches. ``layers`` gives the block pattern that repeats over the model's layers.

``instantiate`` evaluates every shape for a configuration and a row count and returns the flat graph of one
step (embed, every layer, head) with byte sizes. ``fuse`` applies the file's fusion rules — a chain of ops
whose intermediate edges have exactly one consumer collapses into one node, longest rule first — which is
how the graph's launch count is compared with the engine's. ``plan_buffers`` does liveness analysis over
the (fused) graph and packs the edges into one arena with a first-fit allocator, so the peak activation
footprint of a step is known before anything is allocated. ``check_bindings`` resolves every binding of
every layer against a checkpoint's tensor names.

Reference: ``crates/circuit/src/{circuit_toml,instantiate,fuser,fuser_match,planner,model_buffer,dims}.rs``
and ``kernels/circuits/*.toml``.
"""
from __future__ import annotations

import ast
import operator
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

CIRCUIT_DIR = Path(__file__).resolve().parent / "circuits"
FORMAT_BYTES = {"bf16": 2.0, "f16": 2.0, "f32": 4.0, "i32": 4.0, "fp8": 1.0, "fp8_row": 1.0, "fp8_g128": 1.0 + 4.0 / 128,
                "nvfp4": 0.5 + 1.0 / 16, "u8": 1.0}


class CircuitError(ValueError):
    pass


@dataclass
class Edge:
    name: str
    format: str
    shape: str
    rows: int = 0
    cols: int = 0

    @property
    def nbytes(self) -> int:
        return int(self.rows * self.cols * FORMAT_BYTES[self.format] + 0.999)


@dataclass
class Node:
    id: str
    op: str
    inputs: List[str]
    outputs: List[Edge]
    binding: List[str] = field(default_factory=list)
    state: List[str] = field(default_factory=list)
    fused_from: List[str] = field(default_factory=list)


@dataclass
class Circuit:
    name: str
    description: str
    blocks: Dict[str, dict]
    layers: List[str]
    fusions: List[Tuple[str, List[str]]]


# ----------------------------------------------------------------------------- loading
def load(name_or_path) -> Circuit:
    p = Path(name_or_path)
    if not p.exists():
        p = CIRCUIT_DIR / f"{name_or_path}.toml"
    if not p.exists():
        raise CircuitError(f"no circuit {name_or_path!r}")
    d = tomllib.loads(p.read_text())
    if d.get("schema") != 1:
        raise CircuitError(f"{p.name}: unsupported schema {d.get('schema')!r}")
    blocks = d.get("block") or {}
    for bname, b in blocks.items():
        ids = [n.get("id") for n in b.get("node", [])]
        if len(set(ids)) != len(ids) or None in ids:
            raise CircuitError(f"block {bname}: node ids must be present and unique")
        produced = set([b["stream_in"]] if b.get("stream_in") else [])
        for n in b.get("node", []):
            for e in n.get("in", []):
                if e not in produced:
                    raise CircuitError(f"block {bname}: node {n['id']} reads edge {e!r} before anything writes it")
            for o in n.get("out", []):
                if not {"edge", "format", "shape"} <= set(o):
                    raise CircuitError(f"block {bname}: node {n['id']} has an output without edge / format / shape")
                if o["edge"] in produced:
                    raise CircuitError(f"block {bname}: edge {o['edge']!r} is written twice")
                produced.add(o["edge"])
            for s in n.get("state", []):
                if s not in {x["id"] for x in b.get("state", [])}:
                    raise CircuitError(f"block {bname}: node {n['id']} touches undeclared state {s!r}")
        if b.get("stream_out") and b["stream_out"] not in produced:
            raise CircuitError(f"block {bname}: stream_out {b['stream_out']!r} is never written")
    layers = list(d.get("layers") or [])
    for l in layers:
        if l not in blocks:
            raise CircuitError(f"layer pattern names unknown block {l!r}")
    fus = [(f["name"], list(f["pattern"])) for f in d.get("fusion", [])]
    return Circuit(p.stem, d.get("description", ""), blocks, layers, fus)


# ----------------------------------------------------------------------------- dims and shapes
_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.FloorDiv: operator.floordiv}


def eval_dim(expr: str, dims: Dict[str, int]) -> int:
    """Integer arithmetic over named dims (+ - * // and parentheses only)."""
    def ev(n):
        if isinstance(n, ast.Constant) and isinstance(n.value, int):
            return n.value
        if isinstance(n, ast.Name):
            if n.id not in dims:
                raise CircuitError(f"unknown dim {n.id!r} in {expr!r}")
            return int(dims[n.id])
        if isinstance(n, ast.BinOp) and type(n.op) in _OPS:
            return _OPS[type(n.op)](ev(n.left), ev(n.right))
        raise CircuitError(f"unsupported expression {expr!r}")
    return ev(ast.parse(expr.strip(), mode="eval").body)


def dims_of(cfg, n: int) -> Dict[str, int]:
    """The dims a circuit may name, from a ModelConfig and the step's row count."""
    d = {"n": n, "hidden": cfg.hidden_size, "vocab": cfg.vocab_size, "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
         "head_dim": cfg.head_dim, "q_size": cfg.num_heads * cfg.head_dim, "kv_size": cfg.num_kv_heads * cfg.head_dim,
         "intermediate": cfg.intermediate_size, "layers": cfg.num_layers}
    for k in ("gdn_k_heads", "gdn_v_heads", "gdn_k_dim", "gdn_v_dim", "num_experts", "experts_per_token", "moe_intermediate_size",
              "mamba_heads", "mamba_head_dim", "mamba_state", "kv_lora_rank", "qk_rope_dim", "conv_kernel"):
        d[k] = int(getattr(cfg, k, 0) or 0)
    return d


def formats_of(cfg) -> Dict[str, str]:
    from ..ops import ACT_FOR_WEIGHT
    return {"act_format": ACT_FOR_WEIGHT.get(cfg.weight_format, "bf16"), "kv_format": "fp8" if cfg.kv_dtype == "fp8" else "bf16",
            "weight_format": cfg.weight_format}


def _edge(o: dict, dims, fmts, prefix: str) -> Edge:
    fmt = o["format"].format(**fmts) if "{" in o["format"] else o["format"]
    if fmt not in FORMAT_BYTES:
        raise CircuitError(f"unknown format {fmt!r}")
    parts = o["shape"].split(" x ")
    if len(parts) != 2:
        raise CircuitError(f"shape {o['shape']!r} must be 'rows x cols'")
    return Edge(prefix + o["edge"], fmt, o["shape"], eval_dim(parts[0], dims), eval_dim(parts[1], dims))


def instantiate(circuit: Circuit, cfg, n: int, layer_path: str = "model.layers.{i}") -> List[Node]:
    """The flat graph of one step: embed, num_layers x the layer pattern, head. Edge names are prefixed
    with their layer (``L3.xq``); the stream edge of a block feeds the next block."""
    dims, fmts = dims_of(cfg, n), formats_of(cfg)
    out: List[Node] = []
    stream: Optional[str] = None

    def emit(bname: str, prefix: str, L: str):
        nonlocal stream
        b = circuit.blocks[bname]
        rename = {b["stream_in"]: stream} if b.get("stream_in") and stream else {}
        for nd in b.get("node", []):
            outs = [_edge(o, dims, fmts, prefix) for o in nd.get("out", [])]
            ins = [rename.get(e, prefix + e) for e in nd.get("in", [])]
            out.append(Node(prefix + nd["id"], nd["op"], ins, outs, [x.replace("{L}", L) for x in nd.get("binding", [])],
                            [prefix + s for s in nd.get("state", [])]))
        if b.get("stream_out"):
            stream = prefix + b["stream_out"]

    if "embed" in circuit.blocks:
        emit("embed", "", "")
    if circuit.layers:
        for i in range(cfg.num_layers):
            emit(circuit.layers[i % len(circuit.layers)], f"L{i}.", layer_path.format(i=i))
    if "head" in circuit.blocks:
        emit("head", "", "")
    return out


# ----------------------------------------------------------------------------- fusion
def fuse(nodes: Sequence[Node], rules: Sequence[Tuple[str, List[str]]], keep: Iterable[str] = ()) -> List[Node]:
    """Collapse chains that match a rule. A chain node k+1 must read an output of node k, and every edge
    between chain members must have no reader outside the chain (and not be in ``keep``)."""
    readers: Dict[str, int] = {}
    for nd in nodes:
        for e in nd.inputs:
            readers[e] = readers.get(e, 0) + 1
    keep = set(keep)
    rules = sorted(rules, key=lambda r: -len(r[1]))
    out: List[Node] = []
    i = 0
    nodes = list(nodes)
    while i < len(nodes):
        hit = None
        for name, pat in rules:
            chain = nodes[i:i + len(pat)]
            if len(chain) < len(pat) or [c.op for c in chain] != pat:
                continue
            ok = True
            for a, b in zip(chain, chain[1:]):
                link = [o.name for o in a.outputs if o.name in b.inputs]
                if not link or any(readers.get(o.name, 0) != 1 or o.name in keep for o in a.outputs):
                    ok = False
                    break
            if ok:
                hit = (name, chain)
                break
        if hit is None:
            out.append(nodes[i])
            i += 1
            continue
        name, chain = hit
        inner = {o.name for c in chain[:-1] for o in c.outputs}
        ins = []
        for c in chain:
            ins += [e for e in c.inputs if e not in inner and e not in ins]
        out.append(Node(chain[0].id, name, ins, chain[-1].outputs, [b for c in chain for b in c.binding],
                        sorted({s for c in chain for s in c.state}), [c.id for c in chain]))
        i += len(chain)
    return out


# ----------------------------------------------------------------------------- buffer planning
@dataclass
class BufferPlan:
    offsets: Dict[str, int]
    sizes: Dict[str, int]
    peak_bytes: int
    total_bytes: int            # what separate allocations of every edge would take

    def overlaps(self, live: Dict[str, Tuple[int, int]]) -> List[Tuple[str, str]]:
        bad = []
        names = list(self.offsets)
        for i, a in enumerate(names):
            for b in names[i + 1:]:
                if live[a][1] < live[b][0] or live[b][1] < live[a][0]:
                    continue
                if self.offsets[a] < self.offsets[b] + self.sizes[b] and self.offsets[b] < self.offsets[a] + self.sizes[a]:
                    bad.append((a, b))
        return bad


def liveness(nodes: Sequence[Node], outputs: Iterable[str] = ()) -> Dict[str, Tuple[int, int]]:
    """edge -> (index of the node that writes it, index of its last reader); graph outputs live to the end."""
    live: Dict[str, List[int]] = {}
    for i, nd in enumerate(nodes):
        for o in nd.outputs:
            live[o.name] = [i, i]
        for e in nd.inputs:
            if e in live:
                live[e][1] = i
    for e in outputs:
        if e in live:
            live[e][1] = len(nodes)
    return {k: (v[0], v[1]) for k, v in live.items()}


def plan_buffers(nodes: Sequence[Node], outputs: Iterable[str] = (), align: int = 256) -> BufferPlan:
    """First-fit packing of the edges into one arena: edges are placed in order of their first write,
    each at the lowest aligned offset where it collides with no edge that is alive at the same time."""
    live = liveness(nodes, outputs)
    size = {o.name: (o.nbytes + align - 1) // align * align for nd in nodes for o in nd.outputs}
    placed: List[Tuple[str, int]] = []
    offsets: Dict[str, int] = {}
    for name in sorted(size, key=lambda n: (live[n][0], -size[n])):
        busy = sorted((offsets[o], offsets[o] + size[o]) for o, _ in placed
                      if not (live[o][1] < live[name][0] or live[name][1] < live[o][0]))
        at = 0
        for lo, hi in busy:
            if at + size[name] <= lo:
                break
            at = max(at, hi)
        offsets[name] = at
        placed.append((name, at))
    peak = max((offsets[n] + size[n] for n in size), default=0)
    return BufferPlan(offsets, size, peak, sum(size.values()))


# ----------------------------------------------------------------------------- bindings
def check_bindings(nodes: Sequence[Node], names: Iterable[str]) -> List[str]:
    """Bindings that resolve to no tensor of the checkpoint (a module binds when any tensor name starts
    with ``<module>.``)."""
    have = set(names)
    mods = {n.rsplit(".", 1)[0] for n in have}
    return sorted({b for nd in nodes for b in nd.binding if b not in mods and b not in have})


def summary(circuit: Circuit, cfg, n: int) -> dict:
    g = instantiate(circuit, cfg, n)
    f = fuse(g, circuit.fusions)
    plan = plan_buffers(f, outputs=[f[-1].outputs[0].name] if f else [])
    return {"circuit": circuit.name, "rows": n, "ops": len(g), "launches_after_fusion": len(f),
            "activation_bytes_separate": plan.total_bytes, "activation_bytes_planned": plan.peak_bytes,
            "fused": sorted({nd.op for nd in f if nd.fused_from})}
