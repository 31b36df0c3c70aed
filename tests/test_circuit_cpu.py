"""Circuit files: loading and validation, instantiation for a configuration, rule-driven fusion, buffer
planning, and bindings checked against a synthetic checkpoint of the same configuration."""
import pytest

from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.planner import circuit as C


def test_dense_circuit_instantiates_fuses_and_plans():
    cfg = preset("tiny-dense")
    circ = C.load("dense_gqa")
    g = C.instantiate(circ, cfg, n=8)
    per_layer = len(circ.blocks["layer"]["node"])
    assert len(g) == 1 + cfg.num_layers * per_layer + 3
    qkv = next(n for n in g if n.id == "L0.qkv")
    assert qkv.outputs[0].rows == 8 and qkv.outputs[0].cols == (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
    assert qkv.binding == ["model.layers.0.self_attn.q_proj", "model.layers.0.self_attn.k_proj", "model.layers.0.self_attn.v_proj"]
    # the stream edge of a block feeds the next one
    assert next(n for n in g if n.id == "L1.attn_norm").inputs == ["L0.h2"] and next(n for n in g if n.id == "final_norm").inputs == [f"L{cfg.num_layers - 1}.h2"]
    f = C.fuse(g, circ.fusions)
    ops = [n.op for n in f if n.id.startswith("L0.")]
    # eight launches per layer, the engine's own count for this family on one rank
    assert ops == ["rms_norm_quant", "linear", "qk_norm_rope_kvwrite", "attention_quant", "linear_residual", "rms_norm_quant",
                   "linear_swiglu_quant", "linear_residual"]
    fused = next(n for n in f if n.id == "L0.gate_up")
    assert fused.fused_from == ["L0.gate_up", "L0.swiglu", "L0.down_quant"] and fused.outputs[0].name == "L0.actq"
    assert len(f) < len(g)
    plan = C.plan_buffers(f, outputs=["ids"])
    live = C.liveness(f, outputs=["ids"])
    assert plan.overlaps(live) == [] and plan.peak_bytes < plan.total_bytes / 2
    s = C.summary(circ, cfg, 8)
    assert s["launches_after_fusion"] == len(f) and s["activation_bytes_planned"] == plan.peak_bytes


def test_an_edge_with_a_second_reader_blocks_fusion_and_kept_edges_survive():
    cfg = preset("tiny-dense")
    circ = C.load("dense_gqa")
    g = C.instantiate(circ, cfg, n=4)
    f = C.fuse(g, circ.fusions, keep=["L0.xn"])
    assert [n.op for n in f if n.id.startswith("L0.")][:2] == ["rms_norm", "quantize"]
    # h1 has two readers (the norm and the last residual): a rule that would swallow it mid-chain does not apply
    only = C.fuse(g, [("residual_rms_norm_quant", ["residual_add", "rms_norm", "quantize"])])
    assert not any(n.op == "residual_rms_norm_quant" for n in only)


def test_bindings_resolve_against_a_synthetic_checkpoint():
    from metrale_inference_alpha_b200.weights.source import SyntheticSource
    cfg = preset("tiny-dense")
    circ = C.load("dense_gqa")
    g = C.instantiate(circ, cfg, n=1)
    names = list(SyntheticSource(cfg, seed=0).names())
    tied = ["lm_head"] if cfg.tie_embeddings else []               # a tied head has no tensor of its own
    assert C.check_bindings(g, names) == tied
    assert C.check_bindings(g, [n for n in names if ".mlp.up_proj" not in n]) == tied + [f"model.layers.{i}.mlp.up_proj" for i in range(cfg.num_layers)]


def test_malformed_circuits_are_refused(tmp_path):
    def write(body):
        p = tmp_path / "c.toml"
        p.write_text(body)
        return p
    with pytest.raises(C.CircuitError):
        C.load(write("schema = 2\n"))
    with pytest.raises(C.CircuitError):
        C.load(write('schema = 1\n[block.a]\n[[block.a.node]]\nid = "x"\nop = "linear"\nin = ["nope"]\nout = []\n'))
    with pytest.raises(C.CircuitError):
        C.load(write('schema = 1\nlayers = ["zz"]\n'))
    with pytest.raises(C.CircuitError):
        C.load(write('schema = 1\n[block.a]\n[[block.a.node]]\nid = "x"\nop = "o"\nout = [{edge="e", format="bf16", shape="n x 4"}]\n'
                     '[[block.a.node]]\nid = "y"\nop = "o"\nout = [{edge="e", format="bf16", shape="n x 4"}]\n'))
    with pytest.raises(C.CircuitError):
        C.eval_dim("__import__('os')", {})
    assert C.eval_dim("2*kv_heads*head_dim + (n // 2)", {"kv_heads": 2, "head_dim": 8, "n": 5}) == 34
    with pytest.raises(C.CircuitError):
        C.load("no-such-circuit")
