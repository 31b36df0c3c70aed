"""Determinism gates (bench/determinism.py) on the tiny models: known-answer equality regardless of
engine history, and replay equality on recurrent models whose state slots are recycled in between.
Mirrors the reference's ``kat-equality-gate`` and ``ssm-state-poisoning-gate``."""
import pytest

from metrale_inference_alpha_b200.bench import determinism
from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine


def _factory(model, device):
    return lambda: LLMEngine(EngineArgs(model=preset(model), device=device, max_num_seqs=4, max_model_len=256,
                                        num_kv_blocks=40))


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
@pytest.mark.parametrize("model,seeded", [("tiny-dense", False), ("tiny-dense", True), ("tiny-hybrid-moe", False)])
def test_known_answers_do_not_depend_on_history(model, seeded, device):
    rec = determinism.kat_equality(_factory(model, device), n=3, prompt_len=36, max_tokens=12, seeded=seeded)
    assert rec.value == 1.0, rec.config["mismatch"]


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
@pytest.mark.parametrize("model", ["tiny-hybrid-moe", "tiny-nemotron-h"])
def test_replays_on_recurrent_models_are_identical(model, device):
    rec = determinism.state_poisoning(_factory(model, device), replays=6 if device == "cpu" else 12, prompt_len=40,
                                      max_tokens=10)
    assert rec.value == 1.0, rec.config["mismatch"]
    assert rec.config["recurrent_layers"] > 0
