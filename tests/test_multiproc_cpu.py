"""Multi-process CPU tests (gloo, world size 2): tensor-parallel parity of the sharded engine,
the rank-0 control plane with follower ranks, and failure detection when a rank leaves.
Failures are made on the host only (a rank that exits between steps); no device is involved.
Mirrors the reference's multi-rank protocol tests (``crates/comm/tests``, TP worker loop)."""
import json
import os
import socket
import subprocess
import sys

import pytest

from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.sampling.params import SamplingParams

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "multi_cpu", "tp_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(scenario, tmp_path, world=2, timeout=240):
    out = str(tmp_path / "res")
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE) + os.pathsep + os.environ.get("PYTHONPATH", ""),
               OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), WORKER, scenario, out]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    res = {}
    for r in range(world):
        path = f"{out}.{r}"
        if os.path.exists(path):
            res[r] = json.load(open(path))
    return p, res


def _single_rank_ids():
    import importlib.util
    spec = importlib.util.spec_from_file_location("tp_worker", WORKER)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    eng = LLMEngine(EngineArgs(model="tiny-dense", device="cpu", max_num_seqs=4, max_model_len=128, use_cuda_graphs=False))
    return [o.output_ids for o in eng.generate(mod.prompts(), SamplingParams(max_tokens=6, temperature=0.0))]


def test_two_rank_tp_matches_single_rank(tmp_path):
    p, res = _run("parity", tmp_path)
    assert p.returncode == 0, p.stderr[-2000:]
    assert res[0]["ids"] == res[1]["ids"]
    assert res[0]["ids"] == _single_rank_ids()


@pytest.mark.parametrize("family", ["tiny-hybrid-moe", "tiny-nemotron-h", "tiny-kimi-linear"])
def test_two_rank_tp_matches_single_rank_for_hybrid_families(tmp_path, family):
    """Gated-delta-net + MoE and Mamba2 hybrids sharded over two ranks (heads, groups, conv
    channels, expert widths; the MoE output joins the residual through the deferred sum) give the
    single-rank tokens. bf16 weights: with fp8 the shards are quantised separately."""
    import importlib.util
    from metrale_inference_alpha_b200.config.model_config import preset
    p, res = _run(f"parity:{family}", tmp_path)
    assert p.returncode == 0, p.stderr[-2000:]
    assert res[0]["ids"] == res[1]["ids"]
    spec = importlib.util.spec_from_file_location("tp_worker", WORKER)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    eng = LLMEngine(EngineArgs(model=preset(family, weight_format="bf16"), device="cpu", max_num_seqs=4, max_model_len=128,
                               use_cuda_graphs=False))
    want = [o.output_ids for o in eng.generate(mod.prompts(), SamplingParams(max_tokens=6, temperature=0.0))]
    # the cross-rank sum rounds the bf16 partials in a different order than one full-K product, so
    # a random-weight model may flip a late near-tie: the first tokens must agree exactly
    got = res[0]["ids"]
    assert [g[:3] for g in got] == [w[:3] for w in want]
    same = sum(a == b for g, w in zip(got, want) for a, b in zip(g, w))
    assert same >= 0.7 * sum(len(w) for w in want)


def test_control_plane_keeps_followers_in_lockstep(tmp_path):
    p, res = _run("control", tmp_path)
    assert p.returncode == 0, p.stderr[-2000:]
    done = res[0]["done"]
    ref = _single_rank_ids()
    assert [done[f"q{i}"][0] for i in range(3)] == ref
    assert done["victim"][1] == "abort"
    assert res[1]["ended"] == "shutdown"
    assert res[1]["ticks"] == res[0]["ticks"]


def test_rank_leaving_between_steps_is_detected_on_the_host(tmp_path):
    p, res = _run("leave", tmp_path)
    assert p.returncode == 0, p.stderr[-2000:]
    assert res[1]["left_at"] == 3
    assert "peer_lost" in res[0] and res[0]["fault"]
    assert res[0]["steps"] <= 4                      # it stopped before launching further work


def test_poisoned_communicator_refuses_then_reconnects(tmp_path):
    p, res = _run("reconnect", tmp_path)
    assert p.returncode == 0, p.stderr[-2000:]
    for r in (0, 1):
        assert res[r]["before"] == [2.0] * 4 and res[r]["refused"] is True
        assert res[r]["reconnected"] is True and res[r]["healthy"] is True
        assert res[r]["after"] == [3.0] * 4


def test_rank0_http_app_drives_follower_ranks(tmp_path):
    p, res = _run("serve", tmp_path)
    assert p.returncode == 0, p.stderr[-2000:]
    assert res[0]["status"] == 200 and res[0]["ids"] == _single_rank_ids()[0]
    assert res[1]["ended"] == "shutdown"
