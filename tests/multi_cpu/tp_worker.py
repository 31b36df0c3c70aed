"""One CPU rank of a gloo tensor-parallel engine. Scenarios (argv[1]):
  parity   every rank runs the same requests through a TP-sharded tiny model; rank 0 writes
           the generated ids so the parent can compare them with a single-rank run.
  control  rank 0 plays the HTTP owner: it publishes add / abort / shutdown operations over the
           control plane; followers run ``follower_loop``; all ranks must generate the same ids.
  leave    the last rank announces an orderly exit between steps; the others learn it from the
           heartbeat store before their next collective and stop with ``PeerLost``.
Launched by tests/test_multiproc_cpu.py via torch.distributed.run on 127.0.0.1."""
import json
import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
from metrale_inference_alpha_b200.parallel.control import ControlPlane, PeerLost, follower_loop
from metrale_inference_alpha_b200.parallel.tp import GlooTpContext
from metrale_inference_alpha_b200.sampling.params import SamplingParams


def prompts():
    return [[(7 * i + 3 * j) % 250 + 1 for j in range(9 + i)] for i in range(3)]


def main():
    scenario, out_path = sys.argv[1], sys.argv[2]
    dist.init_process_group("gloo", timeout=timedelta(seconds=30))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.set_num_threads(1)
    tp = GlooTpContext(rank, world)
    model = "tiny-dense"
    if scenario.startswith("parity:"):                 # parity:<preset>: another family, in bf16 (sharding only, no per-shard quantisation noise)
        from metrale_inference_alpha_b200.config.model_config import preset
        model, scenario = preset(scenario.split(":", 1)[1], weight_format="bf16"), "parity"
    eng = LLMEngine(EngineArgs(model=model, device="cpu", max_num_seqs=4, max_model_len=128, tp_size=world,
                               use_cuda_graphs=False), tp=tp)
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    result = {"rank": rank}
    if scenario == "parity":
        outs = eng.generate(prompts(), sp)
        result["ids"] = [o.output_ids for o in outs]
    elif scenario == "control":
        cp = ControlPlane.create(timeout_s=20.0)
        if rank == 0:
            ops = [("add", f"q{i}", p, sp) for i, p in enumerate(prompts())]
            done = {}
            ops.append(("add", "victim", prompts()[0], SamplingParams(max_tokens=64)))
            first = True
            while first or eng.has_work():
                for kind, rid, ids, params in cp.exchange(ops):
                    if kind == "add":
                        eng.add_request(ids, params, request_id=rid)
                    elif kind == "abort":
                        eng.abort(rid)
                ops = [("abort", "victim", None, None)] if first else []
                first = False
                for o in eng.step():
                    if o.finished:
                        done[o.request_id] = (o.output_ids, o.finish_reason)
            cp.exchange([("shutdown", None, None, None)])
            cp.leave()
            result["done"] = done
        else:
            result["ended"] = follower_loop(eng, cp)
        result["ticks"] = cp.ticks
    elif scenario == "leave":
        cp = ControlPlane.create(timeout_s=5.0)
        cp.heartbeat_s, cp.dead_after_s = 0.1, 1.0
        eng.add_request(prompts()[0], SamplingParams(max_tokens=100))
        steps = 0
        try:
            while eng.has_work():
                if rank == world - 1 and steps == 3:
                    cp.leave()                       # between steps: nothing of this rank is in flight
                    result["left_at"] = steps
                    break
                ok = cp.agree(True)                  # host-side rendezvous before the next launch
                cp.check_peers()
                eng.step()
                steps += 1
        except PeerLost as e:
            result["peer_lost"] = str(e)
            eng.fault.set(str(e))
        result["steps"] = steps
        result["fault"] = eng.fault.reason()
    elif scenario == "serve":
        # rank 0 owns the HTTP app (driven in-process), followers replay its operations; the chat
        # answer must equal a single-rank engine's and the followers must stop on shutdown
        cp = ControlPlane.create(timeout_s=20.0)
        if rank == 0:
            from fastapi.testclient import TestClient
            from metrale_inference_alpha_b200.server.app import ServerConfig, create_app
            from metrale_inference_alpha_b200.server.tokenizer import load_tokenizer
            tok = load_tokenizer(None, eng.cfg.vocab_size)
            with TestClient(create_app(eng, tok, ServerConfig(model_name="tp"), control=cp)) as c:
                r = c.post("/v1/completions", json={"prompt": prompts()[0], "max_tokens": 6, "temperature": 0,
                                                    "return_token_ids": True})
                result["status"] = r.status_code
                result["ids"] = r.json()["choices"][0]["token_ids"]
        else:
            result["ended"] = follower_loop(eng, cp)
    elif scenario == "reconnect":
        # a collective fails on the host (injected), the context is poisoned and refuses work; all
        # ranks reconnect and the next collective runs on the fresh group
        from metrale_inference_alpha_b200.parallel.tp import CommPoisoned
        t = torch.ones(4)
        tp.all_reduce(t)
        result["before"] = t.tolist()
        tp.poison("injected: collective timed out")
        try:
            tp.all_reduce(torch.ones(4))
            result["refused"] = False
        except CommPoisoned:
            result["refused"] = True
        result["reconnected"] = tp.attempt_reconnect(timeout_s=20.0)
        t = torch.full((4,), float(rank + 1))
        tp.all_reduce(t)
        result["after"] = t.tolist()
        result["healthy"] = tp.is_healthy()
    with open(f"{out_path}.{rank}", "w") as f:
        json.dump(result, f)
    os._exit(0)                                      # no collective teardown: a peer may be gone


if __name__ == "__main__":
    main()
