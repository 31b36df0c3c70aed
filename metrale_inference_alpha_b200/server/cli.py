"""Command line: ``serve``, ``benchmark``, ``doctor``, ``dump-serve-options``.

Role of the reference binary's subcommands (``crates/server/src/main.rs``,
``main_modules/serve_router.rs``, ``main_modules/doctor.rs``): ``serve`` builds the engine and
the HTTP app; ``benchmark`` drives the concurrency ladder through the public engine API;
``doctor`` reports the device, driver, library and lever state without loading a model;
``dump-serve-options`` prints every option with its default as JSON.

Run as ``python -m metrale_inference_alpha_b200.server.cli <subcommand>``.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
from typing import List, Optional


def _add_engine_args(p: argparse.ArgumentParser) -> None:
    from ..engine.llm_engine import EngineArgs
    for f in dataclasses.fields(EngineArgs):
        name = "--" + f.name.replace("_", "-")
        default = f.default
        if f.name == "model":
            p.add_argument(name, default="tiny-dense", help="preset name or checkpoint directory")
        elif isinstance(default, bool):
            p.add_argument(name, default=default, action=argparse.BooleanOptionalAction)
        elif isinstance(default, int):
            p.add_argument(name, type=int, default=default)
        elif isinstance(default, float):
            p.add_argument(name, type=float, default=default)
        elif default is None:
            p.add_argument(name, type=int, default=None)
        else:
            p.add_argument(name, default=default)


def _engine_args(ns) -> "EngineArgs":
    from ..engine.llm_engine import EngineArgs
    kw = {f.name: getattr(ns, f.name) for f in dataclasses.fields(EngineArgs) if hasattr(ns, f.name)}
    return EngineArgs(**kw)


def _serve_translation(ns):
    """An m2m_100 / nllb checkpoint: the translation app instead of the decoder-only engine."""
    import uvicorn
    from transformers import AutoTokenizer
    from .translate import Translator, create_translation_app, open_translation_model
    if not (ns.nllb_src_lang and ns.nllb_tgt_lang):
        raise SystemExit("--nllb-src-lang and --nllb-tgt-lang are required for an NLLB / M2M-100 checkpoint")
    model, _ = open_translation_model(ns.model, ns.device)
    tok = AutoTokenizer.from_pretrained(ns.tokenizer or ns.model, local_files_only=True)
    tr = Translator(model, tok, ns.nllb_src_lang, ns.nllb_tgt_lang)
    uvicorn.run(create_translation_app(tr, ns.served_model_name or os.path.basename(ns.model.rstrip("/"))), host=ns.host, port=ns.port)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="metrale-b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    s = sub.add_parser("serve", help="start the HTTP server")
    _add_engine_args(s)
    s.add_argument("--recipe", default=None, help="YAML file with the model and its serve options (command line wins)")
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8888)
    s.add_argument("--served-model-name", default=None)
    s.add_argument("--tokenizer", default=None, help="directory with tokenizer.json (default: the checkpoint)")
    s.add_argument("--api-key", action="append", default=[])
    s.add_argument("--rate-limit", type=float, default=0.0, help="requests per second per key; 0 = off")
    s.add_argument("--tool-grammar", action="store_true", help="constrain tool calls with a grammar also under tool_choice=auto")
    s.add_argument("--tool-call-parser", default="hermes", choices=["hermes", "qwen3_xml", "qwen3_coder", "mistral", "gemma4", "minimax_xml", "deepseek_v4_dsml",
                            "poolside_v1", "bare_json", "json"])
    s.add_argument("--reasoning-format", default="think")
    s.add_argument("--default-max-tokens", type=int, default=1024)
    s.add_argument("--telemetry", default="basic", choices=["off", "basic", "kernel", "full"],
                   help="off | basic (counters, host-timed lanes) | kernel (CUDA-event lanes + per-kernel device time; `full` is an alias)")
    s.add_argument("--disable-thinking", action="store_true")
    s.add_argument("--tool-max-tokens", type=int, default=8192)
    s.add_argument("--lora-adapter", action="append", default=[], metavar="NAME=DIR", help="PEFT adapter to serve")
    s.add_argument("--max-loras", type=int, default=8)
    s.add_argument("--max-lora-rank", type=int, default=16)
    s.add_argument("--cache-dir", default=None, help="model cache root (default: the Hugging Face hub cache)")
    s.add_argument("--bind", default=None, metavar="HOST:PORT", help="listen address (overrides --host / --port)")
    s.add_argument("--model-name", default=None, help="alias of --served-model-name")
    s.add_argument("--max-seq-len", type=int, default=None, help="alias of --max-model-len")
    s.add_argument("--max-batch-size", type=int, default=None, help="alias of --max-num-seqs")
    s.add_argument("--request-timeout", type=float, default=None, help="alias of --request-timeout-s (seconds)")
    s.add_argument("--auth-token", action="append", default=[], help="accepted bearer token (repeatable; same as --api-key)")
    s.add_argument("--auth-tokens-file", default=None, help="file with one accepted token per line")
    s.add_argument("--require-auth", action="store_true", help="refuse to start without at least one token")
    s.add_argument("--default-top-n-sigma", type=float, default=0.0)
    s.add_argument("--default-min-p", type=float, default=0.0)
    s.add_argument("--max-thinking-budget", type=int, default=0, help="cap and default of thinking_token_budget (0 = none)")
    s.add_argument("--content-loop-watchdog", type=float, default=0.0, metavar="PENALTY",
                   help="> 0: loop penalty for requests that set no repetition_detection")
    s.add_argument("--adaptive-sampling", action="store_true",
                   help="per-token temperature from the generation zone, top-1 confidence, low-entropy runs and repetition")
    s.add_argument("--dump", default="", metavar="DIR", help="write every POST request as a JSON file into DIR")
    s.add_argument("--otlp-endpoint", default="", help="OTLP/HTTP collector base URL for metric pushes")
    s.add_argument("--warmup-prompt", default=None, help="generate from this prompt once before listening")
    s.add_argument("--ngram-speculative", action="store_true", help="same as --speculative ngram")
    s.add_argument("--self-speculative", action="store_true", help="same as --speculative mtp")
    s.add_argument("--master-addr", default=None, help="rendezvous address when ranks are started by hand")
    s.add_argument("--master-port", type=int, default=None)
    s.add_argument("--rank", type=int, default=None)
    s.add_argument("--world-size", type=int, default=None)
    s.add_argument("--nllb-src-lang", default=None, help="NLLB / M2M-100 checkpoints: source language code, e.g. eng_Latn")
    s.add_argument("--nllb-tgt-lang", default=None, help="NLLB / M2M-100 checkpoints: target language code, e.g. fra_Latn")
    s.add_argument("--swap-space-gb", type=float, default=0.0,
                   help="> 0: preempted sequences are swapped to host memory (then swap files) instead of recomputed")

    b = sub.add_parser("benchmark", help="concurrency ladder over the engine API")
    _add_engine_args(b)
    b.add_argument("--concurrency", default="1,2,4,8,16,32,64,128")
    b.add_argument("--isl", type=int, default=128)
    b.add_argument("--osl", type=int, default=1024)
    b.add_argument("--json", action="store_true")
    b.add_argument("--url", default=None, help="sweep a running server over HTTP (streaming chat requests) instead of an in-process engine")
    b.add_argument("--api-key", default=None)
    b.add_argument("--served-model-name", default="default")

    gt = sub.add_parser("gates", help="correctness gates over an in-process engine: order equality, conversation replay, "
                                      "history independence, state poisoning, cross-request contamination, decode floor")
    _add_engine_args(gt)
    gt.add_argument("--only", default=None, help="comma list of: order, replay, kat, poison, contamination, floor")
    gt.add_argument("--rounds", type=int, default=12, help="replays of the conversation / of the probe request")
    gt.add_argument("--decode-floor", type=float, default=0.0, help="tokens/s the single-user decode rate must reach (0: recorded only)")

    for name, helptext in (("tui", "live dashboard of a running server"), ("chat", "terminal chat with a running server")):
        t = sub.add_parser(name, help=helptext)
        t.add_argument("--url", default="http://127.0.0.1:8888")
        t.add_argument("--api-key", default=None)
        t.add_argument("--period", type=float, default=1.0)
        t.add_argument("--model", default="default")
        t.add_argument("--system", default=None)
    dl = sub.add_parser("download", help="fetch a model repository into the cache")
    dl.add_argument("repo")
    dl.add_argument("--cache-dir", default=None)
    dl.add_argument("--endpoint", default=None, help="Hub-compatible endpoint (default: HF_ENDPOINT or huggingface.co)")
    dl.add_argument("--revision", default="main")
    pf = sub.add_parser("preflight", help="check a checkpoint directory against its configuration without loading it")
    pf.add_argument("model")
    pf.add_argument("--cache-dir", default=None)
    ml = sub.add_parser("models", help="list the models in the cache")
    ml.add_argument("--cache-dir", default=None)
    ml.add_argument("--json", action="store_true")

    d = sub.add_parser("doctor", help="report device, driver and library state")
    d.add_argument("--json", action="store_true")

    o = sub.add_parser("dump-serve-options", help="print every serve option and its default")

    pl = sub.add_parser("plan", help="roofline estimate of a decode step (bytes, FLOPs, time per op)")
    pl.add_argument("--model", default="dense-27b-nvfp4")
    pl.add_argument("--batch", type=int, default=128)
    pl.add_argument("--ctx", type=int, default=640)
    pl.add_argument("--tp", type=int, default=1)
    pl.add_argument("--json", action="store_true")
    pl.add_argument("--circuit", default=None, help="also summarise this circuit file (name under planner/circuits or a path): ops, launches after fusion, planned activation bytes")

    sp = sub.add_parser("storage-probe", help="what a scratch directory can do for the KV / expert tiers (O_DIRECT, GDS, read and write rates)")
    sp.add_argument("--dir", default=None)
    sp.add_argument("--blocks", type=int, default=64)
    sp.add_argument("--block-kib", type=int, default=256)
    return ap


def dump_serve_options() -> dict:
    ap = build_parser()
    serve = ap._subparsers._group_actions[0].choices["serve"]      # noqa: SLF001 (argparse has no public API)
    out = {}
    for a in serve._actions:
        if a.dest in ("help",):
            continue
        out[a.option_strings[-1] if a.option_strings else a.dest] = {
            "default": a.default, "help": a.help or "", "choices": list(a.choices) if a.choices else None}
    from ..utils.levers import LEVERS
    out["__env_levers__"] = dict(LEVERS)
    return out


def doctor() -> dict:
    import torch
    rep = {"python": sys.version.split()[0], "torch": torch.__version__, "cuda_runtime": torch.version.cuda,
           "cuda_available": torch.cuda.is_available(), "devices": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            free, total = torch.cuda.mem_get_info(i)
            rep["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                   "total_gb": round(total / 2**30, 1), "free_gb": round(free / 2**30, 1)})
        rep["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
        rep["p2p"] = (torch.cuda.device_count() > 1 and torch.cuda.can_device_access_peer(0, 1))
    from ..ops import _native
    lib = os.path.join(os.path.dirname(_native.__file__), "libmetrale_b200.so")
    rep["native_library"] = {"path": lib, "present": os.path.exists(lib)}
    from ..utils.levers import LEVERS, undeclared
    rep["levers"] = {k: os.environ[k] for k in LEVERS if k in os.environ}
    rep["undeclared_levers"] = undeclared()
    rep["ok"] = not rep["undeclared_levers"] and (
        (not torch.cuda.is_available()) or (rep["native_library"]["present"] and all(d["sm"] == "10.0" for d in rep["devices"])))
    return rep


def run_benchmark(ns) -> List[dict]:
    if getattr(ns, "url", None):
        from ..bench.http_sweep import run_sweep
        rows = run_sweep(ns.url, [int(c) for c in ns.concurrency.split(",")], ns.isl, ns.osl,
                         model=ns.served_model_name, api_key=ns.api_key)
        for r in rows:          # same columns as the in-process ladder
            r.setdefault("ms_per_step", float("nan"))
            r["ttft_p50_ms"] = r["ttft_p50_ms"] if r["ttft_p50_ms"] is not None else float("nan")
            r["ttft_p99_ms"] = r["ttft_p99_ms"] if r["ttft_p99_ms"] is not None else float("nan")
        return rows
    from ..bench.ladder import run_ladder
    return run_ladder(_engine_args(ns), [int(c) for c in ns.concurrency.split(",")], ns.isl, ns.osl)


def run_gates(ns) -> list:
    """The correctness gates of ``bench/`` against one in-process engine built from the serve options."""
    import torch

    from ..bench import determinism, isolation, replay_gates
    from ..engine.llm_engine import LLMEngine
    from ..sampling.params import SamplingParams
    eargs = _engine_args(ns)
    eargs.enable_prefix_caching = True
    want = set((ns.only or "order,replay,kat,poison,contamination,floor").split(","))
    make = lambda: LLMEngine(eargs)
    eng = make()
    vocab = eng.cfg.vocab_size
    g = torch.Generator().manual_seed(5)
    draw = lambda n, length: [torch.randint(1, vocab, (length + 3 * i,), generator=g).tolist() for i in range(n)]
    dev = str(eargs.device)
    recs = []
    if "order" in want:
        recs.append(replay_gates.order_equality(eng, draw(8, 40), orders=3, max_tokens=24, device=dev))
    if "replay" in want:
        noise_prompts = draw(4, 64)
        first = max(48, eng.scheduler.snapshot_interval + eargs.block_size + 8) if eng.runner.pool is not None else 48
        script = [draw(1, first)[0]] + draw(3, 24)
        recs.append(replay_gates.conversation_replay(
            eng, script, rounds=ns.rounds, max_tokens=16, device=dev,
            noise=lambda r: eng.generate([noise_prompts[r % 4]], SamplingParams(max_tokens=8, temperature=0.0))))
    if "floor" in want:
        rec = replay_gates.decode_floor(eng, draw(1, 64)[0], ns.decode_floor, runs=5, max_tokens=64, device=dev)
        recs.append(rec)
    if "contamination" in want:
        rep = isolation.contamination(eng, n_requests=min(8, eargs.max_num_seqs), rounds=2)
        from ..bench.gate import GateRecord, kernel_closure_hash
        recs.append(GateRecord("contamination", "requests whose reply holds another request's secret", float(len(rep["leaks"])), "leaks",
                               higher_is_better=False, config={"pass": rep["ok"], "requests": rep["requests"], "leaks": rep["leaks"][:8]},
                               closure=kernel_closure_hash(), device=dev))
    eng.close()
    if "kat" in want:
        recs.append(determinism.kat_equality(make, device=dev))
    if "poison" in want and eng.runner.pool is not None:
        recs.append(determinism.state_poisoning(make, replays=ns.rounds, device=dev))
    return recs


def _init_ranks(eargs):
    """Process group + tensor-parallel context + control plane for a multi-rank launch."""
    import torch
    import torch.distributed as dist
    from ..parallel.control import ControlPlane
    rank, world, local = (int(os.environ.get(k, "0")) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if str(eargs.device).startswith("cuda"):
        from ..parallel.tp import NcclTpContext
        torch.cuda.set_device(local)
        eargs.device = f"cuda:{local}"
        dist.init_process_group("nccl", device_id=torch.device(eargs.device))
        tp = NcclTpContext(rank, world, eargs.device, fused=eargs.fused_collectives)
    else:
        from ..parallel.tp import GlooTpContext
        dist.init_process_group("gloo")
        tp = GlooTpContext(rank, world)
    if eargs.ep_size > 1:
        tp.ep_rank = rank
    else:
        eargs.tp_size = world
    return tp, ControlPlane.create()


def apply_aliases(ns) -> None:
    """Folds the alias flags into the fields the engine and the server read, and checks the
    authentication options."""
    if ns.bind:
        host, _, port = ns.bind.rpartition(":")
        ns.host, ns.port = (host or ns.host), int(port)
    if ns.model_name and not ns.served_model_name:
        ns.served_model_name = ns.model_name
    if ns.max_seq_len:
        ns.max_model_len = ns.max_seq_len
    if ns.max_batch_size:
        ns.max_num_seqs = ns.max_batch_size
    if ns.request_timeout:
        ns.request_timeout_s = ns.request_timeout
    if ns.ngram_speculative:
        ns.speculative = "ngram"
    if ns.self_speculative:
        ns.speculative = "mtp"
    tokens = list(ns.api_key) + list(ns.auth_token)
    if ns.auth_tokens_file:
        with open(ns.auth_tokens_file) as f:
            tokens += [ln.strip() for ln in f if ln.strip() and not ln.startswith("#")]
    ns.api_key = tokens
    if ns.require_auth and not tokens:
        raise SystemExit("--require-auth: no token given (--auth-token / --auth-tokens-file / --api-key)")
    for flag, env in (("master_addr", "MASTER_ADDR"), ("master_port", "MASTER_PORT"), ("rank", "RANK"),
                      ("world_size", "WORLD_SIZE")):
        v = getattr(ns, flag)
        if v is not None:
            os.environ[env] = str(v)
    if ns.rank is not None:
        os.environ.setdefault("LOCAL_RANK", str(ns.rank))


def serve(ns) -> None:
    import uvicorn
    from ..engine.llm_engine import LLMEngine
    from .app import ServerConfig, create_app
    from .tokenizer import load_tokenizer
    apply_aliases(ns)
    if isinstance(ns.model, str):
        from ..config.model_config import PRESETS
        from .model_library import resolve_model_dir
        ns.model = resolve_model_dir(ns.model, ns.cache_dir, presets=tuple(PRESETS))
    if isinstance(ns.model, str) and os.path.isdir(ns.model):
        from .translate import is_translation_checkpoint
        if is_translation_checkpoint(ns.model):
            return _serve_translation(ns)
    eargs = _engine_args(ns)
    if ns.swap_space_gb > 0:
        eargs.preempt_mode, eargs.swap_space_bytes = "swap", int(ns.swap_space_gb * (1 << 30))
    tp, control = None, None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # launched by torch.distributed.run: every rank builds its shard; rank 0 owns HTTP and
        # publishes each tick's operations, the others replay them (parallel/control.py)
        tp, control = _init_ranks(eargs)
    engine = LLMEngine(eargs, tp=tp)
    if control is not None and control.rank != 0:
        from ..parallel.control import follower_loop
        print(f"[rank {control.rank}] follower ended: {follower_loop(engine, control)}", flush=True)
        return
    for spec in ns.lora_adapter:
        name, _, path = spec.partition("=")
        engine.load_adapter(name, path, ns.max_loras, ns.max_lora_rank)
    tok_dir = ns.tokenizer or (eargs.model if isinstance(eargs.model, str) and os.path.isdir(eargs.model) else None)
    tokenizer = load_tokenizer(tok_dir, engine.cfg.vocab_size)
    if ns.warmup_prompt:
        from ..sampling.params import SamplingParams
        engine.generate([tokenizer.encode(ns.warmup_prompt)], SamplingParams(max_tokens=8, temperature=0.0))
    cfg = ServerConfig(model_name=ns.served_model_name or str(ns.model), auth_tokens=ns.api_key,
                       default_top_n_sigma=ns.default_top_n_sigma, default_min_p=ns.default_min_p,
                       max_thinking_budget=ns.max_thinking_budget, content_loop_watchdog=ns.content_loop_watchdog,
                       dump_dir=ns.dump, otlp_endpoint=ns.otlp_endpoint, adaptive_sampling=ns.adaptive_sampling,
                       rate_per_s=ns.rate_limit, tool_call_parser=ns.tool_call_parser, tool_grammar=getattr(ns, "tool_grammar", False),
                       reasoning_format=ns.reasoning_format, default_max_tokens=ns.default_max_tokens,
                       tool_max_tokens=ns.tool_max_tokens,
                       telemetry=ns.telemetry, disable_thinking=ns.disable_thinking)
    app = create_app(engine, tokenizer, cfg, control=control)
    uvicorn.run(app, host=ns.host, port=ns.port, log_level="info", timeout_graceful_shutdown=20)


def _apply_recipe(argv: List[str]) -> List[str]:
    """`serve --recipe file.yaml ...`: recipe options first, then the command line (which wins)."""
    if not argv or argv[0] != "serve" or "--recipe" not in argv:
        return argv
    import os as _os
    from ..config.recipes import load_recipe, recipe_to_argv
    path = argv[argv.index("--recipe") + 1]
    recipe = load_recipe(path)
    serve = build_parser()._subparsers._group_actions[0].choices["serve"]          # noqa: SLF001
    options = [o for a in serve._actions for o in a.option_strings if o.startswith("--")]
    for k, v in (recipe.get("env") or {}).items():
        _os.environ.setdefault(k, str(v))
    return ["serve"] + recipe_to_argv(recipe, options) + argv[1:]


def main(argv: Optional[List[str]] = None) -> int:
    argv = _apply_recipe(list(sys.argv[1:] if argv is None else argv))
    ns = build_parser().parse_args(argv)
    if ns.cmd == "serve":
        serve(ns)
    elif ns.cmd == "benchmark":
        rows = run_benchmark(ns)
        if ns.json:
            print(json.dumps(rows))
        else:
            print(f"{'C':>4} {'tok/s':>10} {'p50 TTFT ms':>12} {'p99 TTFT ms':>12} {'ms/step':>9}")
            for r in rows:
                print(f"{r['concurrency']:>4} {r['tok_s']:>10.1f} {r['ttft_p50_ms']:>12.1f} {r['ttft_p99_ms']:>12.1f} {r['ms_per_step']:>9.2f}")
    elif ns.cmd == "gates":
        recs = run_gates(ns)
        for r in recs:
            ok = r.config.get("pass", r.value == 1.0)
            print(f"{'PASS' if ok else 'FAIL'}  {r.name:<22} {r.metric}: {r.value:g} {r.unit}  {r.config.get('why') or r.config.get('mismatch') or ''}")
        if not all(r.config.get("pass", r.value == 1.0) for r in recs):
            raise SystemExit(1)
    elif ns.cmd in ("tui", "chat"):
        from .tui import ChatSession, Dashboard, HttpTransport
        tr = HttpTransport(ns.url, ns.api_key)
        if ns.cmd == "tui":
            try:
                Dashboard(tr).run(ns.period)
            except KeyboardInterrupt:
                pass
        else:
            ChatSession(tr, model=ns.model, system=ns.system).repl()
    elif ns.cmd == "download":
        from .model_library import DownloadError, download
        last = [0]

        def show(name, done, total):
            pct = int(100 * done / total) if total else 0
            if pct != last[0]:
                last[0] = pct
                print(f"\r{pct:3d}%  {done / 2**20:10.1f} / {total / 2**20:.1f} MiB  {name[:40]:40s}", end="", flush=True)
        try:
            path = download(ns.repo, ns.cache_dir, ns.endpoint, ns.revision, progress=show)
        except DownloadError as e:
            print(f"\ndownload failed: {e}", file=sys.stderr)
            return 1
        print(f"\n{path}")
    elif ns.cmd == "preflight":
        from ..weights.checkpoint import open_checkpoint
        from ..weights.preflight import preflight
        from .model_library import resolve_model_dir
        cfg, src = open_checkpoint(resolve_model_dir(ns.model, ns.cache_dir))
        rep = preflight(cfg, src)
        print(rep.summary(limit=50))
        return 0 if rep.ok else 1
    elif ns.cmd == "models":
        from .model_library import list_models
        rows = list_models(ns.cache_dir)
        if ns.json:
            print(json.dumps(rows))
        else:
            for r in rows:
                print(f"{r['repo']:50s} {(r['revision'] or '-')[:12]:12s} {r['bytes'] / 2**30:8.2f} GiB  "
                      f"{'ok' if r['complete'] else 'incomplete'}")
    elif ns.cmd == "doctor":
        rep = doctor()
        print(json.dumps(rep, indent=None if ns.json else 2))
        return 0 if rep["ok"] else 1
    elif ns.cmd == "plan":
        from ..config.model_config import preset
        from ..planner import estimate
        if os.path.isdir(ns.model):
            from ..weights.checkpoint import open_checkpoint
            cfg = open_checkpoint(ns.model)[0]
        else:
            cfg = preset(ns.model)
        e = estimate(cfg, ns.batch, ns.ctx, ns.tp)
        if ns.json:
            print(json.dumps(e))
        else:
            print(f"{e['model']}  batch {e['batch']}  ctx {e['ctx']}  tp {e['tp']}  peaks: {e['peaks']}")
            print(f"{'op':28s} {'count':>5} {'us each':>9} {'us total':>10} {'MB each':>10}  bound")
            for r in e["ops"]:
                print(f"{r['op']:28s} {r['count']:>5} {r['us_each']:>9.2f} {r['us_total']:>10.1f} {r['mbytes_each']:>10.3f}  {r['bound']}")
            print(f"step: {e['step_ms_roofline_per_op']} ms per-op roofline, {e['step_ms_bytes_only']} ms bytes only "
                  f"({e['gbytes_per_step']} GB, {e['tflop_per_step']} TFLOP, {e['launches']} launches); "
                  f"upper bound {e['tok_s_upper_bound']} tok/s")
        if ns.circuit:
            from ..planner import circuit as _c
            print(json.dumps(_c.summary(_c.load(ns.circuit), cfg, ns.batch)))
    elif ns.cmd == "storage-probe":
        from ..storage.probe import run_probe
        print(json.dumps(run_probe(ns.dir, blocks=ns.blocks, block_kib=ns.block_kib), indent=2))
    elif ns.cmd == "dump-serve-options":
        print(json.dumps(dump_serve_options(), indent=2, default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
