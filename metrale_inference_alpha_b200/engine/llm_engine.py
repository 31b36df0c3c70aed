"""The public engine API: build a model from a preset / checkpoint, add requests, step.

``LLMEngine.step()`` is one scheduler tick: plan -> execute on the device -> (draft) -> apply.
``generate()`` is the offline convenience loop over ``step()``. The HTTP server drives the
same object from its scheduler thread. Role of the reference's boot phases 1-9
(``crates/server/src/main_modules/serve_load``) and of ``metrale_scheduler::run``.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence as Seq, Union

import torch

from .. import ops
from ..cache import RadixTree, make_radix  # noqa: F401
from ..config.model_config import ModelConfig, preset as cfg_preset
from ..models.decoder import TpContext
from ..sampling.params import SamplingParams
from ..scheduler.core import SchedulerCore
from ..scheduler.policy import SchedulerConfig
from ..scheduler.types import FatalDeviceError, Request, RequestOutput, StepPlan
from ..speculative import KLadder, MtpGate, NgramProposer, SpecStats
from ..utils.fault import FaultLatch
from ..weights.loader import load_weights
from ..weights.source import SafetensorsSource, TensorSource
from .runner import ModelRunner, plan_kv_blocks


@dataclass
class EngineArgs:
    model: Union[str, ModelConfig] = "tiny-dense"     # preset name, checkpoint dir, or a config
    device: str = "cpu"
    seed: int = 0
    max_num_seqs: int = 128
    max_model_len: int = 2048
    max_prefill_tokens: int = 8192
    block_size: int = 16
    gpu_memory_utilization: float = 0.90
    num_kv_blocks: Optional[int] = None
    enable_prefix_caching: bool = True
    scheduler: str = "fifo"
    tbt_deadline_ms: float = 100.0
    use_cuda_graphs: bool = True
    speculative: str = "none"                          # none | mtp | ngram | dflash
    num_drafts: int = 3
    dflash_layers: int = 2                             # block drafter depth (random weights unless a drafter checkpoint is attached)
    dflash_gamma: int = 0                              # block drafter: drafts per proposal; 0 = the width policy (4 at C >= 2; 5 / 8 at C = 1)
    mtp_gate: bool = True
    kv_poison: bool = False
    tp_size: int = 1
    ep_size: int = 1
    request_timeout_s: float = 300.0
    eos_token_id: Optional[int] = None
    fused_collectives: bool = False                    # tensor parallel: GEMM + all-reduce in one kernel over NVLink peer memory
                                                       # instead of NCCL after the GEMM (measured slower so far: off by default)
    ep_dispatch: str = "allreduce"                     # expert parallelism: allreduce (masked-local experts) | a2a (token dispatch over peer memory)
    activation_precision: str = "native"               # native (W4A4 / W8A8) | a16 (bf16 activations, weight-only quantisation)
    static_act_scales: bool = True                     # NVFP4: calibrate down-projection input scales at start-up
    preempt_mode: str = "recompute"                    # recompute | swap (KV + state to host memory / swap files)
    swap_space_bytes: int = 8 << 30
    swap_dir: Optional[str] = None
    decode_rollback_ring: int = 0                      # recurrent models: state snapshots per decoding sequence for rollback_request (0 = off)
    decode_rollback_interval: int = 16                 # a ring snapshot every this many generated tokens
    state_snapshots: int = 0                           # device-resident state snapshots (0 = 16 + ring slots x max_num_seqs)
    state_tier_host_bytes: int = 0                     # > 0: resident snapshots overflow into this much host memory ...
    state_tier_dir: Optional[str] = None               # ... and from there (or directly) into files in this directory
    kv_tier_blocks: int = 0                            # > 0: KV blocks the prefix cache evicts are kept in a second tier of this many blocks ...
    kv_tier_dir: Optional[str] = None                  # ... in files under this directory (default: host memory)
    kv_tier_host_blocks: int = 0                       # with kv_tier_dir: a pinned write-back host cache of this many blocks in front of the files
    kv_tier_codec: str = "raw"                         # raw | nvfp4 | turbo4 | turbo3 | turbo2: lossy record formats of the tier (76 / 68 / 52 / 36 bytes per 128 channels against 256 for bf16)
    expert_arena_slots: int = 0                        # MoE: > 0 pages the routed experts from an expert store into a device arena of this many experts
    expert_store_dir: Optional[str] = None             # ... the store's directory (written from the loaded weights when it has no manifest yet)
    prediction_drafts: int = 8                         # tokens verified per step for requests with a predicted output
    kv_cache_dtype: str = "auto"                       # auto (the model config's) | bf16 | fp8
    kv_high_precision_layers: str = ""                 # e.g. "0,1,63" or "first:2,last:2": these layers keep bf16 KV under fp8
    oom_guard_mb: int = 4096                           # device memory left unclaimed when sizing the KV pool
    fp8_kv_calibration_tokens: int = 0                 # fp8 KV without checkpoint scales: calibrate them online over this many tokens (0 = scale 1.0)
    fp8_kv_headroom: float = 1.0
    pipeline_decode: bool = True                       # launch decode step t + 1 from the device-fed tokens while step t is read back


def parse_layer_list(spec: str, num_layers: int) -> tuple:
    """"0,5,63", "first:2", "last:3" and combinations -> sorted layer indices."""
    out = set()
    for part in (p.strip() for p in spec.split(",") if p.strip()):
        if part.startswith("first:"):
            out.update(range(min(num_layers, int(part[6:]))))
        elif part.startswith("last:"):
            out.update(range(max(0, num_layers - int(part[5:])), num_layers))
        else:
            i = int(part)
            if not 0 <= i < num_layers:
                raise ValueError(f"layer {i} out of range (0..{num_layers - 1})")
            out.add(i)
    return tuple(sorted(out))


class LLMEngine:
    def __init__(self, args: EngineArgs, tp: Optional[TpContext] = None, source: Optional[TensorSource] = None):
        self.args = args
        self.device = torch.device(args.device)
        self.tp = tp or TpContext()
        cfg = args.model
        if isinstance(cfg, str):
            import os
            if os.path.isdir(cfg) or (os.path.isfile(cfg) and cfg.endswith(".gguf")):
                from ..weights.checkpoint import open_checkpoint
                cfg, source = open_checkpoint(cfg, device=args.device)
                if type(source).__name__ != "GgufSource":        # GGUF names are mapped (and checked) by its own source
                    from ..weights.preflight import preflight
                    rep = preflight(cfg, source, check_shapes=False)      # names only: cheap, and fails before any load
                    if not rep.ok:
                        raise ValueError(rep.summary())
            else:
                cfg = cfg_preset(cfg)
        if args.kv_cache_dtype not in ("auto", cfg.kv_dtype):
            import dataclasses
            if args.kv_cache_dtype not in ("bf16", "fp8"):
                raise ValueError(f"kv_cache_dtype must be auto | bf16 | fp8, not {args.kv_cache_dtype!r}")
            cfg = dataclasses.replace(cfg, kv_dtype=args.kv_cache_dtype)
        if args.kv_high_precision_layers:
            import dataclasses
            cfg = dataclasses.replace(cfg, kv_high_precision_layers=parse_layer_list(args.kv_high_precision_layers,
                                                                                       cfg.num_layers))
        self.cfg: ModelConfig = cfg
        self.fault = FaultLatch()
        t0 = time.time()
        from .. import ops as _ops
        _ops.set_activation_precision(args.activation_precision)
        self.weights = load_weights(cfg, source, device=args.device, tp_rank=self.tp.rank,
                                    tp_size=self.tp.size if args.ep_size == 1 or args.tp_size > 1 else 1,
                                    ep_rank=getattr(self.tp, "ep_rank", 0), ep_size=args.ep_size, seed=args.seed)
        self.load_seconds = time.time() - t0
        import os as _os
        self._redzone_every = int(_os.environ.get("METRALE_REDZONE_EVERY", "0") or 0)
        if (cfg.num_experts > 0 and cfg.weight_format == "nvfp4" and torch.device(args.device).type == "cuda"
                and args.use_cuda_graphs
                and any(getattr(getattr(L, "ffn", None), "experts", None) and L.ffn.grouped is None for L in self.weights.layers)):
            # NVFP4 experts whose row count is not a multiple of the 128-row scale-factor tile run one GEMM per
            # active expert, chosen on the host from the step's routing: such a step cannot be replayed from a graph
            args.use_cuda_graphs = False
        self.paged_experts = None
        if args.expert_arena_slots > 0:
            if not args.expert_store_dir:
                raise ValueError("expert_arena_slots needs expert_store_dir")
            from ..storage.expert_store import enable_expert_paging
            self.paged_experts = enable_expert_paging(self.weights, args.expert_store_dir, args.expert_arena_slots,
                                                      args.device)
            # residency is decided on the host from each step's routing: no graph replay over it
            args.use_cuda_graphs = False
        self.sched_cfg = SchedulerConfig(
            max_num_seqs=args.max_num_seqs, max_prefill_tokens=args.max_prefill_tokens,
            max_model_len=min(args.max_model_len, cfg.max_position), block_size=args.block_size,
            policy=args.scheduler, tbt_deadline_ms=args.tbt_deadline_ms,
            enable_prefix_caching=args.enable_prefix_caching, request_timeout_s=args.request_timeout_s,
            decode_ring_slots=args.decode_rollback_ring, decode_ring_interval=args.decode_rollback_interval)
        blocks = args.num_kv_blocks or plan_kv_blocks(cfg, self.weights, args.device, args.block_size,
                                                      args.gpu_memory_utilization,
                                                      reserve_bytes=(2 << 30) + (args.oom_guard_mb << 20))
        # never more than every sequence at full length needs (plus headroom for the prefix cache)
        cap = (self.sched_cfg.max_model_len // args.block_size + 1) * args.max_num_seqs * 2 + 64
        blocks = min(blocks, cap)
        # the batch cap is a deployment constant, so the partitioning (and with it the numerics of
        # a sequence) still never depends on which other requests happen to be running
        ops.configure(attn_part_tokens=1024 if args.max_num_seqs >= 64 else 512)
        self.runner = ModelRunner(cfg, self.weights, args.device, blocks, self.sched_cfg, self.tp,
                                  use_graphs=args.use_cuda_graphs, kv_poison=args.kv_poison,
                                  fp8_kv_calibration_tokens=args.fp8_kv_calibration_tokens,
                                  fp8_kv_headroom=args.fp8_kv_headroom,
                                  num_snapshots=args.state_snapshots or 16 + args.decode_rollback_ring * args.max_num_seqs)
        if self.runner.pool is not None and (args.state_tier_host_bytes > 0 or args.state_tier_dir):
            self.runner.pool.configure_tiers(args.state_tier_host_bytes, args.state_tier_dir)
        if args.ep_dispatch == "a2a" and args.ep_size > 1 and self.tp.size > 1 and self.device.type == "cuda" \
                and cfg.num_experts > 0:
            from ..parallel.ep import EpAllToAll
            per_rank = (max(self.sched_cfg.max_prefill_tokens, args.max_num_seqs * 8) + self.tp.size - 1) // self.tp.size
            self.tp.ep = EpAllToAll(self.tp.rank, self.tp.size, self.device, cfg.hidden_size, per_rank,
                                    cfg.experts_per_token)
        self.calibrated_layers = 0
        if (args.static_act_scales and cfg.weight_format == "nvfp4" and self.device.type == "cuda"
                and args.activation_precision == "native"):
            self.calibrated_layers = self.runner.calibrate_static_scales()
        needs_snap = self.runner.pool is not None
        self.prefix = None
        if args.enable_prefix_caching:
            self.prefix = make_radix(self.runner.kv.allocator, args.block_size, needs_snapshot=needs_snap,
                                    on_snapshot_evict=(self.runner.pool.release_snapshot if needs_snap else None))
            if needs_snap and hasattr(self.prefix, "snapshot_ok"):
                self.prefix.snapshot_ok = self.runner.pool.available
            if args.kv_tier_blocks > 0:
                if needs_snap:
                    raise ValueError("kv_tier_blocks: models with recurrent state keep their prefix hits through state "
                                     "snapshots (state_tier_host_bytes / state_tier_dir), not through KV tiering")
                from ..cache.kv_tier import KvTierStore, TieredRadixTree
                self.kv_tier = KvTierStore(self.runner.kv, args.kv_tier_blocks, args.kv_tier_dir, args.kv_tier_host_blocks,
                                           codec=args.kv_tier_codec)
                self.prefix = TieredRadixTree(self.runner.kv.allocator, args.block_size, self.kv_tier)
        self.spill = None
        if args.preempt_mode == "swap":
            from ..cache.kv_spill import KvSpillManager
            self.sched_cfg.preempt_mode = "swap"
            self.spill = KvSpillManager(self.runner.kv, self.runner.pool, args.swap_space_bytes, args.swap_dir)
        self.scheduler = SchedulerCore(self.sched_cfg, self.runner.kv.allocator, self.prefix, self.runner.pool,
                                       spill=self.spill)
        self._ids = itertools.count(1)
        self.spec_mode = args.speculative
        if self.spec_mode == "mtp" and self.weights.mtp is None:
            self.spec_mode = "none"
        self.ladder = KLadder(max_k=args.num_drafts)
        self.dflash_rung = None
        if self.spec_mode == "dflash":
            from ..speculative.dflash import DflashConfig
            from ..speculative.ladder import DflashRung
            self.dflash_rung = DflashRung()
            self.runner.enable_dflash(DflashConfig(num_layers=args.dflash_layers,
                                                   gamma=max(args.dflash_gamma, self.dflash_rung.wide)))
        self.gate = MtpGate(enabled=(self.spec_mode != "none" and args.mtp_gate))
        self.ngram = NgramProposer()
        self.spec_stats = SpecStats()
        self.step_count = 0
        self._inflight = None            # (plan, handle) of a decode step launched ahead and not yet applied
        self.pipeline = bool(args.pipeline_decode and self.device.type == "cuda" and args.use_cuda_graphs)
        if args.decode_rollback_ring > 0 and self.runner.pool is not None:
            self.pipeline = False          # a ring snapshot must see the state of exactly the applied step
        self.tokenizer = None
        self.stop_strings_active = False

    # ------------------------------------------------------------------ LoRA adapters
    def load_adapter(self, name: str, source, max_adapters: int = 8, max_rank: int = 16) -> int:
        """Make a LoRA adapter available to ``add_request(..., adapter=name)``. ``source`` is a PEFT
        checkpoint directory or a ``lora.LoraAdapter``. Returns the device slot."""
        from ..lora import LoraAdapter, LoraManager
        if self.tp.size > 1:
            raise NotImplementedError("LoRA adapters are served on single-rank engines")
        dec, c = self.runner.decoder, self.cfg
        if dec.lora is None:
            D = c.head_dim
            dims = {"q": (c.hidden_size, c.num_heads * D), "k": (c.hidden_size, c.num_kv_heads * D),
                    "v": (c.hidden_size, c.num_kv_heads * D), "o": (c.num_heads * D, c.hidden_size),
                    "down": (c.intermediate_size, c.hidden_size)}
            dec.lora = LoraManager(c.num_layers, dims, max_adapters, max_rank, device=self.device,
                                   max_rows=max(self.sched_cfg.max_prefill_tokens, self.sched_cfg.max_num_seqs * 8))
        ad = source if isinstance(source, LoraAdapter) else LoraAdapter.from_dir(name, source)
        ad.name = name
        return dec.lora.load(ad)

    def unload_adapter(self, name: str) -> None:
        if self.runner.decoder.lora is not None:
            self.runner.decoder.lora.unload(name)

    # ------------------------------------------------------------------ requests
    # ------------------------------------------------------------------ vision input
    vision = None

    def attach_vision(self, encoder=None, preprocessor=None, seed: int = 0) -> None:
        """Enable ``add_request(..., images=[...])``. Without an encoder the tower of the model
        configuration is built with random weights (synthetic checkpoints); ``open_vision`` loads it
        from a checkpoint's ``visual.`` tensors."""
        from ..vision import ImagePreprocessor, VisionConfig, VisionEncoder
        c = self.cfg
        if c.image_token_id < 0:
            raise ValueError("the model configuration names no image placeholder token")
        if self.args.speculative != "none":
            raise NotImplementedError("image inputs and speculative decoding are not combined")
        if encoder is None:
            vc = VisionConfig.from_hf(dict(c.vision or {}, hidden_size=c.hidden_size))
            encoder = VisionEncoder(vc, VisionEncoder.random_tensors(vc, seed), device=self.device)
        if encoder.cfg.hidden_size != c.hidden_size:
            raise ValueError("the vision tower's output width differs from the model's hidden size")
        vc = encoder.cfg
        self.vision = (encoder, preprocessor or ImagePreprocessor(vc.patch_size, vc.spatial_merge_size, vc.temporal_patch_size))

    def open_vision(self, source) -> None:
        """Load the vision tower from a checkpoint source (tensor names ``visual.*`` or ``model.visual.*``)."""
        from ..vision import VisionConfig, VisionEncoder
        vc = VisionConfig.from_hf(dict(self.cfg.vision or {}, hidden_size=self.cfg.hidden_size))
        names = [n for n in source.names() if n.startswith(("visual.", "model.visual."))]
        if not names:
            raise ValueError("the checkpoint holds no visual.* tensors")
        tensors = {n.split("visual.", 1)[1]: source.get(n) for n in names}
        self.attach_vision(VisionEncoder(vc, tensors, device=self.device))

    def add_request(self, prompt_ids: Seq[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, adapter: Optional[str] = None, images=None) -> str:
        if self.fault.is_set():
            raise FatalDeviceError(self.fault.reason())
        rid = request_id or f"req-{next(self._ids)}"
        params = params or SamplingParams()
        mm = None
        if images:
            if self.vision is None:
                raise ValueError("this engine serves no image inputs (attach_vision was not called)")
            from .multimodal import build_inputs
            enc, pre = self.vision
            prompt_ids, mm = build_inputs(prompt_ids, images, encoder=enc, preprocessor=pre,
                                          image_token_id=self.cfg.image_token_id, merge=enc.cfg.spatial_merge_size,
                                          device=self.device)
        adapter = adapter or params.adapter
        if adapter and (self.runner.decoder.lora is None or adapter not in self.runner.decoder.lora.slots):
            raise ValueError(f"unknown LoRA adapter {adapter!r}")
        req = Request(rid, list(prompt_ids), params, adapter=adapter,
                      eos_token_id=self.args.eos_token_id, mm=mm)
        self.scheduler.add_request(req)
        return rid

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id)

    def has_work(self) -> bool:
        return self._inflight is not None or self.scheduler.has_work()

    def flush(self) -> List[RequestOutput]:
        """Complete (read back and apply) a decode step that was launched ahead, if any."""
        if self._inflight is None:
            return []
        plan, handle = self._inflight
        self._inflight = None
        return self._finish_pipelined(plan, handle, launch_next=False)

    def _finish_pipelined(self, plan: StepPlan, handle, launch_next: bool = True) -> List[RequestOutput]:
        """Step t is on the device. Launch step t + 1 from the device-fed tokens when the scheduler
        can plan it blind, then wait for step t's ids and apply them."""
        nxt = None
        if launch_next:
            ahead = self.scheduler.plan_ahead(plan)
            if ahead is not None:
                h2 = self.runner.launch_decode(ahead, ahead=True)
                if h2 is not None:
                    nxt = (ahead, h2)
        try:
            result = self.runner.finish_decode(handle)
        except RuntimeError as e:
            if isinstance(e, FatalDeviceError) or "CUDA" in str(e) or "device status" in str(e):
                self.fault.set(str(e))
                raise FatalDeviceError(str(e)) from e
            raise
        outs = self.scheduler.apply(plan, result, None)
        self._inflight = nxt
        self.step_count += 1
        return outs

    # ------------------------------------------------------------------ one tick
    def step(self) -> List[RequestOutput]:
        if self.fault.is_set():
            raise FatalDeviceError(self.fault.reason())
        sch = self.scheduler
        if self._inflight is not None:
            plan, handle = self._inflight
            self._inflight = None
            return self._finish_pipelined(plan, handle)
        plan = sch.plan()
        if plan is None:
            return sch.drain_finished()
        if self.pipeline and self.spec_mode == "none" and self.runner.can_pipeline(plan):
            handle = self.runner.launch_decode(plan)
            return self._finish_pipelined(plan, handle)
        speculate = False
        if self.spec_mode != "none" and plan.kind in ("decode", "verify"):
            speculate = self.gate.next_step() == MtpGate.MEASURE_VERIFY or not self.gate.enabled
            if not speculate and plan.kind == "verify":
                # the gate turned speculation off: drop pending drafts
                for it in plan.items:
                    it.tokens, it.verify = it.tokens[:1], 0
                plan = StepPlan("decode", plan.items)
        t0 = time.perf_counter()
        try:
            result = self.runner.execute(plan)
        except FatalDeviceError as e:
            self.fault.set(str(e))
            raise
        except RuntimeError as e:
            if "CUDA" in str(e) or "device status" in str(e):
                self.fault.set(str(e))
                raise FatalDeviceError(str(e)) from e
            raise
        track = self.spec_mode != "none"                   # the gate / ladder bookkeeping is only read when speculating
        before = {it.seq.seq_id: len(it.seq.tokens) for it in plan.items} if track else None
        drafts = None
        outs = sch.apply(plan, result, None)
        self.runner.commit_recurrent(plan)                 # verify steps on recurrent models: write-on-accept
        if speculate:
            k = self.ladder.drafts_for(len(plan.items))
            if self.dflash_rung is not None:
                if plan.kind == "verify" and len(plan.items) == 1:
                    self.dflash_rung.observe(getattr(plan.items[0].seq, "last_accept", 0) > 0)
                k = self.args.dflash_gamma or self.dflash_rung.gamma(len(plan.items))
            if k > 0:
                accepted = [len(it.seq.tokens) - before[it.seq.seq_id] for it in plan.items]
                if self.spec_mode in ("mtp", "dflash"):
                    drafts = self.runner.propose(plan, result, accepted, k)
                else:
                    drafts = [self.ngram.propose(it.seq.tokens, k) if not it.seq.is_finished() else []
                              for it in plan.items]
                for it, d in zip(plan.items, drafts):
                    # verification is by argmax: only greedy requests speculate (a sampled request
                    # batched in the same step keeps its sampler)
                    if not it.seq.is_finished() and it.seq.req.params.greedy:
                        room = it.seq.req.params.max_tokens - it.seq.num_output - 1
                        it.seq.drafts = list(d[:max(0, room)])
        if not speculate and plan.kind in ("decode", "verify"):
            # predicted outputs: a request that brought its own guess of the answer is verified
            # against it a few tokens per step, whatever the engine's own speculation mode
            for it in plan.items:
                pred = it.seq.req.params.prediction_ids
                if pred and it.seq.req.params.greedy and not it.seq.is_finished():     # verification is by argmax: lossless for greedy requests only
                    from ..speculative.ngram import propose_from_prediction
                    room = it.seq.req.params.max_tokens - it.seq.num_output - 1
                    d = propose_from_prediction(it.seq.tokens[it.seq.prompt_len:], pred, min(self.args.prediction_drafts, max(0, room)))
                    it.seq.drafts = d
        dt = time.perf_counter() - t0
        if track and plan.kind in ("decode", "verify"):
            emitted = sum(len(it.seq.tokens) - before[it.seq.seq_id] for it in plan.items)
            self.gate.record(emitted, dt)
            self.spec_stats.steps += 1
            self.spec_stats.emitted += emitted
            self.spec_stats.drafted += sum(it.verify for it in plan.items)
            self.spec_stats.accepted += sum(getattr(it.seq, "last_accept", 0) for it in plan.items)
        self.step_count += 1
        if self._redzone_every and self.step_count % self._redzone_every == 0:
            self.check_red_zones()
        return outs

    # ------------------------------------------------------------------ rollback
    def rollback_request(self, request_id: str, keep_output_tokens: int) -> bool:
        """Rewind a decoding request to its first `keep_output_tokens` generated tokens (a loop
        detector or a tool-call parser decides where). Returns False when the request is not
        decoding or, on a recurrent model, no state snapshot exists at that length
        (`scheduler.rollback_positions` lists the reachable lengths)."""
        self.flush()
        for seq in self.scheduler.running:
            if seq.req.request_id == request_id:
                return self.scheduler.rollback(seq, keep_output_tokens)
        return False

    # ------------------------------------------------------------------ offline loop
    def generate(self, prompts: Iterable[Seq[int]], params: Union[SamplingParams, Seq[SamplingParams], None] = None,
                 images: Optional[Seq] = None) -> List[RequestOutput]:
        """``images``: per prompt, the list of images its placeholder tokens stand for (or None)."""
        prompts = list(prompts)
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        images = list(images) if images is not None else [None] * len(prompts)
        ids = [self.add_request(p, sp, images=im) for p, sp, im in zip(prompts, params, images)]
        done: Dict[str, RequestOutput] = {}
        while len(done) < len(ids):
            outs = self.step()
            for o in outs:
                if o.finished:
                    done[o.request_id] = o
            if not outs and not self.has_work():
                break
        return [done[i] for i in ids if i in done]

    def close(self) -> None:
        """Ordered teardown: finish the step in flight, abort what is queued, drop the CUDA graphs (they hold
        the static buffers), then close what owns files or threads — swap files, state and KV tiers, the expert
        store — and finally the pools. Safe to call twice; the engine takes no requests afterwards.
        Role of the reference's scoped teardown (crates/core/src/scope.rs)."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        try:
            self.flush()
        except Exception:
            pass
        for seq in list(self.scheduler.waiting) + list(self.scheduler.prefilling) + list(self.scheduler.running):
            self.scheduler.abort(seq.req.request_id)
        self.runner.graphs.clear()
        for owner in (getattr(self, "kv_tier", None), getattr(getattr(self, "paged_experts", None), "reader", None)):
            if owner is not None:
                owner.close()
        if self.prefix is not None:
            self.prefix.clear()
        self.fault.set("engine closed")

    def check_red_zones(self) -> list:
        """Compare the guard bands behind the engine's pools (``METRALE_REDZONE``); a damaged band
        latches the fault with the name of the buffer that was overrun."""
        from ..utils.alloc_ledger import ledger
        bad = ledger().check()
        if bad:
            self.fault.set("red zone overwritten behind " + ", ".join(f"{b['name']} ({b['site']}, {b['bytes_overwritten']} bytes)" for b in bad))
        return bad

    def memory_report(self) -> dict:
        """The allocation ledger: long-lived device allocations by name and call site, and what the
        caching allocator holds beyond them."""
        from ..utils.alloc_ledger import ledger
        led = ledger()
        return {"allocations": led.report(), "ledger_bytes": led.total_bytes(), "slack_bytes": led.slack(self.device),
                "redzone_bytes": led.redzone}

    def stats(self) -> dict:
        s = self.scheduler.snapshot()
        s.update({"steps": self.step_count, "graph_replays": self.runner.graph_replays,
                  "h2d_bytes": self.runner.h2d_bytes, "d2h_bytes": self.runner.d2h_bytes,
                  "spec_accept_len": self.spec_stats.accept_len, "gate_mode": self.gate.mode,
                  "kv_blocks": self.runner.kv.num_blocks, "weights_bytes": self.weights.nbytes()})
        if self.prefix:
            s["prefix_cache"] = self.prefix.stats()
        return s
