"""Every ``METRALE_*`` environment lever the engine reads, declared in one table; starting with
an undeclared ``METRALE_*`` variable set is refused (a typo must not silently do nothing).
Role of ``crates/config/src/levers.rs:3-14``."""
from __future__ import annotations

import os
from typing import Dict, List

LEVERS: Dict[str, str] = {
    "METRALE_PDL": "programmatic dependent launch: 0 = off, 1 = every kernel, 2 = GEMMs only (default)",
    "METRALE_B200_AUTOBUILD": "0 = never build the kernel library on import (default 1)",
    "METRALE_COMM_DIAGNOSTICS": "1 = log every collective submission with a sequence number",
    "METRALE_MTP_K_LADDER": "draft-width ladder 'width:k,...' (default 4:3,8:3,16:1,32:1)",
    "METRALE_NO_MTP_K_LADDER": "1 = disable the draft-width ladder",
    "METRALE_ATTN_PART_TOKENS": "split-KV partition size in tokens (default 512)",
    "METRALE_DEBUG_SYNC_KERNELS": "1 = synchronise and check the status word after every step",
    "METRALE_KV_POISON": "1 = fill fresh KV blocks with NaN bytes",
    "METRALE_TELEMETRY": "off | basic | kernel",
    "METRALE_MAX_BODY_BYTES": "HTTP request body limit in bytes (default 32 MiB)",
    "METRALE_LOOP_NO_SUPPRESS": "1 = the cross-turn loop detector never masks the tool-call opener (soft bias only)",
    "METRALE_PERSISTENT_PREFILL": "0 = prefill GEMMs (several token tiles) keep one tile per CTA instead of the persistent two-accumulator kernel",
    "METRALE_NVTX": "1 = NVTX ranges around engine steps (for Nsight timelines)",
    "METRALE_OTLP_ENDPOINT": "OTLP/HTTP collector base URL; set = push metrics every METRALE_OTLP_PERIOD_S (default 10)",
    "METRALE_OTLP_PERIOD_S": "seconds between OTLP pushes",
    "METRALE_NATIVE_RUNTIME": "0 = keep allocator / prefix index / JSON grammar on the Python implementations",
    "METRALE_NVLS": "fused collectives: 0 = one peer store per rank, 1 = NVLink multicast stores, 2 = reduction inside the switch (multimem.ld_reduce)",
    "METRALE_NO_FUSED_COLLECTIVES": "1 = NCCL collectives after plain GEMMs",
    "METRALE_MOE_FOLD_SHARED": "0 = the shared expert keeps its own dense GEMMs instead of riding in the grouped expert stack",
    "METRALE_ATTN_TC_VMN": "tcgen05 prefill attention: 1 = V read as an MN-major operand (no transposition while staging), 0 = transposed",
    "METRALE_GROUPED_CTAS": "1 = grouped expert GEMMs of 16- / 32-row token tiles keep one CTA per SM (default 2: two co-resident CTAs, half the stages each)",
    "METRALE_INDEX_TC": "0 = the sparse-attention indexer score stays on the CUDA-core kernel instead of the mma.sync kernel",
    "METRALE_REDZONE": "bytes of guard band behind every ledger allocation (multiple of 16; default 0 = off)",
    "METRALE_REDZONE_EVERY": "with METRALE_REDZONE: check the guard bands every n-th engine step (default 0 = only on request)",
    "METRALE_ATTN_TC": "0 = prefill attention stays on the mma.sync kernel instead of the tcgen05 / TMEM kernel",
}


def undeclared(environ=None) -> List[str]:
    env = os.environ if environ is None else environ
    return sorted(k for k in env if k.startswith("METRALE_") and k not in LEVERS)


def check_environment(environ=None) -> None:
    bad = undeclared(environ)
    if bad:
        raise SystemExit(f"undeclared METRALE_* environment variable(s): {', '.join(bad)}; "
                         f"known levers: {', '.join(sorted(LEVERS))}")
