"""Benchmark gate records: a measured result is frozen into a record (metric, value, config,
source-closure hash of the kernel library, device, timestamp), compared against a threshold
or an earlier record, and signed with Ed25519 so that a published number can be tied to the
exact kernel sources that produced it. Role of the reference's gate records + signing +
coverage-by-content check (``crates/bench/src/gate``)."""
from __future__ import annotations

import base64
import hashlib
import json
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Dict, Optional


def kernel_closure_hash() -> str:
    """SHA-256 over every kernel source, header and the compiler flags (what the build stamps)."""
    from ..ops import build as b
    return b._digest(b.sources() + sorted(b.CSRC.glob("*.cuh")) + sorted(b.CSRC.glob("*.h")))


@dataclass
class GateRecord:
    name: str
    metric: str
    value: float
    unit: str
    higher_is_better: bool = True
    config: Dict[str, object] = field(default_factory=dict)
    closure: str = ""
    device: str = ""
    created: float = field(default_factory=time.time)
    signature: Optional[str] = None
    public_key: Optional[str] = None

    def payload(self) -> bytes:
        d = asdict(self)
        d.pop("signature"), d.pop("public_key")
        return json.dumps(d, sort_keys=True, separators=(",", ":")).encode()

    def digest(self) -> str:
        return hashlib.sha256(self.payload()).hexdigest()

    # ------------------------------------------------------------------ signing
    def sign(self, private_key) -> "GateRecord":
        from cryptography.hazmat.primitives import serialization
        self.signature = base64.b64encode(private_key.sign(self.payload())).decode()
        pub = private_key.public_key().public_bytes(serialization.Encoding.Raw, serialization.PublicFormat.Raw)
        self.public_key = base64.b64encode(pub).decode()
        return self

    def verify(self, trusted_public_key_b64: Optional[str] = None) -> bool:
        from cryptography.exceptions import InvalidSignature
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PublicKey
        if not self.signature or not self.public_key:
            return False
        if trusted_public_key_b64 is not None and trusted_public_key_b64 != self.public_key:
            return False
        try:
            Ed25519PublicKey.from_public_bytes(base64.b64decode(self.public_key)).verify(
                base64.b64decode(self.signature), self.payload())
            return True
        except InvalidSignature:
            return False

    # ------------------------------------------------------------------ gating
    def passes(self, threshold: float) -> bool:
        return self.value >= threshold if self.higher_is_better else self.value <= threshold

    def regression_vs(self, earlier: "GateRecord", tolerance: float = 0.03) -> Optional[str]:
        """None when this record is no worse than `earlier` beyond `tolerance`, else a message."""
        if earlier.metric != self.metric or earlier.unit != self.unit:
            return f"not comparable: {earlier.metric} [{earlier.unit}] vs {self.metric} [{self.unit}]"
        ratio = self.value / earlier.value if earlier.value else float("inf")
        bad = ratio < 1 - tolerance if self.higher_is_better else ratio > 1 + tolerance
        return f"{self.name}: {self.value:g} vs {earlier.value:g} {self.unit} ({ratio:.3f}x)" if bad else None

    # ------------------------------------------------------------------ IO
    def save(self, path) -> None:
        Path(path).write_text(json.dumps(asdict(self), indent=1, sort_keys=True))

    @classmethod
    def load(cls, path) -> "GateRecord":
        return cls(**json.loads(Path(path).read_text()))

    @classmethod
    def from_bench_line(cls, name: str, line: Dict[str, object], device: str = "") -> "GateRecord":
        """Build a record from the JSON line `bench.py` prints."""
        return cls(name=name, metric=str(line["metric"]), value=float(line["value"]), unit=str(line["unit"]),
                   higher_is_better=bool(line.get("higher_is_better", True)), config=dict(line.get("config", {})),
                   closure=kernel_closure_hash(), device=device)


def new_signing_key():
    from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
    return Ed25519PrivateKey.generate()
