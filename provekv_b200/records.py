"""Manifests and receipts of the two-tier pool, as the reference serialises and digests them.

A pool or shell encoded by the kernels is only a drop-in for the reference's if the records that
bind it -- `PoolManifest`, `ShellManifest`, `PoolBuildReceipt`, `ShellMaterializeReceipt`,
`InjectionReceipt` -- have the reference's JSON text, because every digest of a record is
blake3 over `serde_json::to_string(self)` (proveKV/src/manifest.rs:118-121,253-256,
proveKV/src/receipt.rs:142-145,211-214,291-294).  For a derived `Serialize` that text is the struct's
fields in declaration order, no spaces, unit enum variants as their names, `f64` in the shortest
round-trip form (the `ryu` crate's layout) and non-finite floats as `null`: `serde_text` below writes
exactly that.  (The pool id and layer digests are different: they hash a `json!` map, whose keys sort;
those live in `manifest.py`.)

Validation follows the reference's rules and message texts; errors are the classes of `codec.py`
named after the reference's error variants (proveKV/src/error.rs:5-59).
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field

from .codec import (CODEC_EXACT_FALLBACK, CODEC_FIB_K4_N32, CODEC_FIB_K4_N32_BATCHED, CODEC_TURBO_8BIT,
                    CODEC_TURBO_8BIT_BATCHED, CODEC_TURBO_8BIT_BATCHED_LOSSY, FibConfig, InvalidManifest,
                    InvalidPolicy, InvalidReceipt, InvalidShape, TurboConfig, turbo_batched_codec_id)

__all__ = ["serde_f64", "serde_f32", "F32", "serde_text", "digest_of", "KvTensorShape", "CompressionPolicy", "PoolManifest",
           "ShellManifest", "PoolBuildReceipt", "ShellMaterializeReceipt", "BlockInjectionTrace",
           "InjectionReceipt", "allowed_shell_codecs", "now_unix", "POOL_MANIFEST_SCHEMA",
           "SHELL_MANIFEST_SCHEMA", "POOL_BUILD_RECEIPT_SCHEMA", "SHELL_MATERIALIZE_RECEIPT_SCHEMA",
           "INJECTION_RECEIPT_SCHEMA"]

POOL_MANIFEST_SCHEMA = "pool_manifest_v1"                          # manifest.rs:6
SHELL_MANIFEST_SCHEMA = "shell_manifest_v1"                        # manifest.rs:7
POOL_BUILD_RECEIPT_SCHEMA = "pool_build_receipt_v1"                # receipt.rs:6
SHELL_MATERIALIZE_RECEIPT_SCHEMA = "shell_materialize_receipt_v1"  # receipt.rs:7
INJECTION_RECEIPT_SCHEMA = "injection_receipt_v1"                  # receipt.rs:8


def _ryu_layout(digits: str, k: int, max_kk: int, min_kk: int) -> str:
    """The `ryu` crate's layout of the decimal `digits` x 10^k: plain decimal with at least one fractional
    digit while the decimal point falls within (min_kk, max_kk] digits of the first one, otherwise
    `d.ddde<exp>` with no `+` and no leading zeros."""
    n = len(digits)
    kk = n + k
    if 0 <= k and kk <= max_kk:
        return digits + "0" * k + ".0"
    if 0 < kk <= max_kk:
        return digits[:kk] + "." + digits[kk:]
    if min_kk < kk <= 0:
        return "0." + "0" * (-kk) + digits
    if n == 1:
        return f"{digits}e{kk - 1}"
    return f"{digits[0]}.{digits[1:]}e{kk - 1}"


def _shortest_digits(text: str):
    """(digits, k) with value = digits x 10^k from a shortest round-trip repr such as '1.5e-07' or '12.34'."""
    mant, _, exp = text.partition("e")
    whole, _, frac = mant.partition(".")
    k = (int(exp) if exp else 0) - len(frac)
    digits = (whole + frac).lstrip("0")
    stripped = digits.rstrip("0")
    return stripped, k + len(digits) - len(stripped)


def serde_f64(x: float) -> str:
    """A binary64 as serde_json writes it: the shortest digits that round-trip, in the `ryu` layout
    (decimal point within (-5, 16] digits of the first digit, else exponent form); non-finite -> null."""
    if not math.isfinite(x):
        return "null"
    sign = "-" if math.copysign(1.0, x) < 0 else ""
    if x == 0:
        return sign + "0.0"
    digits, k = _shortest_digits(repr(abs(float(x))))
    return sign + _ryu_layout(digits, k, 16, -5)


def serde_f32(x) -> str:
    """A binary32 as serde_json writes it: shortest digits that round-trip as binary32, `ryu` layout with the
    decimal point within (-6, 13] digits of the first digit."""
    import numpy as np
    v = np.float32(x)
    if not np.isfinite(v):
        return "null"
    sign = "-" if np.signbit(v) else ""
    if v == 0:
        return sign + "0.0"
    digits, k = _shortest_digits(np.format_float_scientific(abs(v), unique=True, trim="-"))
    return sign + _ryu_layout(digits, k, 13, -6)


class F32(float):
    """Marks a number that `serde_text` writes as binary32."""


def serde_text(obj) -> str:
    """Compact JSON of dicts (in insertion order), lists, strings, bools, ints, floats and None."""
    if obj is None:
        return "null"
    if obj is True:
        return "true"
    if obj is False:
        return "false"
    if isinstance(obj, int):
        return str(obj)
    if isinstance(obj, F32):
        return serde_f32(obj)
    if isinstance(obj, float):
        return serde_f64(obj)
    if isinstance(obj, str):
        return json.dumps(obj, ensure_ascii=False)
    if isinstance(obj, (list, tuple)):
        return "[" + ",".join(serde_text(v) for v in obj) + "]"
    if isinstance(obj, dict):
        return "{" + ",".join(json.dumps(k, ensure_ascii=False) + ":" + serde_text(v) for k, v in obj.items()) + "}"
    raise TypeError(f"not serialisable: {type(obj).__name__}")


def digest_of(record) -> str:
    """blake3 of the record's JSON text, lower-case hex."""
    import blake3
    return blake3.blake3(serde_text(record.as_json()).encode()).hexdigest()


def now_unix() -> int:
    """receipt.rs:297-303."""
    return int(time.time())


def _ratio(raw: int, stored: int) -> float:
    """manifest.rs:64-68, receipt.rs:62-66."""
    return raw / stored if stored > 0 else 0.0


def _debug_list(items) -> str:
    """A list of strings as Rust's `{:?}` prints it."""
    return "[" + ", ".join(json.dumps(i, ensure_ascii=False) for i in items) + "]"


def allowed_shell_codecs() -> list[str]:
    """policy.rs:84-111: the three 8-bit ids, the exact fallback, then both batched ids of every other width."""
    ids = [CODEC_TURBO_8BIT, CODEC_TURBO_8BIT_BATCHED, CODEC_TURBO_8BIT_BATCHED_LOSSY, CODEC_EXACT_FALLBACK]
    for bits in range(2, 17):
        if bits != 8:
            ids += [turbo_batched_codec_id(bits, False), turbo_batched_codec_id(bits, True)]
    return ids


@dataclass(frozen=True)
class KvTensorShape:
    """proveKV/src/shape.rs:20-34; `attention_type` is one of mha / mqa / gqa and serialises in lower case (:7)."""
    attention_type: str
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    hidden_size: int

    def __post_init__(self):
        object.__setattr__(self, "attention_type", str(self.attention_type).lower())

    def validate(self) -> None:
        """shape.rs:38-91."""
        for name in ("num_layers", "num_heads", "num_kv_heads", "head_dim", "hidden_size"):
            if getattr(self, name) == 0:
                raise InvalidShape(f"{name} must be > 0")
        kind = self.attention_type.lower()
        if kind == "mha":
            if self.num_kv_heads != self.num_heads:
                raise InvalidShape(f"MHA requires num_kv_heads ({self.num_kv_heads}) == num_heads ({self.num_heads})")
        elif kind == "mqa":
            if self.num_kv_heads != 1:
                raise InvalidShape(f"MQA requires num_kv_heads == 1, got {self.num_kv_heads}")
        elif kind == "gqa":
            if self.num_kv_heads >= self.num_heads:
                raise InvalidShape(f"GQA requires num_kv_heads ({self.num_kv_heads}) < num_heads ({self.num_heads})")
        else:
            raise InvalidShape(f"unknown attention_type: {self.attention_type}")
        if self.hidden_size % self.num_heads != 0:
            raise InvalidShape(f"hidden_size ({self.hidden_size}) must be divisible by num_heads ({self.num_heads})")

    def as_json(self) -> dict:
        return {"attention_type": self.attention_type.lower(), "num_layers": self.num_layers,
                "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
                "hidden_size": self.hidden_size}

    @classmethod
    def from_json(cls, obj: dict) -> "KvTensorShape":
        return cls(obj["attention_type"], int(obj["num_layers"]), int(obj["num_heads"]), int(obj["num_kv_heads"]),
                   int(obj["head_dim"]), int(obj["hidden_size"]))

    def total_kv_bytes(self, num_tokens: int) -> int:
        """shape.rs:104-113: layers x 2 x kv heads x head_dim x tokens f32 values."""
        return self.num_layers * 2 * self.num_kv_heads * self.head_dim * num_tokens * 4


@dataclass(frozen=True)
class CompressionPolicy:
    """proveKV/src/policy.rs:292-350."""
    shared_codec: str = CODEC_FIB_K4_N32_BATCHED
    shell_codec: str = turbo_batched_codec_id(4, False)
    fib_config: FibConfig = field(default_factory=FibConfig)
    turbo_config: TurboConfig = field(default_factory=TurboConfig)

    @classmethod
    def default_two_tier(cls) -> "CompressionPolicy":
        return cls()

    @classmethod
    def default_two_tier_lossy(cls) -> "CompressionPolicy":
        return cls(shell_codec=turbo_batched_codec_id(4, True), turbo_config=TurboConfig(4, 32, True))

    def validate(self) -> None:
        """policy.rs:323-349."""
        allowed_shared = [CODEC_FIB_K4_N32, CODEC_FIB_K4_N32_BATCHED, CODEC_EXACT_FALLBACK]
        if self.shared_codec not in allowed_shared:
            raise InvalidPolicy(f"shared_codec must be one of {_debug_list(allowed_shared)}, got '{self.shared_codec}'")
        allowed_shell = allowed_shell_codecs()
        if self.shell_codec not in allowed_shell:
            raise InvalidPolicy(f"shell_codec must be one of {_debug_list(allowed_shell)}, got '{self.shell_codec}'")
        self.fib_config.validate()
        self.turbo_config.validate()

    def as_json(self) -> dict:
        return {"shared_codec": self.shared_codec, "shell_codec": self.shell_codec,
                "fib_config": self.fib_config.as_json(), "turbo_config": self.turbo_config.as_json()}

    @classmethod
    def from_json(cls, obj: dict) -> "CompressionPolicy":
        fc = obj["fib_config"]
        return cls(obj["shared_codec"], obj["shell_codec"],
                   FibConfig(int(fc["k"]), int(fc["n"]), int(fc["training_samples"]), int(fc["lloyd_restarts"]),
                             int(fc["lloyd_iterations"])),
                   TurboConfig.from_json(obj["turbo_config"]))


def _shell_codec_check(shell_codec: str, turbo_config: TurboConfig) -> None:
    """manifest.rs:146-168,211-233: the codec id has to be the one the turbo configuration implies."""
    expected = turbo_batched_codec_id(turbo_config.bits, turbo_config.lossy_radii)
    if shell_codec != expected:
        raise InvalidManifest(
            f"shell_codec '{shell_codec}' does not match turbo_config (bits={turbo_config.bits}, "
            f"lossy={'true' if turbo_config.lossy_radii else 'false'}); expected '{expected}'")


@dataclass
class PoolManifest:
    """proveKV/src/manifest.rs:23-122."""
    pool_id: str
    shape: KvTensorShape
    policy: CompressionPolicy
    num_shared_tokens: int
    num_layers: int
    pool_size_bytes: int
    shared_codec: str
    compression_ratio: float
    built_at_unix: int
    build_seed: int
    schema_version: str = POOL_MANIFEST_SCHEMA

    @classmethod
    def new(cls, pool_id: str, shape: KvTensorShape, policy: CompressionPolicy, num_shared_tokens: int,
            num_layers: int, pool_size_bytes: int, raw_size_bytes: int, build_seed: int,
            built_at_unix: int) -> "PoolManifest":
        """manifest.rs:51-94: the ratio is raw / stored (0 for an empty pool); an empty policy codec id
        falls back to the per-vector fib id."""
        m = cls(pool_id, shape, policy, num_shared_tokens, num_layers, pool_size_bytes,
                policy.shared_codec or CODEC_FIB_K4_N32, _ratio(raw_size_bytes, pool_size_bytes), built_at_unix,
                build_seed)
        m.validate()
        return m

    def validate(self) -> None:
        """manifest.rs:97-113."""
        if self.schema_version != POOL_MANIFEST_SCHEMA:
            raise InvalidManifest(f"expected schema {POOL_MANIFEST_SCHEMA}, got {self.schema_version}")
        if not self.pool_id:
            raise InvalidManifest("pool_id is empty")
        self.shape.validate()
        self.policy.validate()

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "pool_id": self.pool_id, "shape": self.shape.as_json(),
                "policy": self.policy.as_json(), "num_shared_tokens": self.num_shared_tokens,
                "num_layers": self.num_layers, "pool_size_bytes": self.pool_size_bytes,
                "shared_codec": self.shared_codec, "compression_ratio": float(self.compression_ratio),
                "built_at_unix": self.built_at_unix, "build_seed": self.build_seed}

    @classmethod
    def from_json(cls, obj: dict) -> "PoolManifest":
        return cls(obj["pool_id"], KvTensorShape.from_json(obj["shape"]), CompressionPolicy.from_json(obj["policy"]),
                   int(obj["num_shared_tokens"]), int(obj["num_layers"]), int(obj["pool_size_bytes"]),
                   obj["shared_codec"], float(obj["compression_ratio"]), int(obj["built_at_unix"]),
                   int(obj["build_seed"]), obj["schema_version"])

    def to_json(self) -> str:
        return serde_text(self.as_json())

    def digest(self) -> str:
        return digest_of(self)


@dataclass
class ShellManifest:
    """proveKV/src/manifest.rs:124-257.  `component_kinds` holds "KeyValue" or {"RuntimeSpecific": name},
    the externally tagged form of `ShellComponentKind` (manifest.rs:10-14)."""
    agent_id: str
    pool_digest: str
    num_unique_tokens: int
    num_unique_layers: int
    shell_size_bytes: int
    shell_codec: str
    materialized_at_unix: int
    materialize_seed: int
    head_dim: int
    num_kv_heads: int
    turbo_config: TurboConfig
    component_kinds: list = field(default_factory=list)
    schema_version: str = SHELL_MANIFEST_SCHEMA

    @classmethod
    def new(cls, agent_id: str, pool_digest: str, num_unique_tokens: int, num_unique_layers: int,
            shell_size_bytes: int, shell_codec: str, materialize_seed: int, materialized_at_unix: int,
            head_dim: int, num_kv_heads: int, turbo_config: TurboConfig) -> "ShellManifest":
        """manifest.rs:130-189 (argument order as there: seed before time)."""
        _shell_codec_check(shell_codec, turbo_config)
        m = cls(agent_id, pool_digest, num_unique_tokens, num_unique_layers, shell_size_bytes, shell_codec,
                materialized_at_unix, materialize_seed, head_dim, num_kv_heads, turbo_config)
        m.validate()
        return m

    def validate(self) -> None:
        """manifest.rs:192-250."""
        if self.schema_version != SHELL_MANIFEST_SCHEMA:
            raise InvalidManifest(f"expected schema {SHELL_MANIFEST_SCHEMA}, got {self.schema_version}")
        if not self.agent_id:
            raise InvalidManifest("agent_id is empty")
        if not self.pool_digest:
            raise InvalidManifest("pool_digest is empty")
        _shell_codec_check(self.shell_codec, self.turbo_config)

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "agent_id": self.agent_id, "pool_digest": self.pool_digest,
                "num_unique_tokens": self.num_unique_tokens, "num_unique_layers": self.num_unique_layers,
                "shell_size_bytes": self.shell_size_bytes, "shell_codec": self.shell_codec,
                "materialized_at_unix": self.materialized_at_unix, "materialize_seed": self.materialize_seed,
                "head_dim": self.head_dim, "num_kv_heads": self.num_kv_heads,
                "turbo_config": self.turbo_config.as_json(), "component_kinds": list(self.component_kinds)}

    @classmethod
    def from_json(cls, obj: dict) -> "ShellManifest":
        """`component_kinds` may be absent in records written before the field existed (manifest.rs:127)."""
        return cls(obj["agent_id"], obj["pool_digest"], int(obj["num_unique_tokens"]), int(obj["num_unique_layers"]),
                   int(obj["shell_size_bytes"]), obj["shell_codec"], int(obj["materialized_at_unix"]),
                   int(obj["materialize_seed"]), int(obj["head_dim"]), int(obj["num_kv_heads"]),
                   TurboConfig.from_json(obj["turbo_config"]), list(obj.get("component_kinds", [])),
                   obj["schema_version"])

    def to_json(self) -> str:
        return serde_text(self.as_json())

    def digest(self) -> str:
        return digest_of(self)


@dataclass
class PoolBuildReceipt:
    """proveKV/src/receipt.rs:18-146.  `backend` says where the encode actually ran ("cpu" unless the
    builder states otherwise; receipt.rs:40-46,90-93); a record without the field reads as "cpu"."""
    pool_digest: str
    layer_digests: list
    codebook_digest: str
    rotation_digest: str
    total_tokens: int
    fib_build_ms: int
    pool_size_bytes: int
    raw_size_bytes: int
    compression_ratio: float
    policy_snapshot: CompressionPolicy
    seeded_with: int
    built_at_unix: int
    backend: str = "cpu"
    schema_version: str = POOL_BUILD_RECEIPT_SCHEMA

    @classmethod
    def new(cls, pool_digest: str, layer_digests, codebook_digest: str, rotation_digest: str, total_tokens: int,
            fib_build_ms: int, pool_size_bytes: int, raw_size_bytes: int, policy_snapshot: CompressionPolicy,
            seeded_with: int, built_at_unix: int) -> "PoolBuildReceipt":
        """receipt.rs:49-88 (no validation at construction, as there)."""
        return cls(pool_digest, list(layer_digests), codebook_digest, rotation_digest, total_tokens, fib_build_ms,
                   pool_size_bytes, raw_size_bytes, _ratio(raw_size_bytes, pool_size_bytes), policy_snapshot,
                   seeded_with, built_at_unix)

    def with_backend(self, backend: str) -> "PoolBuildReceipt":
        self.backend = str(backend)
        return self

    def validate(self) -> None:
        """receipt.rs:96-126: schema, pool digest, and non-empty codebook / rotation digests."""
        if self.schema_version != POOL_BUILD_RECEIPT_SCHEMA:
            raise InvalidReceipt(f"expected schema {POOL_BUILD_RECEIPT_SCHEMA}, got {self.schema_version}")
        if not self.pool_digest:
            raise InvalidReceipt("pool_digest is empty")
        if not self.codebook_digest:
            raise InvalidReceipt("codebook_digest is empty (pre-F5 receipt, must rebuild)")
        if not self.rotation_digest:
            raise InvalidReceipt("rotation_digest is empty (pre-F5 receipt, must rebuild)")

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "pool_digest": self.pool_digest,
                "layer_digests": list(self.layer_digests), "codebook_digest": self.codebook_digest,
                "rotation_digest": self.rotation_digest, "total_tokens": self.total_tokens,
                "fib_build_ms": self.fib_build_ms, "pool_size_bytes": self.pool_size_bytes,
                "raw_size_bytes": self.raw_size_bytes, "compression_ratio": float(self.compression_ratio),
                "policy_snapshot": self.policy_snapshot.as_json(), "seeded_with": self.seeded_with,
                "built_at_unix": self.built_at_unix, "backend": self.backend}

    @classmethod
    def from_json(cls, obj: dict) -> "PoolBuildReceipt":
        return cls(obj["pool_digest"], list(obj["layer_digests"]), obj["codebook_digest"], obj["rotation_digest"],
                   int(obj["total_tokens"]), int(obj["fib_build_ms"]), int(obj["pool_size_bytes"]),
                   int(obj["raw_size_bytes"]), float(obj["compression_ratio"]),
                   CompressionPolicy.from_json(obj["policy_snapshot"]), int(obj["seeded_with"]),
                   int(obj["built_at_unix"]), obj.get("backend", "cpu"), obj["schema_version"])

    def to_json(self) -> str:
        return serde_text(self.as_json())

    def digest(self) -> str:
        return digest_of(self)


@dataclass
class ShellMaterializeReceipt:
    """proveKV/src/receipt.rs:148-215."""
    agent_id: str
    pool_digest: str
    shell_digest: str
    num_unique_tokens: int
    shell_size_bytes: int
    materialize_ms: int
    materialized_at_unix: int
    schema_version: str = SHELL_MATERIALIZE_RECEIPT_SCHEMA

    @classmethod
    def new(cls, agent_id, pool_digest, shell_digest, num_unique_tokens, shell_size_bytes, materialize_ms,
            materialized_at_unix) -> "ShellMaterializeReceipt":
        return cls(agent_id, pool_digest, shell_digest, num_unique_tokens, shell_size_bytes, materialize_ms,
                   materialized_at_unix)

    def validate(self) -> None:
        """receipt.rs:183-208."""
        if self.schema_version != SHELL_MATERIALIZE_RECEIPT_SCHEMA:
            raise InvalidReceipt(f"expected schema {SHELL_MATERIALIZE_RECEIPT_SCHEMA}, got {self.schema_version}")
        for name in ("agent_id", "pool_digest", "shell_digest"):
            if not getattr(self, name):
                raise InvalidReceipt(f"{name} is empty")

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "agent_id": self.agent_id, "pool_digest": self.pool_digest,
                "shell_digest": self.shell_digest, "num_unique_tokens": self.num_unique_tokens,
                "shell_size_bytes": self.shell_size_bytes, "materialize_ms": self.materialize_ms,
                "materialized_at_unix": self.materialized_at_unix}

    @classmethod
    def from_json(cls, obj: dict) -> "ShellMaterializeReceipt":
        return cls(obj["agent_id"], obj["pool_digest"], obj["shell_digest"], int(obj["num_unique_tokens"]),
                   int(obj["shell_size_bytes"]), int(obj["materialize_ms"]), int(obj["materialized_at_unix"]),
                   obj["schema_version"])

    def to_json(self) -> str:
        return serde_text(self.as_json())

    def digest(self) -> str:
        return digest_of(self)


@dataclass(frozen=True)
class BlockInjectionTrace:
    """proveKV/src/receipt.rs:231-241: `source` is "pool" or "shell"."""
    layer: int
    source: str
    source_digest: str
    target_position: int

    def as_json(self) -> dict:
        return {"layer": self.layer, "source": self.source, "source_digest": self.source_digest,
                "target_position": self.target_position}


@dataclass
class InjectionReceipt:
    """proveKV/src/receipt.rs:217-295."""
    agent_id: str
    pool_digest: str
    shell_digest: str
    blocks_injected: int
    block_traces: list
    injected_at_unix: int
    schema_version: str = INJECTION_RECEIPT_SCHEMA

    @classmethod
    def new(cls, agent_id, pool_digest, shell_digest, blocks_injected, block_traces,
            injected_at_unix) -> "InjectionReceipt":
        return cls(agent_id, pool_digest, shell_digest, blocks_injected, list(block_traces), injected_at_unix)

    def validate(self) -> None:
        """receipt.rs:263-288."""
        if self.schema_version != INJECTION_RECEIPT_SCHEMA:
            raise InvalidReceipt(f"expected schema {INJECTION_RECEIPT_SCHEMA}, got {self.schema_version}")
        for name in ("agent_id", "pool_digest", "shell_digest"):
            if not getattr(self, name):
                raise InvalidReceipt(f"{name} is empty")

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "agent_id": self.agent_id, "pool_digest": self.pool_digest,
                "shell_digest": self.shell_digest, "blocks_injected": self.blocks_injected,
                "block_traces": [t.as_json() for t in self.block_traces], "injected_at_unix": self.injected_at_unix}

    @classmethod
    def from_json(cls, obj: dict) -> "InjectionReceipt":
        traces = [BlockInjectionTrace(int(t["layer"]), t["source"], t["source_digest"], int(t["target_position"]))
                  for t in obj["block_traces"]]
        return cls(obj["agent_id"], obj["pool_digest"], obj["shell_digest"], int(obj["blocks_injected"]), traces,
                   int(obj["injected_at_unix"]), obj["schema_version"])

    def to_json(self) -> str:
        return serde_text(self.as_json())

    def digest(self) -> str:
        return digest_of(self)
