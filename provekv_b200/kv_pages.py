"""fib-quant's KV page contracts (`fib-quant/src/kv/*.rs`, the crate's default-off `kv` feature) with the
codec arithmetic on the GPU.

A KV tensor `[batch][layer][kv_head][token][head_dim]` (f32, canonical contiguous layout) is cut into
pages of `tokens_per_page` tokens; every (batch, layer, head, token) vector is one block, either the
single-vector fib-quant code (`FibQuantizer::encode`, fib-quant/src/codec.rs:465-503: binary64
normalisation and rotation) or, in the protected regions, the raw f32 values.  Decoding uses
`FibQuantizer::decode` (codec.rs:506-537, binary64 inverse).  Here one launch of the exact encoder
(`numerics = single`) covers the whole tensor in place, one launch of `pkv_fib_decode_exact` the whole
set of coded blocks; pages, blocks, receipts and their digests are assembled on the host exactly as the
reference serialises them:

  * digests are `"blake3:" + hex(blake3(domain || 0x00 || serde_json(value)))` (src/digest.rs:6-19) with the
    struct's fields in declaration order; the tensor digest hashes a tag, the element count and the
    little-endian f32 values (kv/receipt.rs:76-90);
  * block order inside a page: batch, layer, head, token (kv/codec.rs:71-113);
  * the page digest covers every field but itself (kv/page.rs:125-160).

What is taken as given: the codebook digest (it hashes the training report, src/codebook.rs:134-157) is
passed in by the owner of the tables; the rotation digest is computed from the matrix that is actually
used (`rotation_digest`, src/rotation.rs:81-101) rather than from a regenerated one, because the
reference's generator streams cannot be reproduced here.  Not restated: calibration, the attention
quality metrics and the CPU reference attention (`kv/calibration.rs`, `quality.rs`, `attention_ref.rs`),
and the per-channel / role-aware axis policies, which the reference's own codec answers with the raw
fallback (kv/codec.rs:262-282).
"""
from __future__ import annotations

import math
import struct
import time
from dataclasses import dataclass, field

import numpy as np

from .records import F32, serde_text

KV_SHAPE_SCHEMA = "fib_quant_kv_tensor_shape_v1"
KV_LAYOUT_SCHEMA = "fib_quant_kv_cache_layout_v1"
KV_PAGE_GEOMETRY_SCHEMA = "fib_quant_kv_page_geometry_v1"
KV_PROFILE_SCHEMA = "fib_quant_kv_compression_profile_v1"
KV_BLOCK_SCHEMA = "fib_quant_kv_encoded_block_v1"
KV_PAGE_SCHEMA = "fib_quant_kv_encoded_page_v1"
KV_RECEIPT_SCHEMA = "fib_quant_kv_receipt_v1"
PROFILE_SCHEMA = "fib_quant_profile_v1"
CODE_SCHEMA = "fib_code_v1"
ROTATION_SCHEMA = "fib_rotation_v1"
ROTATION_ALGORITHM_VERSION = "qr-gaussian-chacha8-sign-corrected-v1"


class KvError(ValueError):
    """The reference's `FibQuantError` variants that these contracts raise, by message."""


def bytes_digest(data: bytes) -> str:
    import blake3
    return "blake3:" + blake3.blake3(data).hexdigest()


def json_digest(domain: str, obj) -> str:
    """src/digest.rs:6-14."""
    return bytes_digest(domain.encode() + b"\x00" + serde_text(obj).encode())


def kv_tensor_digest(values) -> str:
    """kv/receipt.rs:76-90."""
    v = np.ascontiguousarray(values, dtype="<f4").reshape(-1)
    if not np.isfinite(v).all():
        raise KvError("kv tensor contains non-finite value")
    return bytes_digest(b"fib_quant_kv_tensor_f32_v1\x00" + struct.pack("<Q", v.size) + v.tobytes())


def rotation_digest(dim: int, seed: int, matrix) -> str:
    """src/rotation.rs:81-101 over the row-major f64 matrix."""
    m = np.ascontiguousarray(matrix, dtype=np.float64).reshape(-1)
    return json_digest(ROTATION_SCHEMA, {"rotation_schema": ROTATION_SCHEMA,
                                         "algorithm_version": ROTATION_ALGORITHM_VERSION, "dim": int(dim),
                                         "seed": int(seed), "matrix": [float(t) for t in m]})


@dataclass(frozen=True)
class FibQuantProfileV1:
    """src/profile.rs:64-85; `paper_default` is :88-133."""
    ambient_dim: int
    block_dim: int
    codebook_size: int
    paper_rate_bits_per_coord: float
    wire_index_bits: int
    wire_bits_per_coord: float
    norm_format: str
    rotation_seed: int
    rotation_algorithm_version: str
    codebook_seed: int
    codebook_version: str
    source_mode: str
    radius_method: str
    direction_method: str
    lloyd_restarts: int
    lloyd_iterations: int
    training_samples: int
    empty_cell_policy: str
    schema_version: str = PROFILE_SCHEMA

    @classmethod
    def paper_default(cls, ambient_dim: int, block_dim: int, codebook_size: int, seed: int) -> "FibQuantProfileV1":
        _validate_profile_parts(ambient_dim, block_dim, codebook_size)
        bits = wire_index_bits(codebook_size)
        direction = {2: "fibonacci_spiral", 3: "fibonacci_sphere"}.get(block_dim, "roberts_kronecker")
        p = cls(ambient_dim, block_dim, codebook_size, math.log2(codebook_size) / block_dim, bits, bits / block_dim,
                "fp16_paper", seed, ROTATION_ALGORITHM_VERSION, (seed + 0x9E3779B97F4A7C15) & (2 ** 64 - 1),
                "fib-quant:paper-core-v1", "canonical_spherical_beta",
                "k2_closed_form" if block_dim == 2 else "beta_quantile", direction, 4, 25,
                min(max(30 * codebook_size, 256), 10_000_000), "split_highest_distortion")
        p.validate()
        return p

    def block_count(self) -> int:
        return self.ambient_dim // self.block_dim

    def validate(self) -> None:
        """profile.rs:135-211 (the checks that can fail for a record read back from disk)."""
        if self.schema_version != PROFILE_SCHEMA:
            raise KvError(f"profile schema_version {self.schema_version}, expected {PROFILE_SCHEMA}")
        _validate_profile_parts(self.ambient_dim, self.block_dim, self.codebook_size)
        if self.norm_format != "fp16_paper":
            raise KvError("paper profile requires fp16 norm side header")
        if self.source_mode != "canonical_spherical_beta":
            raise KvError("paper profile requires canonical spherical-Beta source mode")
        if self.rotation_algorithm_version != ROTATION_ALGORITHM_VERSION:
            raise KvError(f"rotation_algorithm_version {self.rotation_algorithm_version}, "
                          f"expected {ROTATION_ALGORITHM_VERSION}")
        if self.wire_index_bits != wire_index_bits(self.codebook_size):
            raise KvError(f"wire_index_bits {self.wire_index_bits} does not match ceil(log2(N)) "
                          f"{wire_index_bits(self.codebook_size)}")
        for name, got, want in (("paper_rate_bits_per_coord", self.paper_rate_bits_per_coord,
                                 math.log2(self.codebook_size) / self.block_dim),
                                ("wire_bits_per_coord", self.wire_bits_per_coord,
                                 self.wire_index_bits / self.block_dim)):
            if not math.isfinite(got) or abs(got - want) > 1.0e-12:
                raise KvError(f"{name} {got} does not match {want}")
        if not 1 <= self.lloyd_restarts <= 1024:
            raise KvError(f"lloyd_restarts {self.lloyd_restarts} outside supported range 1..=1024")
        if not 1 <= self.lloyd_iterations <= 100_000:
            raise KvError(f"lloyd_iterations {self.lloyd_iterations} outside supported range 1..=100000")
        if not self.codebook_size <= self.training_samples <= 10_000_000:
            raise KvError(f"training_samples {self.training_samples} outside supported range "
                          f"{self.codebook_size}..=10000000")

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "ambient_dim": self.ambient_dim, "block_dim": self.block_dim,
                "codebook_size": self.codebook_size, "paper_rate_bits_per_coord": float(self.paper_rate_bits_per_coord),
                "wire_index_bits": self.wire_index_bits, "wire_bits_per_coord": float(self.wire_bits_per_coord),
                "norm_format": self.norm_format, "rotation_seed": self.rotation_seed,
                "rotation_algorithm_version": self.rotation_algorithm_version, "codebook_seed": self.codebook_seed,
                "codebook_version": self.codebook_version, "source_mode": self.source_mode,
                "radius_method": self.radius_method, "direction_method": self.direction_method,
                "lloyd_restarts": self.lloyd_restarts, "lloyd_iterations": self.lloyd_iterations,
                "training_samples": self.training_samples, "empty_cell_policy": self.empty_cell_policy}

    def digest(self) -> str:
        self.validate()
        return json_digest(PROFILE_SCHEMA, self.as_json())


def wire_index_bits(codebook_size: int) -> int:
    """profile.rs:219-225: ceil(log2 N)."""
    if codebook_size < 2:
        raise KvError(f"invalid codebook size {codebook_size}")
    return (codebook_size - 1).bit_length()


def _validate_profile_parts(ambient_dim: int, block_dim: int, codebook_size: int) -> None:
    """profile.rs:227-262."""
    if ambient_dim == 0:
        raise KvError("zero dimension")
    if block_dim == 0 or block_dim >= ambient_dim:
        raise KvError(f"invalid block_dim {block_dim} for ambient_dim {ambient_dim}")
    if ambient_dim % block_dim:
        raise KvError(f"ambient_dim {ambient_dim} not divisible by block_dim {block_dim}")
    if ambient_dim > 16_384:
        raise KvError(f"ambient_dim {ambient_dim} exceeds MAX_AMBIENT_DIM 16384")
    if block_dim > 256:
        raise KvError(f"block_dim {block_dim} exceeds MAX_BLOCK_DIM 256")
    if not 2 <= codebook_size <= 1 << 20:
        raise KvError(f"invalid codebook size {codebook_size}")


@dataclass(frozen=True)
class KvTensorShapeV1:
    """kv/shape.rs:43-160.  role: key | value; attention_kind: mha | mqa | gqa; dtype: f16 | bf16 | f32;
    rope_state: pre_rope | post_rope | not_applicable."""
    role: str
    attention_kind: str
    batch: int
    layers: int
    kv_heads: int
    query_heads: int
    tokens: int
    head_dim: int
    dtype: str
    rope_state: str
    schema_version: str = KV_SHAPE_SCHEMA

    def validate(self) -> None:
        if self.schema_version != KV_SHAPE_SCHEMA:
            raise KvError(f"kv shape schema_version {self.schema_version}, expected {KV_SHAPE_SCHEMA}")
        for name in ("batch", "layers", "kv_heads", "query_heads", "tokens", "head_dim"):
            if getattr(self, name) == 0:
                raise KvError(f"kv shape {name} must be > 0")
        if self.attention_kind == "mha" and self.query_heads != self.kv_heads:
            raise KvError("MHA requires query_heads == kv_heads")
        if self.attention_kind == "mqa" and self.kv_heads != 1:
            raise KvError("MQA requires kv_heads == 1")
        if self.attention_kind in ("gqa", "mqa") and self.query_heads % self.kv_heads:
            raise KvError("query_heads must be divisible by kv_heads")
        if self.attention_kind not in ("mha", "mqa", "gqa") or self.role not in ("key", "value") or \
                self.dtype not in ("f16", "bf16", "f32") or \
                self.rope_state not in ("pre_rope", "post_rope", "not_applicable"):
            raise KvError("unknown enum value in kv shape")
        if self.role == "key" and self.rope_state == "not_applicable":
            raise KvError("key tensors must declare pre_rope or post_rope")
        if self.role == "value" and self.rope_state != "not_applicable":
            raise KvError("value tensors must use not_applicable rope state")

    def validate_block_dim(self, block_dim: int) -> None:
        self.validate()
        if block_dim == 0 or self.head_dim % block_dim:
            raise KvError(f"head_dim {self.head_dim} not divisible by block_dim {block_dim}")

    def vector_count(self) -> int:
        return self.batch * self.layers * self.kv_heads * self.tokens

    def element_count(self) -> int:
        return self.vector_count() * self.head_dim

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "role": self.role, "attention_kind": self.attention_kind,
                "batch": self.batch, "layers": self.layers, "kv_heads": self.kv_heads,
                "query_heads": self.query_heads, "tokens": self.tokens, "head_dim": self.head_dim,
                "dtype": self.dtype, "rope_state": self.rope_state}

    def digest(self) -> str:
        self.validate()
        return json_digest(KV_SHAPE_SCHEMA, self.as_json())


@dataclass(frozen=True)
class KvCacheLayoutV1:
    """kv/layout.rs:19-77: only the canonical contiguous [batch][layer][head][token][dim] order."""
    batch_stride: int
    layer_stride: int
    head_stride: int
    token_stride: int
    dim_stride: int = 1
    order: str = "batch_layer_head_token_dim"
    schema_version: str = KV_LAYOUT_SCHEMA
    shape_schema_version: str = KV_SHAPE_SCHEMA

    @classmethod
    def canonical(cls, shape: KvTensorShapeV1) -> "KvCacheLayoutV1":
        shape.validate()
        token = shape.head_dim
        head = shape.tokens * token
        layer = shape.kv_heads * head
        return cls(shape.layers * layer, layer, head, token)

    def validate_for_shape(self, shape: KvTensorShapeV1) -> None:
        shape.validate()
        if self.schema_version != KV_LAYOUT_SCHEMA:
            raise KvError(f"kv layout schema_version {self.schema_version}, expected {KV_LAYOUT_SCHEMA}")
        if self.shape_schema_version != KV_SHAPE_SCHEMA:
            raise KvError("kv layout shape schema mismatch")
        if self != KvCacheLayoutV1.canonical(shape):
            raise KvError("only canonical contiguous kv layout is supported by the CPU reference codec")

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "shape_schema_version": self.shape_schema_version,
                "order": self.order, "batch_stride": self.batch_stride, "layer_stride": self.layer_stride,
                "head_stride": self.head_stride, "token_stride": self.token_stride, "dim_stride": self.dim_stride}

    def digest(self, shape: KvTensorShapeV1) -> str:
        self.validate_for_shape(shape)
        return json_digest(KV_LAYOUT_SCHEMA, self.as_json())


@dataclass(frozen=True)
class KvPageGeometryV1:
    """kv/layout.rs:79-150."""
    tokens_per_page: int
    head_dim: int
    encoded_block_bytes: int
    vectors_per_block: int = 1
    raw_vector_bytes: int = -1
    schema_version: str = KV_PAGE_GEOMETRY_SCHEMA

    def __post_init__(self):
        if self.raw_vector_bytes < 0:
            object.__setattr__(self, "raw_vector_bytes", self.head_dim * 4)

    def validate_for_shape(self, shape: KvTensorShapeV1) -> None:
        shape.validate()
        if self.schema_version != KV_PAGE_GEOMETRY_SCHEMA:
            raise KvError(f"kv page geometry schema_version {self.schema_version}, expected {KV_PAGE_GEOMETRY_SCHEMA}")
        if self.tokens_per_page == 0 or self.tokens_per_page > shape.tokens:
            raise KvError("tokens_per_page must be in 1..=shape.tokens")
        if self.vectors_per_block != 1:
            raise KvError("CPU reference codec currently supports one vector per block")
        if self.head_dim != shape.head_dim:
            raise KvError("page geometry head_dim must match shape")
        if self.raw_vector_bytes != self.head_dim * 4:
            raise KvError("raw_vector_bytes must equal head_dim * sizeof(f32)")
        if self.encoded_block_bytes == 0:
            raise KvError("encoded_block_bytes must be nonzero")

    def page_count(self, shape: KvTensorShapeV1) -> int:
        self.validate_for_shape(shape)
        return -(-shape.tokens // self.tokens_per_page)

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "tokens_per_page": self.tokens_per_page,
                "vectors_per_block": self.vectors_per_block, "head_dim": self.head_dim,
                "encoded_block_bytes": self.encoded_block_bytes, "raw_vector_bytes": self.raw_vector_bytes}

    def digest(self, shape: KvTensorShapeV1) -> str:
        self.validate_for_shape(shape)
        return json_digest(KV_PAGE_GEOMETRY_SCHEMA, self.as_json())


@dataclass
class KvProtectedPolicyV1:
    """kv/profile.rs:33-77: vectors kept raw."""
    first_tokens_raw: int = 0
    last_tokens_raw: int = 0
    raw_layers: list = field(default_factory=list)
    raw_heads: list = field(default_factory=list)

    def is_protected(self, shape: KvTensorShapeV1, layer: int, head: int, token: int) -> bool:
        return token < self.first_tokens_raw or token + self.last_tokens_raw >= shape.tokens or \
            layer in self.raw_layers or head in self.raw_heads

    def validate_for_shape(self, shape: KvTensorShapeV1) -> None:
        if self.first_tokens_raw > shape.tokens or self.last_tokens_raw > shape.tokens:
            raise KvError("protected token count exceeds shape tokens")
        if any(l >= shape.layers for l in self.raw_layers):
            raise KvError("protected layer outside shape")
        if any(h >= shape.kv_heads for h in self.raw_heads):
            raise KvError("protected head outside shape")

    def as_json(self) -> dict:
        return {"first_tokens_raw": self.first_tokens_raw, "last_tokens_raw": self.last_tokens_raw,
                "raw_layers": list(self.raw_layers), "raw_heads": list(self.raw_heads)}


@dataclass
class KvQualityBudgetV1:
    """kv/profile.rs:95-139."""
    max_logit_mse: float | None = None
    max_attention_tv: float | None = None
    max_topk_disagreement: float | None = None
    max_value_aggregation_mse: float | None = None
    fallback_on_violation: str = "keep_raw"

    def validate(self) -> None:
        for name in ("max_logit_mse", "max_attention_tv", "max_topk_disagreement", "max_value_aggregation_mse"):
            v = getattr(self, name)
            if v is not None and (not math.isfinite(v) or v < 0.0):
                raise KvError(f"{name} must be finite and nonnegative")

    def as_json(self) -> dict:
        return {"max_logit_mse": self.max_logit_mse, "max_attention_tv": self.max_attention_tv,
                "max_topk_disagreement": self.max_topk_disagreement,
                "max_value_aggregation_mse": self.max_value_aggregation_mse,
                "fallback_on_violation": self.fallback_on_violation}


@dataclass
class KvCompressionProfileV1:
    """kv/profile.rs:141-262.  axis_policy: raw | per_token | per_channel | role_aware_kivi_style;
    fallback mode: keep_raw | fail_closed."""
    profile_id: str
    shape_digest: str
    fib_profile: FibQuantProfileV1
    fib_profile_digest: str
    codebook_digest: str
    rotation_digest: str
    role_policy: str
    axis_policy: str
    page_geometry: KvPageGeometryV1
    protected_policy: KvProtectedPolicyV1 = field(default_factory=KvProtectedPolicyV1)
    fallback_mode: str = "keep_raw"
    raw_fallback_available: bool = True
    quality_budget: KvQualityBudgetV1 = field(default_factory=KvQualityBudgetV1)
    calibration_digest: str = "missing:calibration"
    schema_version: str = KV_PROFILE_SCHEMA

    @classmethod
    def from_parts(cls, profile_id: str, shape: KvTensorShapeV1, fib_profile: FibQuantProfileV1,
                   codebook_digest: str, rotation_digest_: str, axis_policy: str,
                   page_geometry: KvPageGeometryV1) -> "KvCompressionProfileV1":
        """profile.rs:160-199; the rotation digest is the caller's (of the matrix in use, see the header)."""
        shape.validate_block_dim(fib_profile.block_dim)
        fib_profile.validate()
        if fib_profile.ambient_dim != shape.head_dim:
            raise KvError("fib profile ambient_dim must equal kv head_dim for CPU reference codec")
        p = cls(profile_id, shape.digest(), fib_profile, fib_profile.digest(), codebook_digest, rotation_digest_,
                shape.role, axis_policy, page_geometry)
        p.validate_for_shape(shape)
        return p

    def validate_for_shape(self, shape: KvTensorShapeV1) -> None:
        if self.schema_version != KV_PROFILE_SCHEMA:
            raise KvError(f"kv profile schema_version {self.schema_version}, expected {KV_PROFILE_SCHEMA}")
        shape.validate_block_dim(self.fib_profile.block_dim)
        if self.shape_digest != shape.digest():
            raise KvError(f"profile digest mismatch: expected {shape.digest()}, actual {self.shape_digest}")
        if self.role_policy != shape.role:
            raise KvError("kv profile role does not match shape role")
        self.fib_profile.validate()
        if self.fib_profile.ambient_dim != shape.head_dim:
            raise KvError("fib profile ambient_dim must equal kv head_dim")
        if self.fib_profile_digest != self.fib_profile.digest():
            raise KvError(f"profile digest mismatch: expected {self.fib_profile.digest()}, "
                          f"actual {self.fib_profile_digest}")
        if not self.rotation_digest:
            raise KvError("kv profile rotation_digest must be nonempty")
        if not self.codebook_digest:
            raise KvError("kv profile codebook_digest must be nonempty")
        self.page_geometry.validate_for_shape(shape)
        self.protected_policy.validate_for_shape(shape)
        self.quality_budget.validate()

    def as_json(self) -> dict:
        return {"schema_version": self.schema_version, "profile_id": self.profile_id,
                "shape_digest": self.shape_digest, "fib_profile": self.fib_profile.as_json(),
                "fib_profile_digest": self.fib_profile_digest, "codebook_digest": self.codebook_digest,
                "rotation_digest": self.rotation_digest, "role_policy": self.role_policy,
                "axis_policy": self.axis_policy, "page_geometry": self.page_geometry.as_json(),
                "protected_policy": self.protected_policy.as_json(),
                "fallback_policy": {"mode": self.fallback_mode,
                                    "raw_fallback_available": self.raw_fallback_available},
                "quality_budget": self.quality_budget.as_json(), "calibration_digest": self.calibration_digest}

    def digest(self, shape: KvTensorShapeV1) -> str:
        self.validate_for_shape(shape)
        return json_digest(KV_PROFILE_SCHEMA, self.as_json())


KV_STRATEGIES = ("raw", "fib_quant_per_token", "fib_quant_per_channel", "role_aware_kivi_style_baseline",
                 "experimental_fib_quant_role_aware")


@dataclass
class KvCompressionPolicyV1:
    """kv/policy.rs:27-66."""
    strategy: str = "raw"
    protected_policy: KvProtectedPolicyV1 = field(default_factory=KvProtectedPolicyV1)
    require_calibration: bool = False
    allow_raw_fallback: bool = True

    @classmethod
    def raw(cls) -> "KvCompressionPolicyV1":
        return cls()

    @classmethod
    def role_aware_baseline(cls) -> "KvCompressionPolicyV1":
        return cls("role_aware_kivi_style_baseline", KvProtectedPolicyV1(0, 1, [], []), False, True)

    def as_json(self) -> dict:
        return {"strategy": self.strategy, "protected_policy": self.protected_policy.as_json(),
                "require_calibration": self.require_calibration, "allow_raw_fallback": self.allow_raw_fallback}


def decide_kv_compression(policy: KvCompressionPolicyV1, shape: KvTensorShapeV1, layer: int, head: int, token: int,
                          has_calibration: bool) -> dict:
    """kv/policy.rs:117-190: the decision for one logical vector as
    ``{"action", "axis_policy", "reasons"}`` (KvCompressionDecisionV1's fields, variants by their serde names)."""
    shape.validate()
    policy.protected_policy.validate_for_shape(shape)
    if layer >= shape.layers or head >= shape.kv_heads or token >= shape.tokens:
        raise KvError("kv policy index outside shape")
    if policy.strategy not in KV_STRATEGIES:
        raise KvError(f"unknown kv compression strategy {policy.strategy}")
    if policy.protected_policy.is_protected(shape, layer, head, token):
        return {"action": "keep_raw", "axis_policy": "raw", "reasons": ["protected_region"]}
    if policy.require_calibration and not has_calibration:
        return {"action": "keep_raw" if policy.allow_raw_fallback else "need_calibration", "axis_policy": "raw",
                "reasons": ["calibration_missing"]}
    role_reason = ["key_role_axis"] if shape.role == "key" else ["value_role_axis"]
    role_axis = "per_channel" if shape.role == "key" else "per_token"
    if policy.strategy == "raw":
        return {"action": "keep_raw", "axis_policy": "raw", "reasons": ["raw_strategy"]}
    if policy.strategy == "fib_quant_per_token":
        return {"action": "compress", "axis_policy": "per_token", "reasons": role_reason}
    if policy.strategy == "fib_quant_per_channel":
        return {"action": "compress", "axis_policy": "per_channel", "reasons": role_reason}
    if policy.strategy == "role_aware_kivi_style_baseline":
        return {"action": "compress", "axis_policy": role_axis, "reasons": role_reason}
    return {"action": "compress", "axis_policy": role_axis, "reasons": ["experimental_role_aware"]}


def _norm_format_len(fmt: str) -> int:
    return 2 if fmt == "fp16_paper" else 4


@dataclass
class KvEncodedBlockV1:
    """kv/block.rs:16-139.  `record` holds a coded vector as the wire keeps it (norm payload, then the packed
    indices); `values` the raw f32 vector of a fallback block."""
    block_id: int
    batch: int
    layer: int
    kv_head: int
    token: int
    fixed_size_bytes: int
    raw_fallback: bool
    reason: str
    record: bytes | None = None
    values: np.ndarray | None = None
    vector_count: int = 1
    schema_version: str = KV_BLOCK_SCHEMA

    def encoding_json(self, ctx: "_CodeContext") -> dict:
        if self.raw_fallback:
            return {"raw_f32": {"values": [F32(t) for t in self.values]}}
        n = ctx.norm_len
        return {"fib_quant": {"code": {
            "schema_version": CODE_SCHEMA, "profile_digest": ctx.fib_profile_digest,
            "codebook_digest": ctx.codebook_digest, "rotation_digest": ctx.rotation_digest,
            "ambient_dim": ctx.fib_profile.ambient_dim, "block_dim": ctx.fib_profile.block_dim,
            "norm_format": ctx.fib_profile.norm_format, "norm_payload": list(self.record[:n]),
            "wire_index_bits": ctx.fib_profile.wire_index_bits, "block_count": ctx.fib_profile.block_count(),
            "indices": list(self.record[n:])}}}

    def as_json(self, ctx: "_CodeContext") -> dict:
        return {"schema_version": self.schema_version, "block_id": self.block_id, "batch": self.batch,
                "layer": self.layer, "kv_head": self.kv_head, "token": self.token,
                "vector_count": self.vector_count, "fixed_size_bytes": self.fixed_size_bytes,
                "raw_fallback": self.raw_fallback, "reason": self.reason, "encoding": self.encoding_json(ctx)}

    def validate(self, head_dim: int, ctx: "_CodeContext") -> None:
        if self.schema_version != KV_BLOCK_SCHEMA:
            raise KvError(f"kv block schema_version {self.schema_version}, expected {KV_BLOCK_SCHEMA}")
        if self.vector_count != 1:
            raise KvError("kv block vector_count must be 1")
        if self.fixed_size_bytes == 0:
            raise KvError("kv block fixed_size_bytes must be nonzero")
        if self.values is not None:
            if not self.raw_fallback:
                raise KvError("raw block must set raw_fallback")
            if len(self.values) != head_dim:
                raise KvError("raw kv block head_dim mismatch")
            if not np.isfinite(self.values).all():
                raise KvError("raw kv block contains non-finite value")
        else:
            if self.raw_fallback:
                raise KvError("compressed block cannot set raw_fallback")
            if ctx.fib_profile.ambient_dim != head_dim:
                raise KvError("fib kv block ambient_dim mismatch")

    def digest(self, head_dim: int, ctx: "_CodeContext") -> str:
        self.validate(head_dim, ctx)
        return json_digest(KV_BLOCK_SCHEMA, self.as_json(ctx))


@dataclass
class _CodeContext:
    """What every fib code of a tensor repeats (codec.rs:490-502)."""
    fib_profile: FibQuantProfileV1
    fib_profile_digest: str
    codebook_digest: str
    rotation_digest: str

    @property
    def norm_len(self) -> int:
        return _norm_format_len(self.fib_profile.norm_format)


@dataclass
class KvEncodedPageV1:
    """kv/page.rs:14-160."""
    page_id: int
    token_start: int
    token_count: int
    source_tensor_digest: str
    profile_digest: str
    shape_digest: str
    page_geometry: KvPageGeometryV1
    encoded_blocks: list
    raw_fallback_blocks: int
    page_digest: str = ""
    shape_schema_version: str = KV_SHAPE_SCHEMA
    schema_version: str = KV_PAGE_SCHEMA

    @classmethod
    def new(cls, page_id, token_start, token_count, source_tensor_digest, profile_digest, shape, page_geometry,
            encoded_blocks, ctx) -> "KvEncodedPageV1":
        page = cls(page_id, token_start, token_count, source_tensor_digest, profile_digest, shape.digest(),
                   page_geometry, list(encoded_blocks), sum(1 for b in encoded_blocks if b.raw_fallback))
        page.page_digest = page.compute_digest(shape, ctx)
        return page

    def compute_digest(self, shape: KvTensorShapeV1, ctx: _CodeContext) -> str:
        self.page_geometry.validate_for_shape(shape)
        return json_digest(KV_PAGE_SCHEMA, {
            "schema_version": self.schema_version, "page_id": self.page_id, "token_start": self.token_start,
            "token_count": self.token_count, "source_tensor_digest": self.source_tensor_digest,
            "profile_digest": self.profile_digest, "shape_digest": self.shape_digest,
            "shape_schema_version": self.shape_schema_version, "page_geometry": self.page_geometry.as_json(),
            "encoded_blocks": [b.as_json(ctx) for b in self.encoded_blocks],
            "raw_fallback_blocks": self.raw_fallback_blocks})

    def validate(self, shape: KvTensorShapeV1, ctx: _CodeContext) -> None:
        if self.schema_version != KV_PAGE_SCHEMA:
            raise KvError(f"kv page schema_version {self.schema_version}, expected {KV_PAGE_SCHEMA}")
        shape.validate()
        if self.shape_schema_version != KV_SHAPE_SCHEMA or self.shape_digest != shape.digest():
            raise KvError("kv page shape digest mismatch")
        self.page_geometry.validate_for_shape(shape)
        if self.token_count == 0 or self.token_start >= shape.tokens:
            raise KvError("invalid kv page token span")
        if self.token_start + self.token_count > shape.tokens:
            raise KvError("kv page token span exceeds shape tokens")
        if self.token_count > self.page_geometry.tokens_per_page:
            raise KvError("kv page token_count exceeds geometry")
        if self.raw_fallback_blocks != sum(1 for b in self.encoded_blocks if b.raw_fallback):
            raise KvError("kv page raw fallback count mismatch")
        for idx, block in enumerate(self.encoded_blocks):
            block.validate(shape.head_dim, ctx)
            if block.block_id != idx:
                raise KvError("kv page block ids must be contiguous")
            if not self.token_start <= block.token < self.token_start + self.token_count:
                raise KvError("kv page block token outside page span")
        if self.page_digest != self.compute_digest(shape, ctx):
            raise KvError("kv page digest mismatch")


@dataclass
class KvEncodedTensorV1:
    """kv/codec.rs:18-25; `receipt` is the KvCompressionReceiptV1 as a dict in field order (kv/receipt.rs:19-33)."""
    shape: KvTensorShapeV1
    layout: KvCacheLayoutV1
    profile: KvCompressionProfileV1
    pages: list
    receipt: dict

    def context(self) -> _CodeContext:
        return _CodeContext(self.profile.fib_profile, self.profile.fib_profile_digest, self.profile.codebook_digest,
                            self.profile.rotation_digest)


def _gpu_profile(profile: KvCompressionProfileV1, rotation, codebook):
    from . import _lib as L
    from .profiles import FibProfile
    fp = profile.fib_profile
    cb = np.ascontiguousarray(codebook, np.float32).reshape(fp.codebook_size, fp.block_dim)
    return FibProfile(fp.ambient_dim, rotation, cb, numerics=L.FIB_NUMERICS_SINGLE)


def encode_kv_tensor(shape: KvTensorShapeV1, layout: KvCacheLayoutV1, profile: KvCompressionProfileV1, values,
                     rotation, codebook, gpu_profile=None, recorded_unix_seconds: int | None = None
                     ) -> KvEncodedTensorV1:
    """`encode_kv_tensor` (kv/codec.rs:34-147) with every vector's code from one GPU launch.

    ``rotation`` (dim x dim f64) and ``codebook`` (N x k f32) are the tables the profile's digests describe.
    Vectors the reference's encoder refuses (zero norm, norm outside fp16) become raw blocks under the
    keep-raw fallback policy with the reference's reason text, or raise under fail-closed."""
    shape.validate()
    layout.validate_for_shape(shape)
    profile.validate_for_shape(shape)
    x = np.ascontiguousarray(values, np.float32).reshape(-1)
    if x.size != shape.element_count():
        raise KvError(f"kv input has {x.size} values, expected {shape.element_count()}")
    if not np.isfinite(x).all():
        raise KvError("kv input contains non-finite value")
    d, T = shape.head_dim, shape.tokens
    x = x.reshape(-1, d)
    source_digest = kv_tensor_digest(x)
    profile_digest = profile.digest(shape)
    ctx = _CodeContext(profile.fib_profile, profile.fib_profile_digest, profile.codebook_digest,
                       profile.rotation_digest)
    geo = profile.page_geometry

    # which vectors are coded, which stay raw and why (kv/codec.rs:73-106, 236-284)
    n_vec = x.shape[0]
    b_i, l_i, h_i, t_i = np.unravel_index(np.arange(n_vec), (shape.batch, shape.layers, shape.kv_heads, T))
    pol = profile.protected_policy
    protected = (t_i < pol.first_tokens_raw) | (t_i + pol.last_tokens_raw >= T) | \
        np.isin(l_i, pol.raw_layers) | np.isin(h_i, pol.raw_heads)
    reason = np.full(n_vec, "fib_quant_per_token", dtype=object)
    reason[protected] = "protected_region"
    raw = protected.copy()
    keep_raw = profile.fallback_mode == "keep_raw"
    if profile.axis_policy == "raw":
        reason[~protected] = "raw_axis_policy"
        raw[:] = True
    elif profile.axis_policy in ("per_channel", "role_aware_kivi_style"):
        if not keep_raw:
            raise KvError("dependency unsupported: CPU reference codec supports per-token FibQuant compression only")
        reason[~protected] = "unsupported_axis_raw_fallback"
        raw[:] = True
    elif profile.axis_policy != "per_token":
        raise KvError(f"unknown axis policy {profile.axis_policy}")
    records = None
    if not raw.all():
        # One launch over every vector; the ones the policy keeps raw ride along as a codable stand-in.
        # The encoder's answer comes back in the records: a refused vector's record is all zero bytes
        # (include/provekv_b200.h, pkv_fib_encode_batches_compact), and the call's status names the first one.
        from . import _lib as L
        from .profiles import encode_batches_compact
        xg = x
        if raw.any():
            xg = x.copy()
            xg[raw] = 0.0
            xg[raw, 0] = 1.0
        prof = gpu_profile or _gpu_profile(profile, rotation, codebook)
        rec = prof.record_bytes
        wire = np.zeros(L.FB2_HEADER_BYTES + n_vec * rec, np.uint8)
        try:
            encode_batches_compact(prof, xg.ctypes.data, 1, n_vec, wire.ctypes.data, wire.size)
        except L.PkvError as e:
            if e.status < 16:        # not a per-vector status
                raise
        records = wire[L.FB2_HEADER_BYTES:].reshape(n_vec, rec)
        norm_len = _norm_format_len(profile.fib_profile.norm_format)
        refused = ~raw & ~records[:, :norm_len].any(axis=1)
        # the reference's two refusals (input is finite here): a vector of zeros has norm zero, anything else
        # the encoder refuses has a norm its wire format cannot hold (codec.rs:603, :1003-1017)
        zero = refused & ~x.any(axis=1)
        texts = ("zero norm vector is not valid on the normal FibQuant encode path",
                 "corrupt payload: norm cannot be represented as finite positive "
                 + ("fp16" if norm_len == 2 else "f32"))
        if refused.any() and not keep_raw:
            # fail-closed: the reference stops at the first refused vector of its page -> batch -> layer -> head
            # -> token walk (codec.rs:72-101); a flat index is ((batch, layer, head), token)
            idx = np.flatnonzero(refused)
            first = idx[np.lexsort((idx, (idx % T) // geo.tokens_per_page))[0]]
            raise KvError(texts[0] if zero[first] else texts[1])
        for text, mask in ((texts[0], zero), (texts[1], refused & ~zero)):
            if mask.any():
                reason[mask] = "encode_fallback:" + text
                raw |= mask

    pages, compressed, raw_blocks, reasons = [], 0, 0, []
    for page_id in range(geo.page_count(shape)):
        t0 = page_id * geo.tokens_per_page
        t1 = min(t0 + geo.tokens_per_page, T)
        blocks = []
        for b in range(shape.batch):
            for layer in range(shape.layers):
                for head in range(shape.kv_heads):
                    base = ((b * shape.layers + layer) * shape.kv_heads + head) * T
                    for tok in range(t0, t1):
                        v = base + tok
                        if raw[v]:
                            blk = KvEncodedBlockV1(len(blocks), b, layer, head, tok, geo.encoded_block_bytes, True,
                                                   str(reason[v]), values=x[v].copy())
                            raw_blocks += 1
                            if blk.reason not in reasons:
                                reasons.append(blk.reason)
                        else:
                            blk = KvEncodedBlockV1(len(blocks), b, layer, head, tok, geo.encoded_block_bytes, False,
                                                   "fib_quant_per_token", record=records[v].tobytes())
                            compressed += 1
                        blocks.append(blk)
        pages.append(KvEncodedPageV1.new(page_id, t0, t1 - t0, source_digest, profile_digest, shape, geo, blocks, ctx))
    receipt = {"schema_version": KV_RECEIPT_SCHEMA, "operation_kind": "compress", "source_digest": source_digest,
               "profile_digest": profile_digest, "shape_digest": shape.digest(),
               "page_digests": [p.page_digest for p in pages], "codebook_digest": profile.codebook_digest,
               "rotation_digest": profile.rotation_digest, "encoded_pages": len(pages),
               "compressed_blocks": compressed, "raw_fallback_blocks": raw_blocks, "fallback_reasons": reasons,
               "recorded_unix_seconds": int(time.time()) if recorded_unix_seconds is None else recorded_unix_seconds}
    return KvEncodedTensorV1(shape, layout, profile, pages, receipt)


def decode_kv_pages(encoded: KvEncodedTensorV1, rotation, codebook, gpu_profile=None,
                    recorded_unix_seconds: int | None = None):
    """`decode_kv_pages` (kv/codec.rs:149-218): ``(values [batch, layers, kv_heads, tokens, head_dim] f32,
    KvDecodeReceiptV1 as a dict)``; every coded block goes through one launch of the binary64 decoder."""
    shape, profile = encoded.shape, encoded.profile
    shape.validate()
    encoded.layout.validate_for_shape(shape)
    profile.validate_for_shape(shape)
    r = encoded.receipt
    if r.get("schema_version") != KV_RECEIPT_SCHEMA or r.get("operation_kind") != "compress":
        raise KvError("invalid kv compression receipt")
    profile_digest = profile.digest(shape)
    if r["profile_digest"] != profile_digest:
        raise KvError(f"profile digest mismatch: expected {profile_digest}, actual {r['profile_digest']}")
    ctx = encoded.context()
    d, T = shape.head_dim, shape.tokens
    out = np.zeros((shape.vector_count(), d), np.float32)
    # blocks in the order the reference walks them; where two name the same vector the later one stays, as in
    # its copy_from_slice per block
    at, raw_vals, coded_rec, is_raw, raw_blocks, page_digests = [], [], [], [], 0, []
    for page in encoded.pages:
        page.validate(shape, ctx)
        if page.profile_digest != r["profile_digest"]:
            raise KvError(f"profile digest mismatch: expected {r['profile_digest']}, actual {page.profile_digest}")
        page_digests.append(page.page_digest)
        for blk in page.encoded_blocks:
            if blk.batch >= shape.batch or blk.layer >= shape.layers or blk.kv_head >= shape.kv_heads or \
                    blk.token >= T:
                raise KvError("kv block index outside shape")
            at.append(((blk.batch * shape.layers + blk.layer) * shape.kv_heads + blk.kv_head) * T + blk.token)
            is_raw.append(blk.raw_fallback)
            if blk.raw_fallback:
                raw_blocks += 1
                raw_vals.append(blk.values)
            else:
                coded_rec.append(blk.record)
    if at:
        is_raw = np.asarray(is_raw, bool)
        vals = np.empty((len(at), d), np.float32)
        if raw_vals:
            vals[is_raw] = np.asarray(raw_vals, np.float32).reshape(-1, d)
        if coded_rec:
            prof = gpu_profile or _gpu_profile(profile, rotation, codebook)
            vals[~is_raw] = prof.decode_exact(b"".join(coded_rec))
        at = np.asarray(at)
        last = np.zeros(out.shape[0], np.int64) - 1
        np.maximum.at(last, at, np.arange(at.size))   # the last block naming each vector
        keep = last[last >= 0]
        out[at[keep]] = vals[keep]
    receipt = {"schema_version": KV_RECEIPT_SCHEMA, "operation_kind": "decode",
               "decoded_digest": kv_tensor_digest(out), "profile_digest": r["profile_digest"],
               "shape_digest": shape.digest(), "page_digests": page_digests,
               "codebook_digest": profile.codebook_digest, "rotation_digest": profile.rotation_digest,
               "decoded_pages": len(encoded.pages), "raw_fallback_blocks": raw_blocks,
               "recorded_unix_seconds": int(time.time()) if recorded_unix_seconds is None else recorded_unix_seconds}
    return out.reshape(shape.batch, shape.layers, shape.kv_heads, T, d), receipt
