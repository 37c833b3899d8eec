"""Manifests and receipts: the JSON text every digest is taken over, and the validation rules.

The expected strings are written out by hand from the struct declarations (field order of
proveKV/src/manifest.rs:23-46,124-148, proveKV/src/receipt.rs:18-38,148-158,217-241 and
proveKV/src/policy.rs:117-127,216-223,292-298); the rule cases follow the reference's unit tests
(manifest.rs:268-365, receipt.rs:305-380, policy.rs:352-430).
"""
import json

import numpy as np

import blake3
import pytest

from provekv_b200 import manifest as M
from provekv_b200 import records as R
from provekv_b200.codec import (FibConfig, InvalidManifest, InvalidPolicy, InvalidReceipt, InvalidShape,
                                TurboConfig, turbo_batched_codec_id)

POLICY_TEXT = ('{"shared_codec":"fib_k4_n32_batched","shell_codec":"turbo_4bit_batched",'
               '"fib_config":{"k":4,"n":32,"training_samples":2048,"lloyd_restarts":4,"lloyd_iterations":8},'
               '"turbo_config":{"bits":4,"projections":32,"radii_compression":"Lossless"}}')
SHAPE_TEXT = '{"attention_type":"gqa","num_layers":4,"num_heads":8,"num_kv_heads":2,"head_dim":64,"hidden_size":512}'


def _shape():
    return R.KvTensorShape("GQA", 4, 8, 2, 64, 512)


def _hash(text: str) -> str:
    return blake3.blake3(text.encode()).hexdigest()


@pytest.mark.parametrize("value,text", [
    (0.0, "0.0"), (-0.0, "-0.0"), (50.0, "50.0"), (1.0 / 3.0, "0.3333333333333333"), (58.14, "58.14"),
    (1e-5, "0.00001"), (1e-6, "1e-6"), (1.5e-7, "1.5e-7"), (1e15, "1000000000000000.0"), (1e16, "1e16"),
    (1.2345678901234568e17, "1.2345678901234568e17"), (1e21, "1e21"), (5e-324, "5e-324"),
    (9007199254740992.0, "9007199254740992.0"), (0.001234, "0.001234"), (-12.5, "-12.5"),
    (float("nan"), "null"), (float("inf"), "null"),
])
def test_binary64_text_follows_the_shortest_round_trip_layout(value, text):
    assert R.serde_f64(value) == text
    if text != "null":
        assert float(text) == value


def test_serde_text_escapes_and_order():
    assert R.serde_text({"b": 1, "a": [True, None, "q\"\\\n\t\x01é"]}) == \
        '{"b":1,"a":[true,null,"q\\"\\\\\\n\\t\\u0001é"]}'
    assert R.serde_text({"n": 2 ** 64 - 1, "i": -5}) == '{"n":18446744073709551615,"i":-5}'
    with pytest.raises(TypeError):
        R.serde_text({"x": object()})


def test_policy_text_and_rules():
    p = R.CompressionPolicy.default_two_tier()
    p.validate()
    assert R.serde_text(p.as_json()) == POLICY_TEXT
    lossy = R.CompressionPolicy.default_two_tier_lossy()
    lossy.validate()
    assert '"shell_codec":"turbo_4bit_batched_lossy"' in R.serde_text(lossy.as_json())
    assert '"radii_compression":"Lossy"' in R.serde_text(lossy.as_json())
    assert R.CompressionPolicy.from_json(json.loads(POLICY_TEXT)) == p
    # a record written before `radii_compression` existed reads as lossless
    assert TurboConfig.from_json({"bits": 8, "projections": 32}) == TurboConfig(8, 32, False)
    for bad in (FibConfig(k=0), FibConfig(n=1), FibConfig(k=257), FibConfig(n=1_048_577),
                FibConfig(training_samples=0), FibConfig(lloyd_restarts=0), FibConfig(lloyd_iterations=0)):
        with pytest.raises(InvalidPolicy):
            bad.validate()
    for bad in (TurboConfig(bits=1), TurboConfig(bits=17), TurboConfig(projections=0)):
        with pytest.raises(InvalidPolicy):
            bad.validate()
    assert TurboConfig(4, 32, False).expected_compression_ratio() == 8.0
    assert TurboConfig(4, 32, True).expected_compression_ratio() == 32.0
    with pytest.raises(InvalidPolicy, match=r'shared_codec must be one of \["fib_k4_n32", "fib_k4_n32_batched", '
                                            r'"exact_f32_fallback"\], got \'turbo_8bit\''):
        R.CompressionPolicy(shared_codec="turbo_8bit").validate()
    with pytest.raises(InvalidPolicy):
        R.CompressionPolicy(shell_codec="turbo_1bit_batched").validate()
    ids = R.allowed_shell_codecs()
    assert len(ids) == 4 + 14 * 2 and ids[:4] == ["turbo_8bit", "turbo_8bit_batched", "turbo_8bit_batched_lossy",
                                                   "exact_f32_fallback"]
    for bits in range(2, 17):
        for lossy_radii in (False, True):
            R.CompressionPolicy(shell_codec=turbo_batched_codec_id(bits, lossy_radii),
                                turbo_config=TurboConfig(bits, 32, lossy_radii)).validate()


def test_shape_rules():
    _shape().validate()
    R.KvTensorShape("mha", 2, 8, 8, 64, 512).validate()
    R.KvTensorShape("MQA", 2, 8, 1, 64, 512).validate()
    for bad in (R.KvTensorShape("gqa", 0, 8, 2, 64, 512), R.KvTensorShape("gqa", 4, 8, 8, 64, 512),
                R.KvTensorShape("mha", 4, 8, 2, 64, 512), R.KvTensorShape("mqa", 4, 8, 2, 64, 512),
                R.KvTensorShape("gqa", 4, 8, 2, 64, 500), R.KvTensorShape("gqa", 4, 8, 2, 0, 512),
                R.KvTensorShape("sliding", 4, 8, 2, 64, 512)):
        with pytest.raises(InvalidShape):
            bad.validate()
    assert R.serde_text(_shape().as_json()) == SHAPE_TEXT


def test_pool_manifest_text_digest_and_rules():
    m = R.PoolManifest.new("abc", _shape(), R.CompressionPolicy.default_two_tier(), 64, 4, 10_000, 500_000, 99, 1700000000)
    text = ('{"schema_version":"pool_manifest_v1","pool_id":"abc","shape":' + SHAPE_TEXT + ',"policy":' + POLICY_TEXT +
            ',"num_shared_tokens":64,"num_layers":4,"pool_size_bytes":10000,"shared_codec":"fib_k4_n32_batched",'
            '"compression_ratio":50.0,"built_at_unix":1700000000,"build_seed":99}')
    assert m.to_json() == text and m.digest() == _hash(text)
    assert R.PoolManifest.from_json(json.loads(text)) == m
    assert R.PoolManifest.new("abc", _shape(), R.CompressionPolicy(), 0, 4, 0, 0, 1, 0).compression_ratio == 0.0
    third = R.PoolManifest.new("abc", _shape(), R.CompressionPolicy(), 1, 4, 3, 1, 1, 0)
    assert '"compression_ratio":0.3333333333333333,' in third.to_json()
    with pytest.raises(InvalidManifest, match="pool_id is empty"):
        R.PoolManifest.new("", _shape(), R.CompressionPolicy(), 64, 4, 1, 1, 1, 0)
    with pytest.raises(InvalidShape):
        R.PoolManifest.new("abc", R.KvTensorShape("gqa", 4, 8, 8, 64, 512), R.CompressionPolicy(), 64, 4, 1, 1, 1, 0)
    m.schema_version = "pool_manifest_v0"
    with pytest.raises(InvalidManifest, match="expected schema pool_manifest_v1, got pool_manifest_v0"):
        m.validate()


@pytest.mark.parametrize("bits,lossy", [(4, False), (4, True), (8, False), (8, True)])
def test_shell_manifest_codec_follows_the_turbo_configuration(bits, lossy):
    codec = turbo_batched_codec_id(bits, lossy)
    m = R.ShellManifest.new("agent_0", "00" * 16, 0, 24, 0, codec, 42, 0, 64, 32, TurboConfig(bits, 32, lossy))
    assert m.shell_codec == f"turbo_{bits}bit_batched" + ("_lossy" if lossy else "")
    m.validate()
    text = ('{"schema_version":"shell_manifest_v1","agent_id":"agent_0","pool_digest":"' + "00" * 16 + '",'
            '"num_unique_tokens":0,"num_unique_layers":24,"shell_size_bytes":0,"shell_codec":"' + codec + '",'
            '"materialized_at_unix":0,"materialize_seed":42,"head_dim":64,"num_kv_heads":32,'
            '"turbo_config":{"bits":%d,"projections":32,"radii_compression":"%s"},"component_kinds":[]}'
            % (bits, "Lossy" if lossy else "Lossless"))
    assert m.to_json() == text and m.digest() == _hash(text)
    assert R.ShellManifest.from_json(json.loads(text)) == m
    m.component_kinds = ["KeyValue", {"RuntimeSpecific": "ssm_state"}]
    assert m.to_json().endswith(',"component_kinds":["KeyValue",{"RuntimeSpecific":"ssm_state"}]}')


def test_shell_manifest_refuses_a_codec_that_disagrees_with_its_configuration():
    with pytest.raises(InvalidManifest, match=r"shell_codec 'turbo_8bit_batched' does not match turbo_config "
                                              r"\(bits=4, lossy=false\); expected 'turbo_4bit_batched'"):
        R.ShellManifest.new("agent_0", "00" * 16, 0, 24, 0, "turbo_8bit_batched", 42, 0, 64, 32, TurboConfig(4, 32))
    m = R.ShellManifest.new("agent_0", "00" * 16, 0, 24, 0, "turbo_4bit_batched", 42, 0, 64, 32, TurboConfig(4, 32))
    m.shell_codec = "turbo_8bit"          # a record read back from disk that lies about its codec
    with pytest.raises(InvalidManifest, match="does not match"):
        m.validate()
    for kw in ({"agent_id": ""}, {"pool_digest": ""}):
        args = {"agent_id": "a", "pool_digest": "p"} | kw
        with pytest.raises(InvalidManifest, match="is empty"):
            R.ShellManifest.new(args["agent_id"], args["pool_digest"], 0, 1, 0, "turbo_4bit_batched", 1, 0, 64, 2,
                                TurboConfig(4, 32))


def test_pool_build_receipt_text_backend_and_rules():
    r = R.PoolBuildReceipt.new("abc123", ["layer0_digest", "layer1_digest"], "codebook_digest", "rotation_digest",
                               100, 42, 10_000, 500_000, R.CompressionPolicy.default_two_tier(), 42, 1700000001)
    r.validate()
    assert r.backend == "cpu" and r.compression_ratio == 50.0
    text = ('{"schema_version":"pool_build_receipt_v1","pool_digest":"abc123",'
            '"layer_digests":["layer0_digest","layer1_digest"],"codebook_digest":"codebook_digest",'
            '"rotation_digest":"rotation_digest","total_tokens":100,"fib_build_ms":42,"pool_size_bytes":10000,'
            '"raw_size_bytes":500000,"compression_ratio":50.0,"policy_snapshot":' + POLICY_TEXT +
            ',"seeded_with":42,"built_at_unix":1700000001,"backend":"%s"}')
    assert r.to_json() == text % "cpu" and r.digest() == _hash(text % "cpu")
    assert r.with_backend("gpu") is r and r.to_json() == text % "gpu" and r.digest() == _hash(text % "gpu")
    back = R.PoolBuildReceipt.from_json(json.loads(r.to_json()))
    assert back == r
    legacy = json.loads(text % "cpu")
    del legacy["backend"]               # written before the field existed
    assert R.PoolBuildReceipt.from_json(legacy).backend == "cpu"
    for name, message in (("pool_digest", "pool_digest is empty"), ("codebook_digest", "codebook_digest is empty"),
                          ("rotation_digest", "rotation_digest is empty")):
        bad = R.PoolBuildReceipt.from_json(json.loads(r.to_json()))
        setattr(bad, name, "")
        with pytest.raises(InvalidReceipt, match=message):
            bad.validate()


def test_shell_and_injection_receipts():
    r = R.ShellMaterializeReceipt.new("agent_1", "pool_abc", "shell_xyz", 50, 5_000, 10, 1700000002)
    r.validate()
    text = ('{"schema_version":"shell_materialize_receipt_v1","agent_id":"agent_1","pool_digest":"pool_abc",'
            '"shell_digest":"shell_xyz","num_unique_tokens":50,"shell_size_bytes":5000,"materialize_ms":10,'
            '"materialized_at_unix":1700000002}')
    assert r.to_json() == text and r.digest() == _hash(text)
    assert R.ShellMaterializeReceipt.from_json(json.loads(text)) == r
    traces = [R.BlockInjectionTrace(0, "pool", "abc", 0), R.BlockInjectionTrace(0, "shell", "def", 1)]
    i = R.InjectionReceipt.new("agent_1", "pool_abc", "shell_xyz", 2, traces, 1700000003)
    i.validate()
    assert i.blocks_injected == 2
    text = ('{"schema_version":"injection_receipt_v1","agent_id":"agent_1","pool_digest":"pool_abc",'
            '"shell_digest":"shell_xyz","blocks_injected":2,"block_traces":['
            '{"layer":0,"source":"pool","source_digest":"abc","target_position":0},'
            '{"layer":0,"source":"shell","source_digest":"def","target_position":1}],"injected_at_unix":1700000003}')
    assert i.to_json() == text and i.digest() == _hash(text)
    assert R.InjectionReceipt.from_json(json.loads(text)) == i
    for rec, cls in ((r, R.ShellMaterializeReceipt), (i, R.InjectionReceipt)):
        for name in ("agent_id", "pool_digest", "shell_digest"):
            bad = cls.from_json(json.loads(rec.to_json()))
            setattr(bad, name, "")
            with pytest.raises(InvalidReceipt, match=f"{name} is empty"):
                bad.validate()


def test_shell_digest_and_injection_trace_order():
    """shell.rs:158-161,322-337: the digest of an agent's shell; an agent without tokens of its own hashes
    a fixed text.  The injection trace lists, per layer, the pool block at token 0 and then the shell
    block behind the shared prefix."""
    assert M.shell_digest("a7", "pool9", [], 5) == _hash("empty_shell:a7:pool9")
    text = '{"agent_id":"a7","layer_digests":["l0","l1"],"pool_digest":"pool9","seed":5}'
    assert M.shell_digest("a7", "pool9", ["l0", "l1"], 5) == _hash(text)
    pm = R.PoolManifest.new("pool9", R.KvTensorShape("gqa", 2, 8, 2, 64, 512), R.CompressionPolicy(), 800, 2, 10, 100, 5, 0)
    sm = R.ShellManifest.new("a7", "pool9", 100, 2, 10, "turbo_4bit_batched", 5, 0, 64, 2, TurboConfig())
    shell = M.AgentShell("a7", sm, [M.ShellLayer(0, [], [], "s0"), M.ShellLayer(1, [], [], "s1")], "pool9")
    rec = M.injection_receipt("a7", pm, ["p0", "p1"], shell, "sd", 7)
    assert [(t.layer, t.source, t.source_digest, t.target_position) for t in rec.block_traces] == \
        [(0, "pool", "p0", 0), (0, "shell", "s0", 800), (1, "pool", "p1", 0), (1, "shell", "s1", 800)]
    assert rec.blocks_injected == 4 and rec.injected_at_unix == 7


def test_binary32_numbers_print_with_their_own_shortest_digits():
    """serde_json prints an f32 field from its binary32 value (ryu's f32 layout: plain digits for decimal
    exponents in (-6, 13], scientific outside), not from the value widened to f64."""
    from provekv_b200.records import F32, serde_f32
    cases = {1.0: "1.0", 0.1: "0.1", -0.0: "-0.0", 1.5e-7: "1.5e-7", 1e-5: "0.00001", 1e-6: "0.000001",
             1e-7: "1e-7", 123456789.0: "123456790.0", 1e12: "1000000000000.0", 1e13: "1e13",
             16777216.0: "16777216.0", 3.4028235e38: "3.4028235e38", 1.17549435e-38: "1.1754944e-38",
             1e-45: "1e-45", 1.0 / 3.0: "0.33333334", 9999999.0: "9999999.0"}
    for v, text in cases.items():
        assert serde_f32(v) == text, (v, serde_f32(v), text)
    assert R.serde_text({"a": [F32(0.1), float(np.float32(0.1))]}) == '{"a":[0.1,0.10000000149011612]}'
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 0x7F800000, 4000, dtype=np.uint32) | (rng.integers(0, 2, 4000, dtype=np.uint32) << 31)
    for f in bits.view(np.float32):
        t = serde_f32(float(f))
        assert np.float32(t) == f                                   # round trip
        digits = t.replace("-", "").replace(".", "").split("e")[0].strip("0")
        assert len(digits) <= 9
