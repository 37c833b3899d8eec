"""fib-quant's KV page contracts (fib-quant/src/kv/*.rs): digests against strings written out by hand,
the validation rules, and -- on the GPU -- every block's code against the oracle's single-vector encoder
and the decoded tensor against its binary64 decoder."""
import json
import struct

import blake3
import numpy as np
import pytest

from provekv_b200 import kv_pages as K


def _tagged(domain: str, text: str) -> str:
    return "blake3:" + blake3.blake3(domain.encode() + b"\x00" + text.encode()).hexdigest()


def _shape(role="key", tokens=10, batch=1, layers=2, heads=2, dim=64):
    return K.KvTensorShapeV1(role, "gqa", batch, layers, heads, 8, tokens, dim, "f32",
                             "post_rope" if role == "key" else "not_applicable")


def test_domain_tagged_digests_of_shape_layout_and_geometry():
    s = _shape()
    text = ('{"schema_version":"fib_quant_kv_tensor_shape_v1","role":"key","attention_kind":"gqa","batch":1,'
            '"layers":2,"kv_heads":2,"query_heads":8,"tokens":10,"head_dim":64,"dtype":"f32","rope_state":"post_rope"}')
    assert K.serde_text(s.as_json()) == text and s.digest() == _tagged("fib_quant_kv_tensor_shape_v1", text)
    lay = K.KvCacheLayoutV1.canonical(s)
    assert (lay.batch_stride, lay.layer_stride, lay.head_stride, lay.token_stride, lay.dim_stride) == \
        (2 * 2 * 10 * 64, 2 * 10 * 64, 10 * 64, 64, 1)
    text = ('{"schema_version":"fib_quant_kv_cache_layout_v1","shape_schema_version":"fib_quant_kv_tensor_shape_v1",'
            '"order":"batch_layer_head_token_dim","batch_stride":2560,"layer_stride":1280,"head_stride":640,'
            '"token_stride":64,"dim_stride":1}')
    assert lay.digest(s) == _tagged("fib_quant_kv_cache_layout_v1", text)
    geo = K.KvPageGeometryV1(4, 64, 12)
    text = ('{"schema_version":"fib_quant_kv_page_geometry_v1","tokens_per_page":4,"vectors_per_block":1,'
            '"head_dim":64,"encoded_block_bytes":12,"raw_vector_bytes":256}')
    assert geo.digest(s) == _tagged("fib_quant_kv_page_geometry_v1", text) and geo.page_count(s) == 3
    v = np.array([1.5, -2.0, 0.25], np.float32)
    want = "blake3:" + blake3.blake3(b"fib_quant_kv_tensor_f32_v1\x00" + struct.pack("<Q", 3) + v.tobytes()).hexdigest()
    assert K.kv_tensor_digest(v) == want
    with pytest.raises(K.KvError):
        K.kv_tensor_digest(np.array([np.inf], np.float32))
    m = np.array([[1.0, 0.0], [0.0, -1.0]])
    text = ('{"rotation_schema":"fib_rotation_v1","algorithm_version":"qr-gaussian-chacha8-sign-corrected-v1",'
            '"dim":2,"seed":9,"matrix":[1.0,0.0,0.0,-1.0]}')
    assert K.rotation_digest(2, 9, m) == _tagged("fib_rotation_v1", text)


def test_shape_layout_geometry_rules():
    _shape().validate()
    _shape("value").validate()
    bad = [K.KvTensorShapeV1("key", "gqa", 1, 2, 2, 8, 10, 64, "f32", "not_applicable"),
           K.KvTensorShapeV1("value", "gqa", 1, 2, 2, 8, 10, 64, "f32", "pre_rope"),
           K.KvTensorShapeV1("key", "mha", 1, 2, 2, 8, 10, 64, "f32", "pre_rope"),
           K.KvTensorShapeV1("key", "mqa", 1, 2, 2, 8, 10, 64, "f32", "pre_rope"),
           K.KvTensorShapeV1("key", "gqa", 1, 2, 3, 8, 10, 64, "f32", "pre_rope"),
           K.KvTensorShapeV1("key", "gqa", 0, 2, 2, 8, 10, 64, "f32", "pre_rope")]
    for s in bad:
        with pytest.raises(K.KvError):
            s.validate()
    s = _shape()
    with pytest.raises(K.KvError, match="only canonical"):
        K.KvCacheLayoutV1(2560, 1280, 640, 128).validate_for_shape(s)
    for geo in (K.KvPageGeometryV1(0, 64, 12), K.KvPageGeometryV1(11, 64, 12), K.KvPageGeometryV1(4, 32, 12),
                K.KvPageGeometryV1(4, 64, 0), K.KvPageGeometryV1(4, 64, 12, vectors_per_block=2),
                K.KvPageGeometryV1(4, 64, 12, raw_vector_bytes=128)):
        with pytest.raises(K.KvError):
            geo.validate_for_shape(s)
    with pytest.raises(K.KvError):
        s.validate_block_dim(5)


def test_fib_profile_defaults_text_and_rules():
    p = K.FibQuantProfileV1.paper_default(64, 4, 32, 7)
    text = ('{"schema_version":"fib_quant_profile_v1","ambient_dim":64,"block_dim":4,"codebook_size":32,'
            '"paper_rate_bits_per_coord":1.25,"wire_index_bits":5,"wire_bits_per_coord":1.25,'
            '"norm_format":"fp16_paper","rotation_seed":7,'
            '"rotation_algorithm_version":"qr-gaussian-chacha8-sign-corrected-v1",'
            '"codebook_seed":11400714819323198492,"codebook_version":"fib-quant:paper-core-v1",'
            '"source_mode":"canonical_spherical_beta","radius_method":"beta_quantile",'
            '"direction_method":"roberts_kronecker","lloyd_restarts":4,"lloyd_iterations":25,'
            '"training_samples":960,"empty_cell_policy":"split_highest_distortion"}')
    assert K.serde_text(p.as_json()) == text and p.digest() == _tagged("fib_quant_profile_v1", text)
    assert p.block_count() == 16 and K.wire_index_bits(33) == 6 and K.wire_index_bits(2) == 1
    q = K.FibQuantProfileV1.paper_default(6, 2, 5, 1)
    assert (q.radius_method, q.direction_method, q.training_samples, q.wire_index_bits) == \
        ("k2_closed_form", "fibonacci_spiral", 256, 3)
    assert K.FibQuantProfileV1.paper_default(9, 3, 8, 1).direction_method == "fibonacci_sphere"
    import dataclasses
    for change in ({"wire_index_bits": 6}, {"norm_format": "f32_reference"}, {"lloyd_restarts": 0},
                   {"training_samples": 31}, {"paper_rate_bits_per_coord": 1.3},
                   {"rotation_algorithm_version": "other"}):
        with pytest.raises(K.KvError):
            dataclasses.replace(p, **change).validate()
    for args in ((0, 4, 32), (64, 64, 32), (64, 5, 32), (64, 4, 1)):
        with pytest.raises(K.KvError):
            K.FibQuantProfileV1.paper_default(*args, 1)


def _profile(shape, **kw):
    fp = K.FibQuantProfileV1.paper_default(shape.head_dim, 4, 32, 42)
    return K.KvCompressionProfileV1.from_parts("p1", shape, fp, "blake3:cb", "blake3:rot", kw.pop("axis", "per_token"),
                                               K.KvPageGeometryV1(kw.pop("tpp", 4), shape.head_dim, 12))


def test_compression_profile_text_and_rules():
    s = _shape()
    p = _profile(s)
    j = p.as_json()
    assert list(j) == ["schema_version", "profile_id", "shape_digest", "fib_profile", "fib_profile_digest",
                       "codebook_digest", "rotation_digest", "role_policy", "axis_policy", "page_geometry",
                       "protected_policy", "fallback_policy", "quality_budget", "calibration_digest"]
    assert j["fallback_policy"] == {"mode": "keep_raw", "raw_fallback_available": True}
    assert K.serde_text(j["quality_budget"]) == ('{"max_logit_mse":null,"max_attention_tv":null,'
                                                '"max_topk_disagreement":null,"max_value_aggregation_mse":null,'
                                                '"fallback_on_violation":"keep_raw"}')
    assert j["calibration_digest"] == "missing:calibration" and j["role_policy"] == "key"
    assert p.digest(s) == _tagged("fib_quant_kv_compression_profile_v1", K.serde_text(j))
    with pytest.raises(K.KvError, match="digest mismatch"):      # the shape digest is compared before the role
        p.validate_for_shape(_shape("value"))
    p.role_policy = "value"
    with pytest.raises(K.KvError, match="role"):
        p.validate_for_shape(s)
    p.role_policy = "key"
    p.protected_policy = K.KvProtectedPolicyV1(first_tokens_raw=11)
    with pytest.raises(K.KvError, match="protected token count"):
        p.validate_for_shape(s)
    p.protected_policy = K.KvProtectedPolicyV1(1, 2, [1], [])
    assert p.protected_policy.is_protected(s, 0, 0, 0) and p.protected_policy.is_protected(s, 0, 0, 8)
    assert p.protected_policy.is_protected(s, 1, 0, 5) and not p.protected_policy.is_protected(s, 0, 1, 7)
    p.quality_budget.max_logit_mse = -1.0
    with pytest.raises(K.KvError, match="max_logit_mse"):
        p.validate_for_shape(s)


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [64, 128])
def test_pages_encoded_and_decoded_on_the_gpu(oracle_mod, dim):
    """Every coded block carries the oracle's single-vector code, protected and refused vectors stay raw with
    the reference's reasons, the decoded tensor is the oracle's binary64 decode, digests chain and tampering
    is caught."""
    from provekv_b200 import _lib as L
    from provekv_b200 import tables
    from kvgen import synthetic_kv
    s = K.KvTensorShapeV1("key", "gqa", 2, 3, 2, 8, 11, dim, "f32", "post_rope")
    rot, cb = tables.haar_rotation(dim, 42), tables.fib_codebook(dim, seed=42)
    fp = K.FibQuantProfileV1.paper_default(dim, 4, 32, 42)
    rec = 2 + dim // 4 * 5 // 8
    prof = K.KvCompressionProfileV1.from_parts("kv-test", s, fp, "blake3:codebook", K.rotation_digest(dim, 42, rot),
                                               "per_token", K.KvPageGeometryV1(4, dim, rec))
    prof.protected_policy = K.KvProtectedPolicyV1(first_tokens_raw=1, last_tokens_raw=2, raw_layers=[], raw_heads=[])
    x = synthetic_kv(s.vector_count(), dim, seed=6).reshape(2, 3, 2, 11, dim)
    x[1, 2, 0, 5] = 0.0                        # zero norm: refused by the encoder, kept raw
    x[0, 1, 1, 4] *= np.float32(3.0e4)         # norm beyond fp16
    lay = K.KvCacheLayoutV1.canonical(s)
    enc = K.encode_kv_tensor(s, lay, prof, x, rot, cb, recorded_unix_seconds=5)
    assert len(enc.pages) == 3 and [p.token_count for p in enc.pages] == [4, 4, 3]
    flat = x.reshape(-1, dim)
    st, want, _, _ = oracle_mod.fib_encode(np.where(np.abs(flat).sum(1, keepdims=True) == 0, 1.0, flat).astype(np.float32),
                                           rot, cb, numerics=L.FIB_NUMERICS_SINGLE, nthreads=4)
    ctx = enc.context()
    seen, raws = 0, {}
    for page in enc.pages:
        page.validate(s, ctx)
        order = [(b.batch, b.layer, b.kv_head, b.token) for b in page.encoded_blocks]
        assert order == sorted(order) and [b.block_id for b in page.encoded_blocks] == list(range(len(order)))
        for b in page.encoded_blocks:
            v = ((b.batch * 3 + b.layer) * 2 + b.kv_head) * 11 + b.token
            if b.raw_fallback:
                raws[(b.batch, b.layer, b.kv_head, b.token)] = b.reason
                assert np.array_equal(b.values, flat[v])
            else:
                assert b.record == want[v].tobytes() and b.reason == "fib_quant_per_token"
            seen += 1
    assert seen == s.vector_count()
    assert raws[(1, 2, 0, 5)] == "encode_fallback:zero norm vector is not valid on the normal FibQuant encode path"
    assert raws[(0, 1, 1, 4)] == "encode_fallback:corrupt payload: norm cannot be represented as finite positive fp16"
    assert raws[(0, 0, 0, 0)] == raws[(1, 2, 1, 10)] == raws[(0, 0, 0, 9)] == "protected_region"
    assert len(raws) == 2 * 3 * 2 * 3 + 2
    r = enc.receipt
    assert (r["operation_kind"], r["encoded_pages"], r["raw_fallback_blocks"], r["compressed_blocks"]) == \
        ("compress", 3, len(raws), s.vector_count() - len(raws))
    assert r["fallback_reasons"][0] == "protected_region" and len(r["fallback_reasons"]) == 3
    assert r["page_digests"] == [p.page_digest for p in enc.pages] and r["source_digest"] == K.kv_tensor_digest(x)
    # a coded block's JSON, spelled out
    blk = next(b for b in enc.pages[0].encoded_blocks if not b.raw_fallback)
    code = blk.as_json(ctx)["encoding"]["fib_quant"]["code"]
    assert list(code) == ["schema_version", "profile_digest", "codebook_digest", "rotation_digest", "ambient_dim",
                          "block_dim", "norm_format", "norm_payload", "wire_index_bits", "block_count", "indices"]
    assert code["norm_payload"] == list(blk.record[:2]) and len(code["indices"]) == rec - 2
    raw_blk = next(b for b in enc.pages[0].encoded_blocks if b.raw_fallback)
    shown = json.loads(K.serde_text(raw_blk.as_json(ctx)))["encoding"]["raw_f32"]["values"]
    assert np.array_equal(np.array(shown, np.float32), raw_blk.values)       # binary32 shortest digits

    dec, dr = K.decode_kv_pages(enc, rot, cb, recorded_unix_seconds=6)
    coded = np.array([not any(k == (b, l, h, t) for k in raws) for b in range(2) for l in range(3) for h in range(2)
                      for t in range(11)])
    st, ref, _, _ = oracle_mod.fib_decode_exact(want[coded], dim, rot, cb)
    got = dec.reshape(-1, dim)
    assert st == 0 and np.array_equal(got[coded].view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(got[~coded], flat[~coded])
    assert dr["decoded_digest"] == K.kv_tensor_digest(dec) and dr["raw_fallback_blocks"] == len(raws)
    assert dr["operation_kind"] == "decode" and dr["decoded_pages"] == 3

    enc.pages[1].encoded_blocks[3].token += 1 if enc.pages[1].encoded_blocks[3].token < 7 else -1
    with pytest.raises(K.KvError, match="digest mismatch"):
        K.decode_kv_pages(enc, rot, cb)
    strict = K.KvCompressionProfileV1.from_parts("kv-strict", s, fp, "blake3:codebook", prof.rotation_digest,
                                                 "per_token", K.KvPageGeometryV1(4, dim, rec))
    strict.fallback_mode = "fail_closed"
    # the reference's walk (page, batch, layer, head, token) meets the out-of-range norm of (0, 1, 1, 4) before the
    # zero vector of (1, 2, 0, 5): both lie in page 1
    with pytest.raises(K.KvError, match="norm cannot be represented"):
        K.encode_kv_tensor(s, lay, strict, x, rot, cb)
    x2 = x.copy()
    x2[0, 1, 1, 4] = x[0, 1, 1, 3]
    with pytest.raises(K.KvError, match="zero norm"):
        K.encode_kv_tensor(s, lay, strict, x2, rot, cb)
    x2[1, 0, 0, 2] *= np.float32(3.0e4)        # page 0 comes before page 1 whatever the batch
    with pytest.raises(K.KvError, match="norm cannot be represented"):
        K.encode_kv_tensor(s, lay, strict, x2, rot, cb)
    rawp = K.KvCompressionProfileV1.from_parts("kv-raw", s, fp, "blake3:codebook", prof.rotation_digest, "raw",
                                               K.KvPageGeometryV1(11, dim, rec))
    allraw = K.encode_kv_tensor(s, lay, rawp, x, rot, cb)
    assert allraw.receipt["compressed_blocks"] == 0 and allraw.receipt["fallback_reasons"] == ["raw_axis_policy"]
    back, _ = K.decode_kv_pages(allraw, rot, cb)
    assert np.array_equal(back, x)


def _tiny(role="value", tokens=4, axis="per_channel", seed=13):
    """The fixture of the reference's own kv tests (fib-quant/tests/kv_*.rs): one head of dim 8, k = 2, N = 8."""
    s = K.KvTensorShapeV1(role, "mha", 1, 1, 1, 1, tokens, 8, "f32", "post_rope" if role == "key" else "not_applicable")
    fp = K.FibQuantProfileV1.paper_default(8, 2, 8, seed)
    import dataclasses
    fp = dataclasses.replace(fp, training_samples=64, lloyd_restarts=1, lloyd_iterations=1)
    p = K.KvCompressionProfileV1.from_parts("fixture", s, fp, "blake3:codebook", "blake3:rotation", axis,
                                            K.KvPageGeometryV1(2, 8, 64))
    return s, K.KvCacheLayoutV1.canonical(s), p


def test_axis_without_an_encoder_keeps_every_vector_raw():
    """fib-quant/tests/kv_encode_decode_reference.rs:63-72: a per-channel profile stores 4 raw blocks, no coded
    one, and decodes to the input exactly; no table and no GPU is involved."""
    s, lay, p = _tiny()
    values = (np.sin((np.arange(32, dtype=np.float32) + np.float32(1.0)) * np.float32(0.07)) + np.float32(0.25)).astype(np.float32)
    enc = K.encode_kv_tensor(s, lay, p, values, None, None)
    assert enc.receipt["compressed_blocks"] == 0 and enc.receipt["raw_fallback_blocks"] == 4
    assert enc.receipt["encoded_pages"] == 2 and len(enc.receipt["page_digests"]) == len(enc.pages) == 2
    assert enc.receipt["fallback_reasons"] == ["unsupported_axis_raw_fallback"]      # kv/codec.rs:287-298
    dec, dr = K.decode_kv_pages(enc, None, None)
    assert np.array_equal(dec.reshape(-1), values) and dr["decoded_pages"] == 2 and dr["raw_fallback_blocks"] == 4
    # kv_corruption_rejection.rs:43-44: a tampered page digest rejects the decode
    enc.pages[0].page_digest += "-tampered"
    with pytest.raises(K.KvError):
        K.decode_kv_pages(enc, None, None)


def test_shape_contract_round_trips_and_bounded_shapes():
    """kv_shape_contracts.rs:28-62 (digests survive a JSON round trip) and kv_property_shapes.rs (every bounded
    shape validates with its canonical layout and a two-token page geometry)."""
    s, lay, p = _tiny("key", axis="per_token", seed=11)
    again = K.KvTensorShapeV1(**{k: v for k, v in json.loads(K.serde_text(s.as_json())).items()})
    assert again.digest() == s.digest()
    lj = json.loads(K.serde_text(lay.as_json()))
    assert K.KvCacheLayoutV1(lj["batch_stride"], lj["layer_stride"], lj["head_stride"], lj["token_stride"]).digest(s) == \
        lay.digest(s)
    assert json.loads(K.serde_text(p.as_json()))["fib_profile"]["radius_method"] == "k2_closed_form"
    for batch in (1, 2):
        for layers in (1, 2):
            for heads in (1, 2, 3):
                for tokens in (1, 2, 5, 7):
                    for mult in (1, 2, 3, 4):
                        sh = K.KvTensorShapeV1("key", "mha", batch, layers, heads, heads, tokens, 2 * mult, "f32", "post_rope")
                        sh.validate()
                        sh.validate_block_dim(2)
                        K.KvCacheLayoutV1.canonical(sh).validate_for_shape(sh)
                        K.KvPageGeometryV1(min(tokens, 2), 2 * mult, 64).validate_for_shape(sh)


def test_policy_decisions():
    """kv_policy_role_aware.rs: the role-aware baseline compresses keys per channel and values per token; a
    protected layer or a missing calibration keeps the vector raw."""
    def shape(role):
        return K.KvTensorShapeV1(role, "gqa", 1, 2, 2, 4, 8, 16, "f32", "pre_rope" if role == "key" else "not_applicable")
    pol = K.KvCompressionPolicyV1.role_aware_baseline()
    key = K.decide_kv_compression(pol, shape("key"), 0, 0, 1, True)
    value = K.decide_kv_compression(pol, shape("value"), 0, 0, 1, True)
    assert (key["action"], key["axis_policy"], key["reasons"]) == ("compress", "per_channel", ["key_role_axis"])
    assert (value["action"], value["axis_policy"], value["reasons"]) == ("compress", "per_token", ["value_role_axis"])
    assert K.decide_kv_compression(pol, shape("value"), 0, 0, 7, True)["reasons"] == ["protected_region"]  # last token
    pol = K.KvCompressionPolicyV1("fib_quant_per_token", K.KvProtectedPolicyV1(1, 0, [1], []), True, True)
    assert K.decide_kv_compression(pol, shape("value"), 0, 0, 0, False)["action"] == "keep_raw"
    assert K.decide_kv_compression(pol, shape("value"), 1, 0, 3, True)["reasons"] == ["protected_region"]
    pol.protected_policy.first_tokens_raw = 0
    missing = K.decide_kv_compression(pol, shape("value"), 0, 0, 2, False)
    assert (missing["action"], missing["reasons"]) == ("keep_raw", ["calibration_missing"])
    pol.allow_raw_fallback = False
    assert K.decide_kv_compression(pol, shape("value"), 0, 0, 2, False)["action"] == "need_calibration"
    assert K.decide_kv_compression(K.KvCompressionPolicyV1.raw(), shape("key"), 0, 0, 2, True)["reasons"] == ["raw_strategy"]
    exp = K.KvCompressionPolicyV1("experimental_fib_quant_role_aware")
    assert K.decide_kv_compression(exp, shape("key"), 0, 0, 2, True) == \
        {"action": "compress", "axis_policy": "per_channel", "reasons": ["experimental_role_aware"]}
    with pytest.raises(K.KvError, match="outside shape"):
        K.decide_kv_compression(pol, shape("value"), 2, 0, 0, True)
