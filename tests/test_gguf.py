"""GGUF container, tensor recipe, derived lock, model lock and loader round trips (CPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from sllm_b200.formats import gguf as G
from sllm_b200.formats import model_lock as ML
from sllm_b200.models import config as MC
from sllm_b200.models.llama import LlamaModel, init_random_weights
from sllm_b200.models import loader


def _simple(tmp_path, **kw):
    a = np.arange(64, dtype="<f4").reshape(4, 16)
    b = np.arange(96, dtype=np.uint8).reshape(3, 32)
    p = str(tmp_path / "m.gguf")
    md = {"general.architecture": "llama", "k.int": 7, "k.neg": -3, "k.f": 0.5, "k.s": "héllo", "k.arr": ["a", "b"],
          "k.ints": [1, 2, 3], "k.big": 1 << 40, "k.bool": True}
    md.update(kw)
    d = G.write_gguf(p, md, [("a", (4, 16), G.T_F32, a.tobytes()), ("b", (3, 32), G.T_I8, b.tobytes())])
    return p, d, a, b


def test_roundtrip_and_determinism(tmp_path):
    p, d, a, b = _simple(tmp_path)
    g = G.GgufFile(p)
    assert g.metadata["k.int"] == 7 and g.metadata["k.neg"] == -3 and g.metadata["k.s"] == "héllo"
    assert g.metadata["k.arr"] == ["a", "b"] and g.metadata["k.ints"] == [1, 2, 3] and g.metadata["k.big"] == 1 << 40
    assert g.metadata["k.bool"] is True
    np.testing.assert_array_equal(g.numpy("a"), a)
    np.testing.assert_array_equal(g.numpy("b"), b)
    assert g.data_start % 32 == 0 and all(t.offset % 32 == 0 for t in g.tensors.values())
    assert g.sha256() == d["sha256"] and g.metadata_sha256 == d["metadata_sha256"]
    assert g.tensor_catalog_sha256 == d["tensor_catalog_sha256"]
    first = open(p, "rb").read()
    p2, d2, _, _ = _simple(tmp_path)
    assert open(p2, "rb").read() == first and d2 == d
    t = g.upload("a", "cpu", torch.float32).view(4, 16)
    assert torch.equal(t, torch.from_numpy(a.copy()))
    g.close()


def _patch(path, fn):
    data = bytearray(open(path, "rb").read())
    fn(data)
    open(path, "wb").write(bytes(data))


def test_reader_fails_closed(tmp_path):
    p, _, _, _ = _simple(tmp_path)
    good = open(p, "rb").read()
    for mutate, msg in [
        (lambda d: d.__setitem__(slice(0, 4), b"GGUX"), "not a GGUF"),
        (lambda d: d.__setitem__(slice(4, 8), struct.pack("<I", 2)), "version"),
        (lambda d: d.__setitem__(slice(8, 16), struct.pack("<Q", 1 << 30)), "out of range"),
    ]:
        open(p, "wb").write(good)
        _patch(p, mutate)
        with pytest.raises(G.GgufError, match=msg):
            G.GgufFile(p)
    open(p, "wb").write(good[:-40])                      # payload beyond EOF
    with pytest.raises(G.GgufError, match="beyond the end"):
        G.GgufFile(p)
    open(p, "wb").write(good[:60])                       # header cut
    with pytest.raises(G.GgufError):
        G.GgufFile(p)
    with pytest.raises(G.GgufError, match="duplicate"):
        G.write_gguf(p, {}, [("a", (4,), G.T_F32, b"\0" * 16), ("a", (4,), G.T_F32, b"\0" * 16)])
    with pytest.raises(G.GgufError):
        G.write_gguf(p, {}, [("a", (1, 1, 1, 1, 4), G.T_F32, b"\0" * 16)])
    os.symlink(p, str(tmp_path / "link.gguf"))
    with pytest.raises(G.GgufError, match="regular"):
        G.GgufFile(str(tmp_path / "link.gguf"))


def _raw_header(tensors, kv=()):
    """Hand-assembled header for structural rejection tests: tensors = (name, dims, type, offset)."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv)))
    for k, v in kv:
        out += struct.pack("<Q", len(k)) + k.encode() + struct.pack("<I", G.V_U32) + struct.pack("<I", v)
    for name, dims, tt, off in tensors:
        out += struct.pack("<Q", len(name)) + name.encode() + struct.pack("<I", len(dims))
        for d in dims:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", tt, off)
    out += b"\0" * ((-len(out)) % 32)
    return out


@pytest.mark.parametrize("tensors,kv,msg", [
    ([("a", [8], 0, 0), ("b", [8], 0, 16)], (), "aligned"),
    ([("a", [16], 0, 0), ("b", [8], 0, 32)], (), "overlaps"),
    ([("a", [8], 0, 0), ("a", [8], 0, 32)], (), "duplicate tensor"),
    ([("a", [8], 7, 0)], (), "unknown tensor type"),
    ([("a", [2, 2, 2, 2, 2], 0, 0)], (), "rank"),
    ([("a", [8], 0, 0)], (("k", 1), ("k", 2)), "duplicate metadata"),
    ([("a", [8], 0, 0)], (("general.alignment", 64),), "alignment"),
    ([("a", [33], 39, 0)], (), "block size"),
    ([("a", [1 << 62, 1 << 62], 0, 0)], (), "out of range"),
])
def test_structural_rejections(tmp_path, tensors, kv, msg):
    p = str(tmp_path / "x.gguf")
    open(p, "wb").write(bytes(_raw_header(tensors, kv)) + b"\0" * 256)
    with pytest.raises(G.GgufError, match=msg):
        G.GgufFile(p)


def test_block_layout_regroup():
    rng = np.random.default_rng(0)
    packed = rng.integers(0, 256, (6, 64), dtype=np.uint8)           # K = 128
    e8 = rng.integers(100, 140, (6, 4), dtype=np.uint8)
    blocks = G.mxfp4_to_gguf_blocks(packed, e8)
    assert blocks.shape == (6, 4, 17) and G.tensor_nbytes((6, 128), G.T_MXFP4) == blocks.nbytes
    p2, s2 = G.mxfp4_from_gguf_blocks(blocks)
    np.testing.assert_array_equal(p2, packed); np.testing.assert_array_equal(s2, e8)
    bs = rng.integers(0, 127, (6, 8), dtype=np.uint8)
    nb = G.nvfp4_to_gguf_blocks(packed, bs)
    assert nb.shape == (6, 2, 36) and G.tensor_nbytes((6, 128), G.T_NVFP4) == nb.nbytes
    p3, s3 = G.nvfp4_from_gguf_blocks(nb)
    np.testing.assert_array_equal(p3, packed); np.testing.assert_array_equal(s3, bs)


def test_recipe_and_derived_lock(tmp_path):
    p = str(tmp_path / "r.gguf")
    b = [{"logical_tensor": "w", "value_tensor": "w", "encoding": "fp8-e4m3fn-kblock128-f32-scale", "role": "weight",
          "logical_shape": [2, 128], "scope": "consumed", "scales": [{"role": "block", "tensor": "w.scale"}]}]
    md = G.recipe_metadata(b)
    tensors = [("w", (2, 128), G.T_I8, b"\1" * 256), ("w.scale", (2, 1), G.T_F32, b"\0" * 8)]
    d = G.write_gguf(p, md, tensors)
    g = G.GgufFile(p)
    assert g.recipe()["bindings"][0]["value_tensor"] == "w"
    lock = G.make_derived_lock(p, d, "toy:fp8", ["sha256:" + "0" * 64], {"id": "t", "args": {}})
    lp = str(tmp_path / "r.lock.json")
    json.dump(lock, open(lp, "w"))
    G.verify_gguf(p, G.read_derived_lock(lp)).close()
    # tampering with the payload, the recipe digest or the lock is detected
    _patch(p, lambda dd: dd.__setitem__(len(dd) - 1, dd[-1] ^ 1))
    with pytest.raises(G.GgufError, match="does not match"):
        G.verify_gguf(p, lock)
    bad = dict(lock); bad["semantic_model_id"] = "other"
    json.dump(bad, open(lp, "w"))
    with pytest.raises(G.GgufError, match="fingerprint"):
        G.read_derived_lock(lp)
    md2 = dict(md); md2[G.RECIPE_SHA_KEY] = "0" * 64
    G.write_gguf(p, md2, tensors)
    with pytest.raises(G.GgufError, match="digest"):
        G.GgufFile(p).recipe()
    b2 = [dict(b[0], scales=[{"role": "block", "tensor": "missing"}])]
    G.write_gguf(p, G.recipe_metadata(b2), tensors)
    with pytest.raises(G.GgufError, match="missing tensor"):
        G.GgufFile(p).recipe()


def test_model_lock(tmp_path):
    root = tmp_path / "cache"
    root.mkdir()
    (root / "config.json").write_text('{"a": 1}')
    (root / "tokenizer.json").write_text("{}")
    doc = ML.make_model_lock(str(root), "fixture/tiny", "0123456789abcdef0123456789abcdef01234567", ["tiny"],
                             {"model_type": "llama"}, {"generation_stop_policy": {"version": 1, "stop_token_ids": [2]}})
    lp = tmp_path / "lock.json"
    lp.write_text(json.dumps(doc))
    lock = ML.read_model_lock(str(lp))
    assert lock.fingerprint.startswith("sha256:") and lock.stop_token_ids == [2] and lock.aliases == ["tiny"]
    c = lock.verify_cache(str(root))
    assert c.read("config.json") == b'{"a": 1}'
    c.close()
    (root / "config.json").write_text('{"a": 2}')
    with pytest.raises(ML.ModelLockError, match="digest"):
        lock.verify_cache(str(root))
    for text, msg in [('{"a": 1, "a": 2}', "duplicate"), ('{"a": 1.5}', "floating"), ('{"a": NaN}', "non-finite"),
                      ("[" * 100 + "]" * 100, "deep|invalid"), ('{"a": 99999999999999999999}', "safe range")]:
        with pytest.raises(ML.ModelLockError, match=msg):
            ML.parse_restricted_json(text.encode())
    bad = json.loads(json.dumps(doc)); bad["model"]["repo_id"] = "other"
    with pytest.raises(ML.ModelLockError, match="fingerprint"):
        ML.parse_model_lock(json.dumps(bad).encode())
    bad = json.loads(json.dumps(doc)); bad["model"]["files"][0]["path"] = "../x"; bad["fingerprint"] = ML.fingerprint(bad)
    with pytest.raises(ML.ModelLockError, match="unsafe"):
        ML.parse_model_lock(json.dumps(bad).encode())
    # canonical key order is by UTF-16 code units
    assert ML.canonical_json({"\U0001f600": 1, "￿": 2}) == '{"\U0001f600":1,"￿":2}'


@pytest.mark.parametrize("wf", ["fp32", "fp8"])
def test_llama_export_load_roundtrip(tmp_path, wf):
    cfg = MC.tiny_llama()
    cfg.weight_format = wf
    if wf == "fp8":
        cfg.ffn = 512          # column shards of 1x128-scaled weights must align to the scale blocks
    w = init_random_weights(cfg, "cpu", seed=3)
    p = str(tmp_path / "tiny.gguf")
    lock = loader.export_llama_gguf(cfg, w, p, chat_template="{{ messages }}")
    g = G.verify_gguf(p, lock)
    cfg2, w2 = loader.load_llama_gguf(g, "cpu")
    assert cfg2 == cfg
    assert torch.equal(w2.embed, w.embed)
    for a, b in zip(w.layers, w2.layers):
        for n in ("qkv", "o", "gate_up", "down"):
            la, lb = getattr(a, n), getattr(b, n)
            assert la.kind == lb.kind and torch.equal(la.w, lb.w)
            if la.scale_t is not None:
                assert torch.equal(la.scale_t, lb.scale_t)
    assert torch.equal(w.lm_head.w, w2.lm_head.w)
    # tensor-parallel shards of the file equal the shards the random initialiser keeps
    for r in range(2):
        _, ws = loader.load_llama_gguf(g, "cpu", tp_size=2, tp_rank=r)
        wr = init_random_weights(cfg, "cpu", seed=3, tp_size=2, tp_rank=r)
        for a, b in zip(wr.layers, ws.layers):
            for n in ("qkv", "o", "gate_up", "down"):
                la, lb = getattr(a, n), getattr(b, n)
                if wf == "fp32":
                    assert torch.equal(la.w, lb.w)
                else:
                    assert la.w.shape == lb.w.shape and la.scale_t.shape == lb.scale_t.shape
        assert ws.vocab_offset == wr.vocab_offset and ws.lm_head.w.shape == wr.lm_head.w.shape
    assert type(loader.tokenizer_from_gguf(g)).__name__ == "ByteTokenizer"
    g.close()


@pytest.mark.parametrize("wf", ["mxfp4", "nvfp4"])
def test_llama_4bit_export_load_roundtrip(tmp_path, wf):
    """4-bit weights travel as standard GGML blocks (types 39 / 40) and come back bit-identical in the resident layout."""
    cfg = MC.tiny_llama()
    cfg.weight_format, cfg.kv_format, cfg.ffn = wf, "bf16", 512
    w = init_random_weights(cfg, "cpu", seed=4)
    p = str(tmp_path / "tiny4.gguf")
    lock = loader.export_llama_gguf(cfg, w, p)
    g = G.verify_gguf(p, lock)
    want_type = G.T_MXFP4 if wf == "mxfp4" else G.T_NVFP4
    assert g.tensors["blk.0.attn_q.weight"].ttype == want_type
    enc = {b["logical_tensor"]: b for b in g.recipe()["bindings"]}["blk.0.ffn_down.weight"]
    assert enc["encoding"] == (loader.MXFP4_ENCODING if wf == "mxfp4" else loader.NVFP4_ENCODING)
    cfg2, w2 = loader.load_llama_gguf(g, "cpu")
    assert cfg2 == cfg
    for a, b in zip(w.layers, w2.layers):
        for n in ("qkv", "o", "gate_up", "down"):
            la, lb = getattr(a, n), getattr(b, n)
            assert lb.kind == "w4" and torch.equal(la.w4.tiles, lb.w4.tiles)
            if wf == "nvfp4":
                assert torch.equal(la.w4.tensor_scale, lb.w4.tensor_scale)
    # a tensor-parallel shard decodes to the same values as the matching slice of the full matrix
    _, ws = loader.load_llama_gguf(g, "cpu", tp_size=2, tp_rank=1)
    full = w.layers[0].down.w4.dequantized(0)
    assert torch.equal(ws.layers[0].down.w4.dequantized(0), full[:, full.shape[1] // 2:])
    g.close()


def test_fp8_channel_scale_weights_load_as_block_scaled(tmp_path):
    """One scale per output row is the 1x128 form with the scale repeated along K: the loader accepts it exactly."""
    from sllm_b200.formats import codecs
    cfg = MC.tiny_llama()
    cfg.weight_format, cfg.kv_format, cfg.ffn = "fp8", "fp8", 512
    w = init_random_weights(cfg, "cpu", seed=6)
    p = str(tmp_path / "chan.gguf")
    lock = loader.export_llama_gguf(cfg, w, p, fp8_channel_scales=True)
    g = G.verify_gguf(p, lock)
    b = {x["logical_tensor"]: x for x in g.recipe()["bindings"]}["blk.1.attn_output.weight"]
    assert b["encoding"] == "fp8-e4m3fn-channel-f32-scale"
    _, w2 = loader.load_llama_gguf(g, "cpu")
    lw = w2.layers[1].o
    codes, sc = codecs.quantize_fp8_outer_rows(w.layers[1].o.dequantized().numpy())
    assert lw.kind == "fp8" and np.array_equal(lw.w.numpy(), codes)
    assert lw.scale_t.shape == (cfg.q_size // 128, cfg.d_model)
    np.testing.assert_array_equal(lw.dequantized().numpy(), codecs.dequantize_fp8_outer_rows(codes, sc))
    g.close()
