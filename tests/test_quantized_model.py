"""Quantised-model descriptors and the mixed-precision importer, on a synthetic checkpoint written by the test
(safetensors container, compressed-tensors naming): recipe validation, inventory, scale planes, digest, resident
weights and a CPU generation through them."""
import json
import struct

import numpy as np
import pytest
import torch

from sllm_b200.formats import codecs
from sllm_b200.formats import quantized_model as QM
from sllm_b200.models import config as MC

GEO = QM.ModelGeometry(n_layers=2, d_model=128, q_size=128, kv_size=64, ffn=256, vocab=320)
P = GEO.prefix


def _config(**over):
    spec = lambda bits, strategy, dynamic=False, group=None: dict(num_bits=bits, type="float", strategy=strategy,
                                                                  dynamic=dynamic, symmetric=True, group_size=group)
    q = {"format": "mixed-precision", "quant_method": "compressed-tensors", "quantization_status": "compressed",
         "config_groups": {
             "group_0": {"format": "float-quantized", "weights": spec(8, "channel"),
                         "input_activations": spec(8, "token", True)},
             "group_1": {"format": "nvfp4-pack-quantized", "weights": spec(4, "tensor_group", False, 16),
                         "input_activations": spec(4, "tensor_group", "local", 16)}},
         "kv_cache_scheme": spec(8, "tensor"), "ignore": ["lm_head"]}
    q.update(over)
    return json.dumps({"quantization_config": q}).encode()


def _bf16_bytes(x: np.ndarray) -> bytes:
    return (x.astype(np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()


def _write_checkpoint(root, seed=0, drop=None, extra=None):
    rng = np.random.default_rng(seed)
    tensors = {}
    dense = {}

    def add(name, dtype, shape, raw):
        tensors[name] = (dtype, tuple(shape), raw)

    def add_bf16(name, arr):
        add(name, "BF16", arr.shape, _bf16_bytes(arr))

    emb = (rng.standard_normal((GEO.vocab, GEO.d_model)) * 0.05).astype(np.float32)
    add_bf16(f"{P}.embed_tokens.weight", emb)
    add_bf16(f"{P}.norm.weight", np.ones(GEO.d_model, dtype=np.float32))
    for l in range(GEO.n_layers):
        lp = f"{P}.layers.{l}"
        for proj, rows, cols in (("q", GEO.q_size, GEO.d_model), ("k", GEO.kv_size, GEO.d_model), ("v", GEO.kv_size, GEO.d_model),
                                 ("o", GEO.d_model, GEO.q_size)):
            w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
            codes, sc = codecs.quantize_fp8_outer_rows(w)
            base = f"{lp}.self_attn.{proj}_proj"
            add(base + ".weight", "F8_E4M3", (rows, cols), codes.tobytes())
            add_bf16(base + ".weight_scale", codecs.round_bf16(sc.reshape(rows, 1)))
            add_bf16(base + ".input_scale", np.ones((1,), dtype=np.float32))
            dense[base] = codecs.dequantize_fp8_outer_rows(codes, codecs.round_bf16(sc))
        for proj, rows, cols in (("gate", GEO.ffn, GEO.d_model), ("up", GEO.ffn, GEO.d_model), ("down", GEO.d_model, GEO.ffn)):
            w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
            packed, block, ts = codecs.quantize_nvfp4(w, tensor_scale=2.0 ** -9)      # gate and up share the outer scale
            base = f"{lp}.mlp.{proj}_proj"
            add(base + ".weight_packed", "U8", packed.shape, packed.tobytes())
            add(base + ".weight_scale", "F8_E4M3", block.shape, block.tobytes())
            add(base + ".weight_global_scale", "F32", (1,), struct.pack("<f", 1.0 / float(ts)))   # stored as a reciprocal
            add(base + ".input_global_scale", "F32", (1,), struct.pack("<f", 37.0))
            dense[base] = codecs.dequantize_nvfp4(packed, block, ts, cols)
        add_bf16(f"{lp}.input_layernorm.weight", np.ones(GEO.d_model, dtype=np.float32))
        add_bf16(f"{lp}.post_attention_layernorm.weight", np.ones(GEO.d_model, dtype=np.float32))
        add_bf16(f"{lp}.self_attn.k_scale", np.array([0.0625 * (l + 1)], dtype=np.float32))
        add_bf16(f"{lp}.self_attn.v_scale", np.array([0.03125 * (l + 1)], dtype=np.float32))
    add_bf16("model.vision_tower.something", np.zeros((4,), dtype=np.float32))       # outside the language model: ignored
    for name in drop or ():
        tensors.pop(name)
    for name, (dtype, shape, raw) in (extra or {}).items():
        tensors[name] = (dtype, shape, raw)
    header, blob, off = {}, bytearray(), 0
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blob += raw
        off += len(raw)
    hj = json.dumps(header).encode()
    (root / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + bytes(blob))
    (root / "config.json").write_bytes(_config())
    return dense


def test_recipe_validation():
    r = QM.parse_recipe(_config())
    assert r.attention_weight is QM.TensorEncoding.FP8_E4M3FN_CHANNEL_BF16_SCALE
    assert r.mlp_weight is QM.TensorEncoding.NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER and r.ignored == ("lm_head",)
    assert r.to_dict()["schema_version"] == QM.RECIPE_SCHEMA
    assert QM.TensorEncoding.NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER is not QM.TensorEncoding.MXFP4_E2M1_BLOCK32_E8M0
    for bad in (dict(format="int-quantized"), dict(quant_method="awq"), dict(config_groups={}), dict(ignore="lm_head"),
                dict(kv_cache_scheme=None)):
        with pytest.raises(QM.QuantizedModelError):
            QM.parse_recipe(_config(**bad))
    with pytest.raises(QM.QuantizedModelError):
        QM.parse_recipe(b"{not json")
    sc = QM.StaticFp8KvScale(0x3D80, 0x3D00)            # bf16 bit patterns of 0.0625 and 0.03125
    assert (sc.key, sc.value) == (0.0625, 0.03125)


def test_inventory_digest_and_rejections(tmp_path):
    _write_checkpoint(tmp_path)
    qm = QM.open_mixed_precision_checkpoint(str(tmp_path), GEO)
    d = qm.tensors[f"{P}.layers.1.mlp.down_proj.weight"]
    assert d.encoding is QM.TensorEncoding.NVFP4_E2M1_BLOCK16_E4M3FN_F32_OUTER and d.logical_shape == (128, 256)
    assert d.value_shape == (128, 128) and d.plane(QM.ScalePlaneRole.WEIGHT_OUTER).reciprocal
    assert abs(float(qm.read_scale(d.plane(QM.ScalePlaneRole.WEIGHT_OUTER))[0]) - 2.0 ** -9) < 1e-12
    a = qm.tensors[f"{P}.layers.0.self_attn.k_proj.weight"]
    assert a.role is QM.TensorRole.ATTENTION_PROJECTION and a.plane(QM.ScalePlaneRole.WEIGHT_CHANNEL).shape == (64, 1)
    assert qm.kv_scales[1].key == 0.125 and qm.kv_scales[0].value == 0.03125
    assert qm.digest.startswith("sha256:")
    # same structure, other values: same digest; other KV scale or shape: another digest
    other = tmp_path / "b"
    other.mkdir()
    _write_checkpoint(other, seed=5)
    assert QM.open_mixed_precision_checkpoint(str(other), GEO).digest == qm.digest
    k1 = f"{P}.layers.1.self_attn.k_scale"
    _write_checkpoint(other, extra={k1: ("BF16", (1,), _bf16_bytes(np.array([0.5], dtype=np.float32)))})
    assert QM.open_mixed_precision_checkpoint(str(other), GEO).digest != qm.digest
    # a missing scale tensor, a wrong shape, an unconsumed language-model tensor, a negative KV scale
    for kw in (dict(drop=[f"{P}.layers.0.mlp.up_proj.weight_global_scale"]),
               dict(extra={f"{P}.layers.0.self_attn.q_proj.weight_scale": ("BF16", (64, 1), b"\0" * 128)}),
               dict(extra={f"{P}.layers.0.mystery": ("F32", (1,), b"\0" * 4)}),
               dict(extra={k1: ("BF16", (1,), _bf16_bytes(np.array([-1.0], dtype=np.float32)))})):
        _write_checkpoint(other, **kw)
        with pytest.raises(QM.QuantizedModelError):
            QM.open_mixed_precision_checkpoint(str(other), GEO)
    # container damage: overlapping ranges, a range past the end
    raw = (tmp_path / "model.safetensors").read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    names = list(hdr)
    hdr[names[1]]["data_offsets"] = hdr[names[0]]["data_offsets"][:1] + [hdr[names[0]]["data_offsets"][0] + (hdr[names[1]]["data_offsets"][1] - hdr[names[1]]["data_offsets"][0])]
    hj = json.dumps(hdr).encode()
    (other / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + raw[8 + n:])
    with pytest.raises(QM.QuantizedModelError):
        QM.read_safetensors_header(str(other / "model.safetensors"))
    (other / "model.safetensors").write_bytes(raw[:-16])
    with pytest.raises(QM.QuantizedModelError):
        QM.read_safetensors_header(str(other / "model.safetensors"))


def test_resident_weights_execute_the_recipe(tmp_path):
    """FP8 attention + NVFP4 MLP + per-layer static FP8 KV scales, run on the CPU oracle path."""
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.engine.engine import Engine
    from sllm_b200.models.llama import LlamaModel
    dense = _write_checkpoint(tmp_path)
    qm = QM.open_mixed_precision_checkpoint(str(tmp_path), GEO)
    cfg = MC.ModelConfig(name="tiny-mixed", n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256, vocab=320,
                         tie_embeddings=True, weight_format="mixed-fp8-nvfp4", kv_format="fp8-static", max_context=128)
    w, kv_scales = QM.load_resident(qm, cfg, "cpu")
    l0 = w.layers[0]
    assert (l0.qkv.kind, l0.o.kind, l0.gate_up.kind, l0.down.kind) == ("fp8", "fp8", "w4", "w4")
    base = f"{P}.layers.0."
    qkv = np.concatenate([dense[base + f"self_attn.{x}_proj"] for x in "qkv"], axis=0)
    got = l0.qkv.dequantized().float().numpy()
    assert np.abs(got - qkv).max() <= 0.07 * np.abs(qkv).max()            # channel scales -> 1x128 block scales (re-quantised)
    gu = np.concatenate([dense[base + f"mlp.{x}_proj"] for x in ("gate", "up")], axis=0)
    assert np.array_equal(l0.gate_up.w4.dequantized().float().numpy(), gu.astype(np.float32))   # codes and scales bit-exact
    assert kv_scales == [(0.0625, 0.03125), (0.125, 0.0625)]
    model = LlamaModel(cfg, w, None)
    cache = PagedKVCache(cfg, 32, torch.device("cpu"), kv_heads=model.local_kv_heads, static_scales=kv_scales)
    assert cache.layer(1).k_static == 0.125 and cache.layer(0).v_static == 0.03125
    eng = Engine(cfg, model, cache, torch.device("cpu"), max_batch=2, use_cuda_graphs=False)
    prompt = list(range(5, 40))
    out = eng.generate([prompt], 6)[0]
    assert len(out) == 6 and eng.generate([prompt + out[:3]], 3)[0] == out[3:]
    with pytest.raises(ValueError):
        PagedKVCache(cfg, 8, torch.device("cpu"), static_scales=[(1.0, 1.0)])


def test_converter_writes_a_servable_gguf(tmp_path, capsys):
    """`sllm-convert-gguf --kind mixed-precision`: lock-verified source -> GGUF with FP8 block-scaled attention, NVFP4
    type-40 MLP tensors and the per-layer KV scales in the configuration; loading it reproduces the generation."""
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.cli import convert
    from sllm_b200.engine.engine import Engine
    from sllm_b200.formats import gguf as G
    from sllm_b200.formats import model_lock as ML
    from sllm_b200.models import loader
    from sllm_b200.models.llama import LlamaModel
    src = tmp_path / "src"
    src.mkdir()
    _write_checkpoint(src)
    cfg_doc = json.loads((src / "config.json").read_bytes())
    cfg_doc.update({"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
                    "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 256, "vocab_size": 320,
                    "max_position_embeddings": 128})
    (src / "config.json").write_text(json.dumps(cfg_doc))
    lock = ML.make_model_lock(str(src), "local/tiny-mixed", "0" * 40, ["tiny-mixed"], {"family": "llama"}, {"kind": "none"})
    (tmp_path / "lock.json").write_text(json.dumps(lock))
    out, dl = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    rc = convert.main(["--kind", "mixed-precision", "--lock", str(tmp_path / "lock.json"), "--cache", str(src),
                       "--output", out, "--derived-lock", dl])
    assert rc == 0
    event = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert event["written"] and event["recipe"]["mlp_weight"] == "nvfp4-e2m1-block16-e4m3fn-f32-outer"
    assert event["recipe_digest"].startswith("sha256:")
    g = G.verify_gguf(out, G.read_derived_lock(dl))
    types = {g.tensors["blk.0.ffn_down.weight"].ttype, g.tensors["blk.0.attn_q.weight"].ttype}
    assert types == {G.T_NVFP4, G.T_I8}
    cfg, w = loader.load_llama_gguf(g, "cpu")
    assert cfg.kv_format == "fp8-static" and cfg.kv_static_scales == [[0.0625, 0.03125], [0.125, 0.0625]]
    m = LlamaModel(cfg, w, None)
    cache = PagedKVCache(cfg, 32, torch.device("cpu"), kv_heads=m.local_kv_heads)
    assert cache.layer(1).k_static == 0.125
    eng = Engine(cfg, m, cache, torch.device("cpu"), max_batch=2, use_cuda_graphs=False)
    qm = QM.open_mixed_precision_checkpoint(str(src), GEO)
    w0, kv0 = QM.load_resident(qm, cfg, "cpu")
    m0 = LlamaModel(cfg, w0, None)
    e0 = Engine(cfg, m0, PagedKVCache(cfg, 32, torch.device("cpu"), kv_heads=2, static_scales=kv0), torch.device("cpu"),
                max_batch=2, use_cuda_graphs=False)
    prompt = list(range(5, 30))
    assert eng.generate([prompt], 5) == e0.generate([prompt], 5)
