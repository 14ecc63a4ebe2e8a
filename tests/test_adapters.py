"""LoRA adapters and control vectors: lock parsing, oracle, and effect on the CPU model."""
import json

import pytest
import torch

from sllm_b200.engine.engine import build_engine
from sllm_b200.models import adapters as AD
from sllm_b200.models import config as MC


def test_lock_roundtrip_oracle_and_rejections(tmp_path):
    torch.manual_seed(0)
    a, b = torch.randn(4, 32) * 0.1, torch.randn(48, 4) * 0.1
    lp = AD.write_lora(str(tmp_path), "style", 8.0, [(0, "qkv", a, b)])
    ad = AD.load_lora(lp)
    t = ad.targets[(0, "qkv")]
    assert t.rank == 4 and t.in_features == 32 and t.out_features == 48
    x, y = torch.randn(32).bfloat16(), torch.randn(48).bfloat16()
    eff = ad.effective_scale(t.rank, 0.5)
    assert eff == 0.5 * 8.0 / 4
    got = AD.apply_lora_oracle(t, x, y, eff)
    want = (y.float() + eff * (t.b.float() @ (t.a.float() @ x.float()))).bfloat16()
    assert torch.allclose(got.float(), want.float(), atol=2e-2)
    # batched execution path equals the oracle row by row
    s = AD.AdapterSet([(ad, 0.5)])
    xs, ys = torch.randn(3, 32).bfloat16(), torch.randn(3, 48).bfloat16()
    out = s.lora_delta(0, "qkv", xs, ys)
    for i in range(3):
        assert torch.allclose(out[i].float(), AD.apply_lora_oracle(t, xs[i], ys[i], eff).float(), atol=2e-2)
    assert torch.equal(s.lora_delta(1, "qkv", xs, ys), ys)            # no target for that layer
    v = torch.randn(2, 16)
    cv = AD.load_control_vector(AD.write_control_vector(str(tmp_path), "calm", 1, v))
    h = torch.randn(16).bfloat16()
    assert torch.equal(AD.apply_control_vector_oracle(cv, h, 2, 2.0), (h.float() + 2.0 * cv.vectors[1].float()).bfloat16())
    with pytest.raises(AD.AdapterError):
        AD.apply_control_vector_oracle(cv, h, 0, 1.0)
    for bad_scale in (float("nan"), float("inf"), 100.0):
        with pytest.raises(AD.AdapterError):
            AD.AdapterSet([(ad, bad_scale)])
    # tampered payload, unknown field, out-of-range offsets
    blob = tmp_path / "style.lora.bin"
    raw = bytearray(blob.read_bytes()); raw[0] ^= 1; blob.write_bytes(bytes(raw))
    with pytest.raises(AD.AdapterError, match="digest"):
        AD.load_lora(lp)
    raw[0] ^= 1; blob.write_bytes(bytes(raw))
    d = json.loads(open(lp).read())
    d["extra"] = 1
    (tmp_path / "x.json").write_text(json.dumps(d))
    with pytest.raises(AD.AdapterError):
        AD.load_lora(str(tmp_path / "x.json"), str(blob))
    d.pop("extra"); d["targets"][0]["b_offset"] = 10 ** 9
    (tmp_path / "y.json").write_text(json.dumps(d))
    with pytest.raises(AD.AdapterError, match="outside"):
        AD.load_lora(str(tmp_path / "y.json"), str(blob))


def test_adapters_change_the_model_and_zero_scale_does_not(tmp_path):
    cfg = MC.tiny_llama()
    eng = build_engine(cfg, "cpu", seed=1, num_pages=64, max_batch=2, use_cuda_graphs=False)
    prompt = list(range(5, 25))
    s0 = eng.new_sequence(prompt)
    base = eng.prefill([s0], sample=False)
    eng.free_sequence(s0)
    torch.manual_seed(1)
    d = cfg.d_model
    qkv_out = cfg.q_size + 2 * cfg.kv_size
    ad = AD.load_lora(AD.write_lora(str(tmp_path), "l", 16.0, [(0, "qkv", torch.randn(8, d), torch.randn(qkv_out, 8)),
                                                              (1, "down", torch.randn(8, cfg.ffn), torch.randn(d, 8))]))
    cv = AD.load_control_vector(AD.write_control_vector(str(tmp_path), "c", 0, torch.randn(2, d)))
    for scale, changed in ((0.0, False), (1.0, True)):
        eng.model.adapters = AD.AdapterSet([(ad, scale)], [(cv, scale)])
        s = eng.new_sequence(prompt)
        out = eng.prefill([s], sample=False)
        eng.free_sequence(s)
        assert (not torch.allclose(out, base, atol=1e-3)) == changed
    eng.model.adapters = None
