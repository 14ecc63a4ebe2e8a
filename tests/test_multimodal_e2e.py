"""Images end to end on the CPU oracle path: converter --with-vision, `sllm generate --image`, HTTP image parts."""
import base64
import io
import json

import numpy as np
import pytest
import torch

from sllm_b200.cli import common, convert, main as sllm
from sllm_b200.frontend import vision as V
from sllm_b200.models import vision_tower as VT


def _png(seed=0, h=70, w=90) -> bytes:
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray((np.random.default_rng(seed).random((h, w, 3)) * 255).astype(np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d = tmp_path_factory.mktemp("mm")
    g, l = str(d / "mm.gguf"), str(d / "mm.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-llama", "--weight-format", "fp32", "--with-vision", "tiny",
                         "--output", g, "--derived-lock", l]) == 0
    img = d / "a.png"
    img.write_bytes(_png())
    return g, l, str(img)


def _open(model):
    import argparse
    a = argparse.Namespace(gguf=model[0], derived_lock=model[1], device_index=0, target=common.TARGET, kv_cache_encoding=None,
                           context_length=None, cpu=True)
    return common.open_model(a, max_batch=4)


def test_file_carries_tower_and_sections(model):
    eng, tok, g, lock = _open(model)
    assert eng.vision is not None and eng.cfg.mrope_sections == [8, 12] and eng.cfg.image_token_id == eng.cfg.vocab - 1
    assert eng.vision.w.tensor_count() == 3 + 12 * 2 + 6 and eng.vision.cfg.out_hidden == eng.cfg.d_model
    want = VT.init_random_vision_weights(VT.VisionConfig(**eng.cfg.vision), "cpu", seed=2, dtype=torch.float32)
    assert torch.equal(eng.vision.w.blocks[1].qkv.w, want.blocks[1].qkv.w)
    assert torch.equal(eng.vision.w.merger_fc2_b, want.merger_fc2_b)


def _direct(model, text, images, n):
    """Reference: the engine driven by hand."""
    eng, tok, _, _ = _open(model)
    tok_id = eng.cfg.image_token_id
    mm = VT.MultimodalPrompt(eng.vision, V.process_many(images), VT.encode_with_images(tok, text, tok_id), tok_id)
    embeds, pos3 = mm(eng)
    s = eng.new_sequence(mm.tokens)
    out = [int(eng.prefill([s], sample=False, embeds=embeds, rope_pos3=pos3).argmax(-1)[0])]
    s.tokens.append(out[0])
    while len(out) < n:
        t = eng.decode([s])[0]
        s.tokens.append(t)
        out.append(t)
    return out, len(mm.tokens)


def test_cli_generate_with_image(capsys, model):
    capsys.readouterr()
    rc = sllm.main(["generate", "--gguf", model[0], "--derived-lock", model[1], "--cpu", "--prompt", "what is this",
                    "--image", model[2], "--max-new-tokens", "6"])
    out = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.strip()]
    assert rc == 0 and len(out[0]["tokens"]) == 6
    from sllm_b200.frontend.chat import ChatMessage, render_chatml
    text = render_chatml([ChatMessage("user", "<|vision_start|><|image_pad|><|vision_end|>what is this")], thinking="disabled")
    want, n_prompt = _direct(model, text, [V.BoundedImage.from_local_path(model[2])], 6)
    assert out[0]["tokens"] == want and out[0]["usage"]["prompt_tokens"] == n_prompt
    # without an image the same prompt gives other tokens (the visual rows matter) and a file without a tower refuses
    capsys.readouterr()
    assert sllm.main(["generate", "--gguf", model[0], "--derived-lock", model[1], "--cpu", "--prompt", "what is this",
                      "--max-new-tokens", "6"]) == 0
    plain = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert plain["usage"]["prompt_tokens"] < n_prompt


def test_http_image_part(model):
    from fastapi.testclient import TestClient
    from sllm_b200.server.app import ModelRegistry, ServerConfig, build_app
    from sllm_b200.server.backend import EngineBackend
    eng, tok, _, _ = _open(model)
    backend = EngineBackend(eng, tok, aliases=("mm",), queue_capacity=8)
    try:
        c = TestClient(build_app(ModelRegistry({"mm": backend}), ServerConfig()))
        assert backend.props()["vision"] is True
        url = "data:image/png;base64," + base64.b64encode(_png()).decode()
        body = {"model": "mm", "max_completion_tokens": 5, "temperature": 0,
                "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}},
                                                          {"type": "text", "text": "what is this"}]}]}
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        u = r.json()["usage"]
        p = V.process_image(V.BoundedImage.from_bytes(_png()))
        assert u["completion_tokens"] == 5 and u["prompt_tokens"] > p.visual_tokens
        # two different images in one request
        url2 = "data:image/png;base64," + base64.b64encode(_png(seed=1, h=40, w=40)).decode()
        body["messages"][0]["content"].insert(1, {"type": "image_url", "image_url": {"url": url2}})
        assert c.post("/v1/chat/completions", json=body).status_code == 200
    finally:
        backend.shutdown(5.0)
