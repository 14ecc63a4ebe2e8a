"""Vision tower: numerics against the fp32 oracle, tensor inventory, multimodal prompt assembly."""
import numpy as np
import pytest
import torch

from sllm_b200.frontend import vision as V
from sllm_b200.models import vision_tower as VT


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_inventory_matches_the_297_tensor_manifest():
    cfg = VT.VisionConfig()
    assert cfg.patch_dim == 1536 and cfg.head_dim == 64
    w = VT.init_random_vision_weights(VT.tiny_vision(), "cpu", dtype=torch.float32)
    assert w.tensor_count() == 3 + 12 * 2 + 6
    assert 3 + 12 * cfg.depth + 6 == 297


@pytest.mark.parametrize("grid", [(1, 4, 6), (1, 8, 2), (2, 4, 4)])
def test_forward_matches_oracle_cpu(grid):
    cfg = VT.tiny_vision()
    w = VT.init_random_vision_weights(cfg, "cpu", seed=3, dtype=torch.float32)
    n = grid[0] * grid[1] * grid[2]
    patches = torch.randn(n, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    got = VT.VisionTower(cfg, w).forward(patches, grid)
    want = VT.reference_forward(cfg, w, patches, grid)
    assert got.shape == (n // 4, cfg.out_hidden)
    assert _rel(got, want) < 1e-4


def test_patch_order_matches_preprocessor():
    """The tower's (row, column) of patch p is where the preprocessor took patch p from."""
    gh, gw = 4, 6
    img = np.zeros((gh * 16, gw * 16, 3), dtype=np.float32)
    for r in range(gh):
        for c in range(gw):
            img[r * 16:(r + 1) * 16, c * 16:(c + 1) * 16] = r * 100 + c
    x = img.reshape(gh // 2, 2, 16, gw // 2, 2, 16, 3).transpose(0, 3, 1, 4, 6, 2, 5).reshape(gh * gw, -1)
    rows, cols = VT.patch_rows_cols((1, gh, gw), 2)
    assert np.array_equal(x[:, 0], rows * 100 + cols)


def test_attention_is_not_causal_and_images_are_independent():
    cfg = VT.tiny_vision()
    w = VT.init_random_vision_weights(cfg, "cpu", seed=3, dtype=torch.float32)
    tower = VT.VisionTower(cfg, w)
    g = torch.Generator().manual_seed(2)
    a = torch.randn(16, cfg.patch_dim, generator=g)
    b = a.clone()
    b[-1] += 1.0                               # the last patch changes: the first merged row must change too
    ya, yb = tower.forward(a, (1, 4, 4)), tower.forward(b, (1, 4, 4))
    assert not torch.allclose(ya[0], yb[0])


def test_assemble_multimodal_positions_and_rows():
    d, img_tok = 8, 99
    g1, g2 = (1, 4, 6), (1, 2, 2)
    n1, n2 = 6, 1
    tokens = [1, 2, 3] + [img_tok] * n1 + [4, 5] + [img_tok] * n2 + [6]
    emb = torch.arange(len(tokens) * d, dtype=torch.float32).view(len(tokens), d)
    r1, r2 = torch.full((n1, d), -1.0), torch.full((n2, d), -2.0)
    out, pos = VT.assemble_multimodal(tokens, img_tok, emb, [(r1, g1), (r2, g2)])
    assert torch.equal(out[3:9], r1) and torch.equal(out[11:12], r2) and torch.equal(out[:3], emb[:3])
    # a single image agrees with the preprocessor's own helper
    want = V.mrope_positions(3, g1, 2)
    assert np.array_equal(pos[:, :11], want)
    # the second image starts after the text that followed the first
    assert pos[:, 11].tolist() == [want[0, -1] + 1] * 3
    assert pos[:, 12].tolist() == [want[0, -1] + 2] * 3
    with pytest.raises(ValueError):
        VT.assemble_multimodal(tokens, img_tok, emb, [(r1, g1)])
    with pytest.raises(ValueError):
        VT.assemble_multimodal(tokens, img_tok, emb, [(r2, g2), (r1, g1)])


def test_end_to_end_from_image_bytes():
    import io
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray((np.random.default_rng(0).random((70, 90, 3)) * 255).astype(np.uint8)).save(buf, format="PNG")
    p = V.process_image(V.BoundedImage.from_bytes(buf.getvalue()))
    cfg = VT.tiny_vision()
    w = VT.init_random_vision_weights(cfg, "cpu", seed=1, dtype=torch.float32)
    rows = VT.VisionTower(cfg, w).forward(torch.from_numpy(p.patches), p.grid_thw)
    assert rows.shape == (p.visual_tokens, cfg.out_hidden) and torch.isfinite(rows).all()


@pytest.mark.gpu
def test_forward_matches_oracle_gpu():
    cfg = VT.VisionConfig(depth=2, hidden=256, heads=4, intermediate=512, out_hidden=512, position_grid=8)
    w = VT.init_random_vision_weights(cfg, "cuda", seed=3)
    grid = (1, 8, 12)
    patches = torch.randn(96, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    got = VT.VisionTower(cfg, w).forward(patches.cuda(), grid)
    want = VT.reference_forward(cfg, w, patches.bfloat16().float(), grid)
    assert _rel(got, want) < 3e-2


# ------------------------------------------------------------------ multi-axis rotary positions and the engine
def _mm_engine(dev="cpu"):
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as mc
    cfg = mc.tiny_llama()
    cfg.max_context = 256
    cfg.mrope_sections = [8, 12]               # 32 rotary pairs: 8 temporal, 12 height, 12 width
    if dev != "cpu":
        cfg.weight_format, cfg.kv_format = "bf16", "bf16"
    return build_engine(cfg, dev, seed=0, max_batch=4, use_cuda_graphs=dev != "cpu")


def test_mrope_reference_sections():
    from sllm_b200.ops import reference as ref
    x = torch.randn(5, 2, 64, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([3, 4, 5, 6, 7], dtype=torch.int32)
    same = ref.rope_split_half(x, pos, 10000.0, 64, None, pos.unsqueeze(0).expand(3, -1), (8, 12))
    assert torch.allclose(same, ref.rope_split_half(x, pos, 10000.0, 64))
    p3 = torch.stack([pos, pos * 0 + 1, pos * 0 + 9]).int()
    got = ref.rope_split_half(x, pos, 10000.0, 64, None, p3, (8, 12))
    t_only = ref.rope_split_half(x, p3[0], 10000.0, 64)
    h_only = ref.rope_split_half(x, p3[1], 10000.0, 64)
    w_only = ref.rope_split_half(x, p3[2], 10000.0, 64)
    for lo, hi, want in ((0, 8, t_only), (8, 20, h_only), (20, 32, w_only)):
        assert torch.allclose(got[..., lo:hi], want[..., lo:hi]) and torch.allclose(got[..., 32 + lo:32 + hi], want[..., 32 + lo:32 + hi])


def _multimodal_logits(dev):
    """(logits after a one-shot multimodal prefill of prompt + 3 forced tokens,
        logits after prefilling the prompt and decoding the same 3 tokens one by one)."""
    from sllm_b200 import ops
    img_tok, grid = 1000, (1, 4, 6)
    n_img = 6
    base = [5, 6, 7] + [img_tok] * n_img + [8, 9]
    forced = [11, 12, 13]
    outs = []
    for one_shot in (True, False):
        eng = _mm_engine(dev)
        d = eng.cfg.d_model
        rows = torch.randn(n_img, d, generator=torch.Generator().manual_seed(4)).to(eng.device)
        toks = base + (forced if one_shot else [])
        emb = ops.embedding(eng.model.w.embed, torch.tensor(toks, dtype=torch.int32, device=eng.device), 1.0)
        embeds, pos3 = VT.assemble_multimodal(toks, img_tok, emb, [(rows.to(emb.dtype), grid)])
        s = eng.new_sequence(toks)
        lg = eng.prefill([s], sample=False, embeds=embeds, rope_pos3=torch.from_numpy(pos3))
        assert s.rope_delta == int(pos3.max()) + 1 - len(toks) and s.rope_delta < 0
        if not one_shot:
            for t in forced:
                s.tokens.append(t)
                lg = eng.decode([s], sample=False)
        outs.append(lg.float().cpu().clone())
    return outs


def test_multimodal_prefill_then_decode_matches_one_shot_cpu():
    a, b = _multimodal_logits("cpu")
    assert _rel(b, a) < 1e-4


def test_text_only_through_the_multimodal_entry_is_unchanged():
    from sllm_b200 import ops
    toks = list(range(3, 20))
    eng = _mm_engine()
    want = eng.prefill([eng.new_sequence(toks)], sample=False).clone()
    eng2 = _mm_engine()
    emb = ops.embedding(eng2.model.w.embed, torch.tensor(toks, dtype=torch.int32), 1.0)
    embeds, pos3 = VT.assemble_multimodal(toks, 1000, emb, [])
    s = eng2.new_sequence(toks)
    got = eng2.prefill([s], sample=False, embeds=embeds, rope_pos3=torch.from_numpy(pos3))
    assert s.rope_delta == 0 and torch.allclose(got, want, atol=1e-5)


@pytest.mark.gpu
def test_multimodal_prefill_then_decode_matches_one_shot_gpu():
    a, b = _multimodal_logits("cuda")
    assert _rel(b, a) < 3e-2


@pytest.mark.gpu
def test_mrope_kernel_matches_reference():
    from sllm_b200 import ops
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.models import config as mc
    from sllm_b200.ops import reference as ref
    cfg = mc.tiny_llama()
    cfg.weight_format, cfg.kv_format = "bf16", "bf16"
    t, hq, hkv, hd = 7, 4, 2, 64
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0)).bfloat16()
    pos = torch.arange(t, dtype=torch.int32, device="cuda")
    p3 = torch.stack([pos // 2, pos % 3 + 1, 6 - pos]).int().contiguous()
    cache = PagedKVCache(cfg, 8, "cuda", kv_heads=hkv)
    table = torch.arange(4, dtype=torch.int32, device="cuda").view(1, 4)
    sidx = torch.zeros(t, dtype=torch.int32, device="cuda")
    want_q = ref.rope_split_half(qkv.float().view(t, hq + 2 * hkv, hd)[:, :hq].cpu(), pos.cpu(), cfg.rope_theta, hd, None,
                                 p3.cpu(), (8, 12))
    q = ops.rope_kv_append(qkv.clone(), pos, sidx, table, cache.layer(0), hq, hkv, hd, cfg.rope_theta, None,
                           rope_pos3=p3, mrope_sections=(8, 12))
    assert _rel(q.view(t, hq, hd), want_q) < 1e-2
