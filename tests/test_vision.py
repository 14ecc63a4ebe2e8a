"""Vision preprocessing: bounded decode, smart resize, patch order, limits (CPU)."""
import base64
import io

import numpy as np
import pytest

from sllm_b200.frontend import vision as V

PIL = pytest.importorskip("PIL.Image")


def _png(w, h, seed=0):
    rng = np.random.default_rng(seed)
    arr = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    buf = io.BytesIO()
    PIL.fromarray(arr).save(buf, format="PNG")
    return buf.getvalue(), arr


def test_smart_resize_rules():
    assert V.smart_resize(512, 512) == (512, 512)
    assert V.smart_resize(500, 700) == (512, 704)
    assert V.smart_resize(48, 48) == (256, 256)                       # raised to the minimum area
    h, w = V.smart_resize(6000, 6000)
    assert h * w <= V.MAX_IMAGE_PIXELS and h % 32 == 0 and w % 32 == 0
    with pytest.raises(V.VisionError):
        V.smart_resize(10, 5000)


def test_patch_order_matches_loop_oracle():
    data, arr = _png(64, 96, 1)
    img = V.BoundedImage.from_bytes(data)
    assert img.mime == "image/png"
    p = V.process_image(img)
    assert (p.resized_height, p.resized_width) == (256, 256) or p.resized_height % 32 == 0
    gh, gw = p.grid_thw[1:]
    assert p.patches.shape == (gh * gw, 1536) and p.visual_tokens == gh * gw // 4 == len(p.merged_positions)
    resized = np.asarray(PIL.fromarray(arr).resize((p.resized_width, p.resized_height), PIL.BICUBIC), dtype=np.uint8)
    out = []
    for br in range(gh // 2):                      # the reference's loop nest, restated
        for bc in range(gw // 2):
            for mr in range(2):
                for mc in range(2):
                    for ch in range(3):
                        for _t in range(2):
                            for pr in range(16):
                                for pc in range(16):
                                    y, x = (br * 2 + mr) * 16 + pr, (bc * 2 + mc) * 16 + pc
                                    out.append((np.float32(resized[y, x, ch]) / np.float32(255) - np.float32(0.5)) / np.float32(0.5))
            if br == 0 and bc == 1:
                break
        break
    want = np.array(out, dtype=np.float32)
    assert np.array_equal(p.patches.reshape(-1)[:want.size], want)
    assert p.patch_sha256 == V.process_image(img).patch_sha256          # deterministic


def test_input_forms_and_limits(tmp_path):
    data, _ = _png(40, 40)
    url = "data:image/png;base64," + base64.b64encode(data).decode()
    assert V.BoundedImage.from_data_url(url).sha256 == V.BoundedImage.from_bytes(data).sha256
    with pytest.raises(V.VisionError, match="MIME"):
        V.BoundedImage.from_data_url("data:image/jpeg;base64," + base64.b64encode(data).decode())
    with pytest.raises(V.VisionError):
        V.BoundedImage.from_data_url("data:image/png;base64," + base64.b64encode(data).decode() + "=")
    with pytest.raises(V.VisionError):
        V.BoundedImage.from_data_url("http://example.com/x.png")
    with pytest.raises(V.VisionError, match="unsupported"):
        V.BoundedImage.from_bytes(b"BM" + b"\0" * 64)
    with pytest.raises(V.VisionError, match="malformed"):
        V.BoundedImage.from_bytes(data[:40]).decode_rgb()
    f = tmp_path / "a.png"
    f.write_bytes(data)
    imgs = [V.BoundedImage.from_local_path(str(f))] * 3
    with pytest.raises(V.VisionError, match="too many"):
        V.process_many(imgs)
    assert len(V.process_many(imgs[:2])) == 2
    frames = [PIL.fromarray(np.zeros((32, 32, 3), dtype=np.uint8)), PIL.fromarray(np.ones((32, 32, 3), dtype=np.uint8))]
    buf = io.BytesIO()
    frames[0].save(buf, format="GIF", save_all=True, append_images=frames[1:])
    with pytest.raises(V.VisionError, match="animated"):
        V.BoundedImage.from_bytes(buf.getvalue()).decode_rgb()


def test_mrope_positions():
    pos = V.mrope_positions(3, (1, 4, 6), 2)
    assert pos.shape == (3, 3 + 6 + 2)
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3
    assert pos[0, 3:9].tolist() == [3] * 6 and pos[1, 3:9].tolist() == [3, 3, 3, 4, 4, 4] and pos[2, 3:9].tolist() == [3, 4, 5, 3, 4, 5]
    assert pos[:, 9:].tolist() == [[6, 7]] * 3
