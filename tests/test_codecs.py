"""Host codecs: exhaustive / boundary checks of the quantised encodings (CPU only)."""
import numpy as np
import pytest
import torch

from sllm_b200.formats import codecs as c


def test_e4m3_roundtrip_all_codes():
    codes = np.arange(256, dtype=np.uint8)
    vals = c.decode_e4m3fn(codes)
    back = c.encode_e4m3fn(vals)
    for b in range(256):
        if b in (0x7F, 0xFF):
            assert back[b] == 0x7F
        elif b == 0x80:
            assert back[b] in (0x00, 0x80)
        else:
            assert back[b] == b, (b, vals[b], back[b])


def test_e4m3_matches_torch_and_special_values():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 50, 20000), rng.normal(0, 0.01, 20000), [448, 449, 1e9, -1e9, 0.0, -0.0]])
    x = x.astype(np.float32)
    ours = c.encode_e4m3fn(x)
    ref = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    same = (ours == ref) | ((ours & 0x7F) == 0) & ((ref & 0x7F) == 0)
    assert same.all(), np.nonzero(~same)[0][:5]
    assert c.encode_e4m3fn(np.array([np.nan, np.inf, -np.inf], dtype=np.float32)).tolist() == [0x7F, 0x7E, 0xFE]
    # ties go to the even code: 0.5*(v[i]+v[i+1]) -> even of the two
    v = c.decode_e4m3fn(np.arange(0x7E, dtype=np.uint8)).astype(np.float64)
    mid = ((v[:-1] + v[1:]) / 2).astype(np.float32)
    enc = c.encode_e4m3fn(mid)
    exact = ((v[:-1] + v[1:]) / 2) == mid.astype(np.float64)
    assert ((enc[exact] & 1) == 0).all()


def test_e2m1_codes_and_ties():
    assert c.decode_e2m1(np.arange(16, dtype=np.uint8)).tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -5.0], dtype=np.float32)
    assert c.encode_e2m1(x).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 0, 8 | 6]


def test_e8m0_and_even_scale():
    assert c.decode_e8m0(np.array([127, 128, 0], dtype=np.uint8)).tolist()[:2] == [1.0, 2.0]
    assert c.decode_e8m0(np.array([0], dtype=np.uint8))[0] == np.float32(2.0 ** -127)
    with pytest.raises(ValueError):
        c.decode_e8m0(np.array([255], dtype=np.uint8))
    # amax 6 -> exponent 2 -> code 127; 7 rounds up at the 1.75 boundary -> exponent 3 -> code 128
    assert c.encode_e8m0_for_amax(np.array([6.0, 6.9, 7.0, 0.0, 1.0], dtype=np.float32)).tolist() == [127, 127, 128, 0, 125]


def test_fp8_block_quant_roundtrip():
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.02, (7, 300)).astype(np.float32)
    w[3] = 0
    q, s = c.quantize_fp8_k_blocks(w)
    assert s.shape == (7, 3) and (s[3] == 1.0).all()
    d = c.dequantize_fp8_k_blocks(q, s)
    assert np.abs(d - w).max() <= np.abs(w).max() * 0.07
    qo, so = c.quantize_fp8_outer_rows(w)
    assert np.abs(c.dequantize_fp8_outer_rows(qo, so) - w).max() <= np.abs(w).max() * 0.07
    # agreement with the torch restatement used as the kernel oracle
    from sllm_b200.ops import reference as ref
    tq, ts = ref.quant_fp8_1x128(torch.from_numpy(w))
    assert np.array_equal(tq.numpy(), q) and np.allclose(ts.t().numpy(), s, rtol=1e-6)


def test_nvfp4_and_mxfp4_roundtrip():
    rng = np.random.default_rng(2)
    w = rng.normal(0, 0.05, (5, 70)).astype(np.float32)
    w[2, 16:32] = 0  # zero block -> zero scale byte -> zero codes
    p, bs, ts = c.quantize_nvfp4(w)
    assert p.shape == (5, 35) and bs.shape == (5, 5)
    assert bs[2, 1] == 0 and (c.unpack_nibbles(p, 70)[2, 16:32] == 0).all()
    d = c.dequantize_nvfp4(p, bs, ts, 70)
    assert np.abs(d - w).max() <= np.abs(w).max() * 0.3
    assert abs(float(ts) - np.abs(w).max() / (448 * 6)) < 1e-9
    pm, sm = c.quantize_mxfp4(w)
    dm = c.dequantize_mxfp4(pm, sm, 70)
    assert np.abs(dm - w).max() <= np.abs(w).max() * 0.3
    # low nibble = even index
    codes = np.array([[1, 2, 3]], dtype=np.uint8)
    assert c.pack_nibbles(codes).tolist() == [[0x21, 0x03]]


def test_fnuz_table_and_bf16_rounding():
    t = c.fn_to_fnuz_table()
    assert t[0x7F] == 0x80 and t[0x80] == 0x00
    v = c.decode_e4m3fn(np.arange(256, dtype=np.uint8))
    u = c.decode_e4m3fnuz(t)
    ok = ~np.isnan(v) & (np.abs(v) <= 240)
    assert np.allclose(u[ok], v[ok], rtol=0.07, atol=2 ** -10)
    x = np.array([1.0, 1.00390625, 1.01171875, np.nan], dtype=np.float32)
    r = c.round_bf16(x)
    want = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(r[:3], want[:3]) and np.isnan(r[3])


def test_kv_quantisers():
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (3, 2, 64)).astype(np.float32)
    q, s = c.quantize_kv_fp8(x)
    assert s.shape == (3, 2) and np.allclose(s, np.abs(x).max(-1) / 448)
    p, b, o = c.quantize_kv_nvfp4(x)
    assert p.shape == (3, 2, 32) and b.shape == (3, 2, 4) and o.shape == (3, 2)
