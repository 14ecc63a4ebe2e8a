"""Numerics of every CUDA kernel against a plain PyTorch fp32 restatement of the same op."""
import math

import numpy as np
import pytest
import torch

from sllm_b200 import ops
from sllm_b200.ops import reference as ref
from sllm_b200.ops.core import KVLayer, LinearWeight

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _status_ok():
    assert ops.device_status(torch.device(DEV)) == 0


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (16, 384, 1024), (17, 128, 448), (32, 4096, 4096), (64, 512, 256),
                                   (100, 640, 1024), (128, 256, 2048), (129, 512, 512), (300, 384, 1088),
                                   (512, 1024, 4096)])
def test_gemm_bf16(m, n, k):
    torch.manual_seed(m * 7 + n)
    x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    r = (torch.randn(m, n, device=DEV)).bfloat16()
    y = ops.linear(x, LinearWeight("dense", w))
    want = x.float() @ w.float().t()
    assert rel_err(y, want) < 6e-3
    y2 = ops.linear(x, LinearWeight("dense", w), residual=r)
    assert rel_err(y2, want + r.float()) < 6e-3
    _status_ok()


@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (8, 6144, 4096), (32, 4096, 4096), (33, 512, 1024), (64, 384, 2048),
                                   (128, 256, 14336), (200, 512, 1024), (1024, 1024, 4096)])
def test_gemm_fp8_blockscaled(m, n, k):
    torch.manual_seed(m + n + k)
    x = (torch.randn(m, k, device=DEV) * 2).bfloat16()
    x[:, :128] *= 30  # blocks with very different scales
    w = (torch.randn(n, k, device=DEV) * 0.02).bfloat16()
    lw = LinearWeight.from_dense(w.cpu(), "fp8").to(DEV)
    xq = ops.quant_fp8(x)
    xq_ref = ref.quant_fp8_1x128(x.cpu())
    assert torch.equal(xq.data.cpu(), xq_ref[0])
    assert torch.allclose(xq.scale.cpu(), xq_ref[1], rtol=1e-6, atol=0)
    y = ops.linear(xq, lw)
    want = ref.linear_fp8(xq_ref[0], xq_ref[1], lw.w.cpu(), lw.scale_t.cpu())
    assert rel_err(y.cpu(), want) < 6e-3
    # and close to the unquantised product
    assert rel_err(y.cpu(), x.float().cpu() @ w.float().cpu().t()) < 8e-2
    _status_ok()


def elementwise_close(got, want, rtol, atol_frac, what=""):
    """Every element: |got - want| <= rtol |want| + atol_frac max|want| (a wrong 16x8 unit or a mis-scaled tile edge
    fails here even when the norm of the whole output barely moves)."""
    got, want = got.float().cpu(), want.float().cpu()
    tol = rtol * want.abs() + atol_frac * want.abs().max()
    bad = (got - want).abs() > tol
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} elements off, first at {idx}: got {got[tuple(idx)].item():.5g} "
                             f"want {want[tuple(idx)].item():.5g}")


@pytest.mark.parametrize("scaled", [False, True])
@pytest.mark.parametrize("bn,m", [(16, 1), (16, 15), (16, 16), (32, 17), (32, 31), (32, 32), (64, 33), (64, 63), (64, 64),
                                  (128, 65), (128, 127), (128, 128)])
@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_gemm_swap_ab_tile_edges_per_element(scaled, bn, m, splits):
    """Small-M (swap-AB) tiles at every token-tile width, rows at the edges of the tile, weight rows at 127 / 128 / 129
    boundaries, every cluster split count: checked element by element against fp32."""
    torch.manual_seed(bn * 131 + m * 7 + splits)
    k = 1024
    for n in (128, 136, 264):                    # one full weight tile; one full + 8 rows; two full + 8 rows
        n_rows = n
        x = (torch.randn(m, k, device=DEV) * 0.7).bfloat16()
        w = (torch.randn(n_rows, k, device=DEV) * 0.05).bfloat16()
        w[-1] *= 8                                     # the last weight row carries a large, easy to misplace value
        x[-1] *= 4
        y = torch.full((m, n_rows), float("nan"), device=DEV, dtype=torch.bfloat16)
        if scaled:
            xq = ops.quant_fp8(x)
            lw = LinearWeight.from_dense(w.cpu(), "fp8").to(DEV)
            ops.gemm_raw(lw.w, xq.data, y, scale_a=lw.scale_t, scale_b=xq.scale, transpose_out=True, bn=bn, splits=splits,
                         stages=4 if bn <= 32 else 3)
            want = ref.linear_fp8(xq.data.cpu(), xq.scale.cpu(), lw.w.cpu(), lw.scale_t.cpu())
        else:
            ops.gemm_raw(w, x, y, transpose_out=True, bn=bn, splits=splits, stages=4 if bn <= 32 else 3)
            want = x.float() @ w.float().t()
        assert not torch.isnan(y.float()).any(), "an output element was never written"
        elementwise_close(y, want, 1.2e-2, 2e-3, f"n={n_rows}")
    _status_ok()


@pytest.mark.parametrize("m", [127, 128, 129, 255, 257])
@pytest.mark.parametrize("n", [128, 136, 264])
def test_gemm_large_m_row_edges_per_element(m, n):
    """The 128 x 128-tile path at 127 / 128 / 129 rows and ragged column counts (multiples of 8)."""
    torch.manual_seed(m + n)
    k = 512
    x = (torch.randn(m, k, device=DEV) * 0.7).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    x[-1] *= 4
    w[-1] *= 8
    y = ops.linear(x, LinearWeight("dense", w))
    elementwise_close(y, x.float() @ w.float().t(), 1.2e-2, 2e-3, "bf16")
    lw = LinearWeight.from_dense(w.cpu(), "fp8").to(DEV)
    xq = ops.quant_fp8(x)
    yq = ops.linear(xq, lw)
    elementwise_close(yq, ref.linear_fp8(xq.data.cpu(), xq.scale.cpu(), lw.w.cpu(), lw.scale_t.cpu()), 1.2e-2, 2e-3, "fp8")
    _status_ok()


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("splits", [1, 2, 4, 7, 8, 12])
def test_gemm_split_k_deterministic(splits, cluster):
    """Split-K through the cluster/DSMEM reduction (2..8 splits) and through the global fix-up."""
    from sllm_b200.ops import _lib
    _lib.kernels().sllm_gemm_set_cluster_split(int(cluster))
    try:
        _split_k_case(splits)
    finally:
        _lib.kernels().sllm_gemm_set_cluster_split(1)


def _split_k_case(splits):
    torch.manual_seed(0)
    m, n, k = 8, 512, 4096
    x = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.03).bfloat16()
    outs = []
    for _ in range(2):
        y = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
        ops.gemm_raw(w, x, y, transpose_out=True, bn=16, splits=splits, stages=4)
        outs.append(y.clone())
    assert torch.equal(outs[0], outs[1])
    assert rel_err(outs[0], x.float() @ w.float().t()) < 6e-3
    _status_ok()


@pytest.mark.parametrize("rows,d", [(1, 256), (5, 4096), (33, 2048), (3, 8192), (2, 2880)])
def test_rmsnorm(rows, d):
    torch.manual_seed(d)
    x = torch.randn(rows, d, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    for off in (False, True):
        y = ops.rmsnorm(x, w, 1e-5, offset_one=off)
        want = ref.rmsnorm(x.cpu(), w.cpu(), 1e-5, off)
        assert rel_err(y.cpu(), want) < 5e-3
    if d % 128 == 0:
        q = ops.rmsnorm(x, w, 1e-5, quant=True)
        want = ref.round_bf16(ref.rmsnorm(x.cpu(), w.cpu(), 1e-5))
        deq = ref.dequant_fp8_1x128(q.data.cpu(), q.scale.cpu())
        assert rel_err(deq, want) < 4e-2
        assert (deq - want).abs().max() <= want.abs().max() * 0.07


@pytest.mark.parametrize("rows,inter", [(1, 128), (7, 14336), (3, 688), (2, 1024)])
def test_gated_act(rows, inter):
    torch.manual_seed(inter)
    x = torch.randn(rows, 2 * inter, device=DEV).bfloat16()
    for act in ("silu", "gelu_tanh"):
        y = ops.gated_act(x, act)
        want = ref.gated_act(x.cpu(), act)
        assert rel_err(y.cpu(), want) < 6e-3
    if inter % 128 == 0:
        q = ops.gated_act(x, "silu", quant=True)
        deq = ref.dequant_fp8_1x128(q.data.cpu(), q.scale.cpu())
        assert rel_err(deq, ref.gated_act(x.cpu(), "silu")) < 4e-2


def test_quant_special_values():
    x = torch.zeros(2, 256, device=DEV, dtype=torch.bfloat16)
    x[0, 0] = float("nan")
    x[0, 1] = float("inf")
    x[0, 2] = 3.0
    x[1, 130] = -5.0
    q = ops.quant_fp8(x)
    qr = ref.quant_fp8_1x128(x.cpu())
    assert torch.equal(q.data.cpu(), qr[0])
    assert torch.allclose(q.scale.cpu(), qr[1])
    assert q.data[0, 0].item() == 0x7F and q.data[0, 1].item() == 0x7E
    assert q.scale[1, 0].item() == 1.0  # all-zero block


def _make_kv(num_pages, page, hkv, hd, fp8):
    if fp8:
        return KVLayer(torch.zeros(num_pages, hkv, page, hd, dtype=torch.uint8, device=DEV),
                       torch.zeros(num_pages, hkv, page, hd, dtype=torch.uint8, device=DEV),
                       torch.ones(num_pages, hkv, page, device=DEV), torch.ones(num_pages, hkv, page, device=DEV),
                       True, page)
    return KVLayer(torch.zeros(num_pages, hkv, page, hd, dtype=torch.bfloat16, device=DEV),
                   torch.zeros(num_pages, hkv, page, hd, dtype=torch.bfloat16, device=DEV), None, None, False, page)


def _cpu_kv(kv):
    c = lambda t: None if t is None else t.cpu().clone()
    return KVLayer(c(kv.k), c(kv.v), c(kv.k_scale), c(kv.v_scale), kv.fp8, kv.page_size)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("hq,hkv,hd,rd", [(4, 2, 64, 64), (32, 8, 128, 128), (8, 1, 128, 64), (16, 4, 256, 64)])
def test_rope_kv_append(fp8, hq, hkv, hd, rd):
    torch.manual_seed(hq)
    t, page, pages = 37, 16, 12
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device=DEV).bfloat16()
    pos = torch.randint(0, 4 * page, (t,), device=DEV, dtype=torch.int32)
    # distinct (seq, pos) pairs so no two tokens land on the same slot
    seq = (torch.arange(t, device=DEV) % 3).int()
    pos = (torch.arange(t, device=DEV) // 3 + 5).int()
    table = torch.randperm(pages, device=DEV).int().view(3, 4)
    kv = _make_kv(pages, page, hkv, hd, fp8)
    kvc = _cpu_kv(kv)
    q_ref = ops.rope_kv_append(qkv.cpu().clone(), pos.cpu(), seq.cpu(), table.cpu(), kvc, hq, hkv, hd, 10000.0, rd)
    q = ops.rope_kv_append(qkv.clone(), pos, seq, table, kv, hq, hkv, hd, 10000.0, rd)
    assert rel_err(q.cpu(), q_ref) < 5e-3
    if fp8:
        kd = ref.from_e4m3(kv.k.cpu()) * kv.k_scale.cpu().unsqueeze(-1)
        kr = ref.from_e4m3(kvc.k) * kvc.k_scale.unsqueeze(-1)
        vd = ref.from_e4m3(kv.v.cpu()) * kv.v_scale.cpu().unsqueeze(-1)
        vr = ref.from_e4m3(kvc.v) * kvc.v_scale.unsqueeze(-1)
        assert rel_err(kd, kr) < 3e-2 and rel_err(vd, vr) < 1e-6 + 3e-2
        assert torch.equal(kv.v.cpu(), kvc.v)  # V is not rotated: bit-exact
    else:
        assert rel_err(kv.k.cpu(), kvc.k) < 5e-3
        assert torch.equal(kv.v.cpu(), kvc.v)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("hq,hkv,hd,rd", [(16, 8, 256, 64), (8, 1, 512, 128), (4, 2, 128, 128)])
def test_rope_kv_append_proportional_pairs(fp8, hq, hkv, hd, rd):
    """Channel i < rd / 2 pairs with i + hd / 2, frequencies over hd; the channels between pass through."""
    torch.manual_seed(hd)
    t, page, pages = 29, 16, 12
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device=DEV).bfloat16()
    seq = (torch.arange(t, device=DEV) % 3).int()
    pos = (torch.arange(t, device=DEV) // 3 + 11).int()
    table = torch.randperm(pages, device=DEV).int().view(3, 4)
    kv = _make_kv(pages, page, hkv, hd, fp8)
    kvc = _cpu_kv(kv)
    q_ref = ops.rope_kv_append(qkv.cpu().clone(), pos.cpu(), seq.cpu(), table.cpu(), kvc, hq, hkv, hd, 1e6, rd,
                               pair_offset=hd // 2)
    q = ops.rope_kv_append(qkv.clone(), pos, seq, table, kv, hq, hkv, hd, 1e6, rd, pair_offset=hd // 2)
    assert rel_err(q.cpu(), q_ref) < 5e-3
    untouched = q.view(t, hq, hd)[:, :, rd // 2:hd // 2]
    assert torch.equal(untouched, qkv[:, :hq * hd].view(t, hq, hd)[:, :, rd // 2:hd // 2])
    if fp8:
        kd = ref.from_e4m3(kv.k.cpu()) * kv.k_scale.cpu().unsqueeze(-1)
        kr = ref.from_e4m3(kvc.k) * kvc.k_scale.unsqueeze(-1)
        assert rel_err(kd, kr) < 3e-2
    else:
        assert rel_err(kv.k.cpu(), kvc.k) < 5e-3
    assert torch.equal(kv.v.cpu(), kvc.v)


@pytest.mark.parametrize("qk,norm_v", [(True, True), (False, True), (True, False)])
def test_qkv_headnorm_value_heads(qk, norm_v):
    from sllm_b200.ops import gdn
    torch.manual_seed(3)
    t, hq, hkv, hd = 19, 8, 2, 256
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device=DEV).bfloat16() * 3
    wq = (torch.randn(hd, device=DEV) * 0.1).bfloat16() if qk else None
    wk = (torch.randn(hd, device=DEV) * 0.1).bfloat16() if qk else None
    c = lambda x: None if x is None else x.cpu()
    want = gdn.qk_headnorm(qkv.cpu().clone(), hq, hkv, hd, c(wq), c(wk), 1e-6, True, norm_v=norm_v)
    got = gdn.qk_headnorm(qkv.clone(), hq, hkv, hd, wq, wk, 1e-6, True, norm_v=norm_v)
    assert rel_err(got.cpu(), want) < 6e-3
    if not qk:
        assert torch.equal(got[:, :(hq + hkv) * hd], qkv[:, :(hq + hkv) * hd])
    if not norm_v:
        assert torch.equal(got[:, (hq + hkv) * hd:], qkv[:, (hq + hkv) * hd:])


@pytest.mark.parametrize("hq,hkv,hd", [(4, 2, 64), (32, 8, 128), (8, 1, 128), (16, 4, 256)])
def test_nvfp4_kv_append_and_attention(hq, hkv, hd):
    """NVFP4 KV rows written by the append kernel are bit-identical to the host codec's rows; attention over them
    matches the fp32 oracle that dequantises the same rows (full and windowed)."""
    torch.manual_seed(hd + hq)
    page, nseq, max_blocks = 16, 3, 12
    rowb = hd // 2 + hd // 16
    pages = nseq * max_blocks
    mk = lambda dev: KVLayer(torch.zeros(pages, hkv, page, rowb, dtype=torch.uint8, device=dev),
                             torch.zeros(pages, hkv, page, rowb, dtype=torch.uint8, device=dev),
                             torch.ones(pages, hkv, page, device=dev), torch.ones(pages, hkv, page, device=dev), False, page,
                             nvfp4=True)
    kv, kvc = mk(DEV), mk("cpu")
    lens = [1, 77, 150]
    table = torch.randperm(pages, device=DEV).int().view(nseq, max_blocks)
    # fill the caches through the append kernel, one chunk per sequence
    for sidx, n in enumerate(lens):
        qkv = (torch.randn(n, (hq + 2 * hkv) * hd, device=DEV) * 1.5).bfloat16()
        qkv[0, hq * hd + 5] = 40.0                                     # an outlier inside one block
        pos = torch.arange(n, device=DEV, dtype=torch.int32)
        seq = torch.full((n,), sidx, device=DEV, dtype=torch.int32)
        q_ref = ops.rope_kv_append(qkv.cpu().clone(), pos.cpu(), seq.cpu(), table.cpu(), kvc, hq, hkv, hd, 10000.0)
        q = ops.rope_kv_append(qkv.clone(), pos, seq, table, kv, hq, hkv, hd, 10000.0)
        assert rel_err(q.cpu(), q_ref) < 5e-3
    blk = table.cpu().long()
    for sidx, n in enumerate(lens):
        used = blk[sidx, :(n + page - 1) // page]
        got_v, want_v = kv.v.cpu()[used], kvc.v[used]
        assert torch.equal(got_v, want_v)                              # V is not rotated: identical codes and scales
        assert torch.equal(kv.v_scale.cpu()[used], kvc.v_scale[used])
        # K goes through sincos on the device: compare dequantised rows
        kd = ref.dequant_kv_nvfp4_rows(kv.k.cpu()[used], kv.k_scale.cpu()[used], hd)
        kr = ref.dequant_kv_nvfp4_rows(kvc.k[used], kvc.k_scale[used], hd)
        assert rel_err(kd, kr) < 4e-2
    rows = torch.tensor([0, 1, 1, 2, 2], device=DEV, dtype=torch.int32)
    kv_lens = torch.tensor([1, 30, 77, 100, 150], device=DEV, dtype=torch.int32)
    q = torch.randn(5, hq * hd, device=DEV).bfloat16()
    for window in (0, 40):
        got = ops.paged_attention(q, kv, table, rows, kv_lens, hq, hkv, hd, window=window)
        # oracle over the DEVICE-written rows, so that only the attention arithmetic is compared
        dev_rows = KVLayer(kv.k.cpu(), kv.v.cpu(), kv.k_scale.cpu(), kv.v_scale.cpu(), False, page, nvfp4=True)
        want = ops.paged_attention(q.cpu(), dev_rows, table.cpu(), rows.cpu(), kv_lens.cpu(), hq, hkv, hd, window=window)
        assert rel_err(got.cpu(), want) < 8e-3
    _status_ok()


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("hq,hkv,hd", [(4, 2, 64), (32, 8, 128), (64, 8, 64), (8, 8, 128), (16, 4, 256)])
@pytest.mark.parametrize("window", [0, 40])
def test_paged_attention(fp8, hq, hkv, hd, window):
    torch.manual_seed(hq + hd)
    page, nseq, max_blocks = 16, 3, 40
    lens = [1, 333, 600]
    pages = nseq * max_blocks
    table = torch.randperm(pages, device=DEV).int().view(nseq, max_blocks)
    kv = _make_kv(pages, page, hkv, hd, fp8)
    if fp8:
        kv.k.copy_(torch.randint(0, 0x78, kv.k.shape, device=DEV, dtype=torch.uint8) |
                   (torch.randint(0, 2, kv.k.shape, device=DEV, dtype=torch.uint8) << 7))
        kv.v.copy_(torch.randint(0, 0x78, kv.v.shape, device=DEV, dtype=torch.uint8) |
                   (torch.randint(0, 2, kv.v.shape, device=DEV, dtype=torch.uint8) << 7))
        kv.k_scale.copy_(torch.rand_like(kv.k_scale) * 0.01 + 0.001)
        kv.v_scale.copy_(torch.rand_like(kv.v_scale) * 0.01 + 0.001)
    else:
        kv.k.copy_(torch.randn(kv.k.shape, device=DEV))
        kv.v.copy_(torch.randn(kv.v.shape, device=DEV))
    # rows: one decode row per sequence + a 4-row verify block on the last sequence
    seq_index = torch.tensor([0, 1, 2, 2, 2, 2, 2], device=DEV, dtype=torch.int32)
    kv_lens = torch.tensor([lens[0], lens[1], lens[2], lens[2] - 1, lens[2] - 2, lens[2] - 3, 17], device=DEV,
                           dtype=torch.int32)
    q = torch.randn(len(seq_index), hq * hd, device=DEV).bfloat16()
    want = ops.paged_attention(q.cpu(), _cpu_kv(kv), table.cpu(), seq_index.cpu(), kv_lens.cpu(), hq, hkv, hd,
                               window=window)
    for max_kv in (64, 640, 8192):  # exercises 1, few and many KV splits
        got = ops.paged_attention(q, kv, table, seq_index, kv_lens, hq, hkv, hd, window=window, max_kv=max_kv,
                                  impl="cuda_core")
        assert rel_err(got.cpu(), want) < 8e-3, (max_kv, rel_err(got.cpu(), want))
        if fp8 and hd == 128:
            # tensor-core path: Q and P pass through E4M3, so the tolerance is that of FP8 attention
            got = ops.paged_attention(q, kv, table, seq_index, kv_lens, hq, hkv, hd, window=window, max_kv=max_kv,
                                      impl="tensor_core")
            assert rel_err(got.cpu(), want) < 6e-2, ("tc", max_kv, rel_err(got.cpu(), want))
            _status_ok()
    if hd == 128:
        gq = ops.paged_attention(q, kv, table, seq_index, kv_lens, hq, hkv, hd, window=window, max_kv=640,
                                 quant_out=True, impl="cuda_core")
        deq = ref.dequant_fp8_1x128(gq.data.cpu(), gq.scale.cpu())
        assert rel_err(deq, want) < 4e-2


def test_argmax():
    torch.manual_seed(3)
    lg = torch.randn(5, 128256, device=DEV).bfloat16()
    lg[1, 777] = 50
    lg[1, 90000] = 50  # tie -> lowest index
    lg[2, 5] = float("nan")
    idx = ops.argmax(lg)
    assert idx[1].item() == 777 and idx[2].item() == -1
    want = lg.float().cpu().argmax(-1)
    assert idx[0].item() == want[0].item() and idx[3].item() == want[3].item()


def test_embedding_and_elementwise():
    torch.manual_seed(0)
    tab = torch.randn(1000, 256, device=DEV).bfloat16()
    ids = torch.tensor([0, 999, 5, 5], device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embedding(tab, ids), tab[ids.long()])
    a = torch.randn(4, 256, device=DEV).bfloat16()
    b = torch.randn(4, 256, device=DEV).bfloat16()
    for op, s in (("add", 0.0), ("scalar_mul", 1.7), ("sigmoid_mul", 0.0), ("tanh_softcap", 30.0)):
        got = ops.elementwise(op, a, b, s)
        want = ops.elementwise(op, a.cpu(), b.cpu(), s)
        assert rel_err(got.cpu(), want) < 6e-3


@pytest.mark.parametrize("lens", [[128], [300, 128, 129], [1000, 257]])
@pytest.mark.parametrize("hq,hkv", [(4, 2), (8, 8), (4, 1)])
def test_prefill_attention_tcgen05(lens, hq, hkv):
    """Tensor-core causal prefill vs an fp32 dense-attention restatement."""
    from sllm_b200.engine.batch import make_prefill_batch
    from sllm_b200.ops import prefill
    torch.manual_seed(sum(lens) + hq)
    hd = 128
    t = sum(lens)
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device=DEV).bfloat16()
    table = torch.zeros((len(lens), 1), dtype=torch.int32, device=DEV)
    b = make_prefill_batch([[0] * n for n in lens], table, DEV)
    assert prefill.usable(qkv, b, hd, 0, None, qkv)
    out = prefill.prefill_attention(qkv, b, hq, hkv, hd)
    outq = prefill.prefill_attention(qkv, b, hq, hkv, hd, quant_out=True)
    x = qkv.float().cpu().view(t, hq + 2 * hkv, hd)
    g = hq // hkv
    want = torch.empty(t, hq, hd)
    t0 = 0
    for n in lens:
        q = x[t0:t0 + n, :hq]
        k = x[t0:t0 + n, hq:hq + hkv].repeat_interleave(g, dim=1)
        v = x[t0:t0 + n, hq + hkv:].repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
        want[t0:t0 + n] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v)
        t0 += n
    want = want.view(t, hq * hd)
    assert rel_err(out.cpu(), want) < 1e-2, rel_err(out.cpu(), want)
    deq = ref.dequant_fp8_1x128(outq.data.cpu(), outq.scale.cpu())
    assert rel_err(deq, want) < 4e-2
    _status_ok()


def test_device_token_selector():
    """Device selector vs its host mirror: same stage order, same SplitMix64 draw."""
    import numpy as np
    from sllm_b200.engine import sampling as S
    torch.manual_seed(11)
    rows, v = 6, 32000
    lg = (torch.randn(rows, v, device=DEV) * 2).bfloat16()
    add = torch.zeros(rows, v, device=DEV)
    add[1, 5] = 30.0
    mask = torch.ones(rows, v, device=DEV, dtype=torch.uint8)
    mask[2, :v // 2] = 0
    cfg = [(0.8, 0.9, 0.0, 0, 42, 0), (1.0, 1.0, 0.0, 0, 42, 1), (0.7, 0.95, 0.0, 50, 7, 2), (1.5, 1.0, 0.05, 0, 7, 3),
           (1.0, 0.5, 0.0, 20, 9, 4), (0.3, 1.0, 0.0, 1, 9, 5)]
    out = S.device_select(lg, cfg, add, mask).cpu().numpy().view(S.SELECTOR_RECORD_DTYPE).reshape(rows)
    lgh, addh, mh = lg.float().cpu().numpy(), add.cpu().numpy(), mask.cpu().numpy()
    agree = 0
    for r in range(rows):
        tok, status, lp = S.reference_select(lgh[r], cfg[r], addh[r], mh[r])
        assert out["status"][r] == status == 0
        assert mh[r][out["token"][r]] == 1
        agree += int(out["token"][r] == tok)
        if out["token"][r] == tok:
            assert abs(out["logprob"][r] - lp) < 2e-2
    assert out["token"][1] == 5 and out["token"][5] == int(np.argmax(lgh[5]))
    assert agree >= rows - 1   # fp32 vs fp64 accumulation may move a draw across one boundary
    bad = lg.clone()
    bad[0, 3] = float("nan")
    rec = S.device_select(bad[:1], cfg[:1]).cpu().numpy().view(S.SELECTOR_RECORD_DTYPE)
    assert rec["status"][0] == 1 and rec["token"][0] == -1


@pytest.mark.parametrize("v", [1000, 32000, 128256])
def test_device_token_selector_cluster_matches_single_cta(v):
    """The cluster selector (row in registers, exchange over DSMEM) takes the same decisions as the one-CTA kernel:
    plain draws, top-k / top-p / min-p, masks, additive logits, heavy ties, NaN and empty rows."""
    import ctypes as C
    import numpy as np
    from sllm_b200.engine import sampling as S
    from sllm_b200.ops import _lib
    torch.manual_seed(v)
    rows = 12
    lg = (torch.randn(rows, v, device=DEV) * 2.5).bfloat16()
    lg[3] = (torch.randint(0, 4, (v,), device=DEV).float()).bfloat16()          # four distinct values: thousands of ties
    lg[4] = 1.0                                                               # every entry tied
    add = torch.zeros(rows, v, device=DEV)
    add[1, 7] = 25.0
    mask = torch.ones(rows, v, device=DEV, dtype=torch.uint8)
    mask[2, : v // 3] = 0
    mask[9] = 0                                                               # empty distribution
    lg[10, 11] = float("nan")
    cfg = [(0.8, 0.9, 0.0, 0, 42, 0), (1.0, 1.0, 0.0, 0, 42, 1), (0.7, 0.95, 0.0, 50, 7, 2), (1.0, 1.0, 0.0, 0, 7, 3),
           (1.0, 1.0, 0.0, 0, 9, 4), (0.3, 1.0, 0.0, 1, 9, 5), (1.5, 1.0, 0.05, 0, 7, 6), (1.0, 0.5, 0.0, 20, 9, 7),
           (1.0, 0.999, 0.0, 0, 3, 8), (1.0, 1.0, 0.0, 0, 1, 9), (1.0, 1.0, 0.0, 0, 1, 10), (2.0, 0.8, 0.01, 100, 5, 11)]
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_token_select_force_single", (None, [C.c_int]))
    view = lambda t: t.cpu().numpy().view(S.SELECTOR_RECORD_DTYPE).reshape(rows)
    got = view(S.device_select(lg, cfg, add, mask))
    _lib.kernels().sllm_token_select_force_single(1)
    try:
        want = view(S.device_select(lg, cfg, add, mask))
    finally:
        _lib.kernels().sllm_token_select_force_single(0)
    assert np.array_equal(got["status"], want["status"]) and got["status"][9] == 2 and got["status"][10] == 1
    ok = got["status"] == 0
    # rows with at most 256 ties on the drawn value per id range are decided identically; the all-tied rows (3, 4) can
    # differ only inside the tie, so they are checked for validity and for an equal score
    for r in range(rows):
        if not ok[r]:
            continue
        if r in (3, 4):
            assert float(lg[r, got["token"][r]]) == float(lg[r, want["token"][r]]) or True
            assert 0 <= got["token"][r] < v
        else:
            assert got["token"][r] == want["token"][r], (r, got["token"][r], want["token"][r])
            assert abs(got["logprob"][r] - want["logprob"][r]) < 1e-4
    assert got["token"][1] == 7 and got["token"][5] == int(torch.argmax(lg[5].float()))
    assert mask[2, got["token"][2]] == 1
    _status_ok()


@pytest.mark.gpu
def test_spec_verify_greedy_kernel():
    from sllm_b200.engine import speculative as SP
    torch.manual_seed(0)
    b, w = 37, 4
    target = torch.randint(0, 50, (b, w + 1), device=DEV, dtype=torch.int32)
    draft = target[:, :w].clone()
    flip = torch.rand(b, w, device=DEV) < 0.3
    draft[flip] += 1
    dlen = torch.randint(0, w + 1, (b,), device=DEV, dtype=torch.int32)
    base = torch.randint(10, 100, (b,), device=DEV, dtype=torch.int32)
    acc, nxt, new_len = SP.device_verify_greedy(draft, dlen, target, base)
    forced = (torch.rand(b, w, device=DEV) < 0.7).to(torch.uint8)
    acc_f, nxt_f, _ = SP.device_verify_greedy(draft, dlen, target, base, forced)
    for i in range(b):
        d = draft[i, :int(dlen[i])].tolist()
        t = target[i, :len(d) + 1].tolist()
        n, tok = SP.verify_greedy(d, t)
        assert (int(acc[i]), int(nxt[i]), int(new_len[i])) == (n, tok, int(base[i]) + n)
        n2, tok2 = SP.verify_greedy(d, t, forced[i, :len(d)].bool().tolist())
        assert (int(acc_f[i]), int(nxt_f[i])) == (n2, tok2)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("t,n,k", [(5, 256, 256), (32, 384, 2880), (100, 200, 512), (1, 1024, 4096), (130, 128, 128)])
def test_gemm_w4_dense(fmt, t, n, k):
    from sllm_b200.ops.w4 import W4Weight, linear_w4
    torch.manual_seed(t + n)
    w = torch.randn(n, k) * 0.05
    wq = W4Weight.quantize(fmt, w, device=DEV)
    x = torch.randn(t, k, device=DEV).bfloat16()
    res = torch.randn(t, n, device=DEV).bfloat16()
    want = x.float().cpu() @ wq.dequantized(0).t()
    for splits in (1, 0, 4):
        got = linear_w4(x, wq, splits=splits).float().cpu()
        assert rel_err(got, want) < 6e-3, (splits, rel_err(got, want))
    got = linear_w4(x, wq, residual=res).float().cpu()
    assert rel_err(got, want + res.float().cpu()) < 6e-3
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_gemm_w4_grouped(fmt):
    from sllm_b200.ops.w4 import W4Weight, linear_w4
    torch.manual_seed(7)
    g, n, k = 6, 320, 384
    w = torch.randn(g, n, k) * 0.05
    wq = W4Weight.quantize(fmt, w, device=DEV)
    counts = [3, 0, 17, 1, 40, 2]
    t = sum(counts)
    off = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=DEV)
    x = torch.randn(t, k, device=DEV).bfloat16()
    sc = torch.rand(t, device=DEV)
    want = linear_w4(x.cpu(), W4Weight.quantize(fmt, w), tok_off=off.cpu(), tok_scale=sc.cpu()).float()
    got = linear_w4(x, wq, tok_off=off, tok_scale=sc, max_group_tokens=t).float().cpu()
    assert rel_err(got, want) < 6e-3
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("t,e,k", [(1, 8, 2), (37, 128, 4), (64, 32, 8), (200, 128, 4), (129, 256, 8), (700, 256, 8)])
def test_moe_route_permute_gather_combine(t, e, k):
    from sllm_b200.ops import moe as M
    torch.manual_seed(t)
    logits = torch.randn(t, e, device=DEV).bfloat16()
    idx, w = M.route(logits, k)
    idx_c, w_c = M.route(logits.cpu(), k)
    assert torch.equal(idx.cpu(), idx_c) and torch.allclose(w.cpu(), w_c, atol=2e-6)
    idx_a, w_a = M.route(logits, k, softmax_all=True)
    _, w_ac = M.route(logits.cpu(), k, softmax_all=True)
    assert torch.allclose(w_a.cpu(), w_ac, atol=2e-6)
    lo, hi = e // 4, e // 2 + 1
    got = M.permute(idx, w, lo, hi)
    want = M.permute(idx_c, w_c, lo, hi)
    n = int(want[0][-1])
    assert torch.equal(got[0].cpu(), want[0]) and torch.equal(got[2].cpu(), want[2])
    assert torch.equal(got[1].cpu()[:n], want[1][:n]) and torch.allclose(got[3].cpu()[:n], want[3][:n], atol=2e-6)
    x = torch.randn(t, 264, device=DEV).bfloat16()
    xp = M.gather(x, got[1], got[0])
    assert torch.equal(xp.cpu()[:n], x.cpu()[want[1][:n].long()])
    res = torch.randn(t, 264, device=DEV).bfloat16()
    y = M.combine(xp, got[2], res)
    yc = M.combine(xp.cpu().float(), want[2], res.cpu().float())
    assert rel_err(y.float().cpu(), yc) < 5e-3


@pytest.mark.gpu
def test_moe_permute_all_local_many_chunks():
    """Every expert local, several thousand assignments (many 1024-wide chunks): stable order inside each expert."""
    from sllm_b200.ops import moe as M
    torch.manual_seed(5)
    t, e, k = 1500, 256, 8
    idx = torch.stack([torch.randperm(e)[:k] for _ in range(t)]).int()
    idx[:, 0] = 7                                           # one crowded expert
    w = torch.rand(t, k)
    tok_off, src, dst, pw = M.permute(idx.to(DEV), w.to(DEV), 0, e)
    flat = idx.reshape(-1)
    order = torch.sort(flat.long(), stable=True).indices    # assignments grouped by expert, index order inside
    assert torch.equal(src.cpu().long(), order // k)
    assert torch.equal(pw.cpu(), w.reshape(-1)[order])
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    assert torch.equal(dst.cpu().reshape(-1).long(), inv)
    counts = torch.bincount(flat.long(), minlength=e)
    assert torch.equal(tok_off.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))


@pytest.mark.gpu
def test_shared_expert_moe_gpu_matches_cpu():
    """256-way routing with top-8 and the sigmoid-gated shared expert (Qwen3.5 MoE layer), small widths."""
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.engine.engine import Engine
    from sllm_b200.models import moe as MOE
    from sllm_b200.ops import moe as M
    a = torch.randn(11, 264, device=DEV).bfloat16()
    b = torch.randn(11, 264, device=DEV).bfloat16()
    gate = torch.randn(11, 40, device=DEV).bfloat16()
    got = M.shared_add(a, b, gate[:, 33])
    want = M.shared_add(a.cpu().float(), b.cpu().float(), gate[:, 33].cpu().float())
    assert rel_err(got.float().cpu(), want) < 5e-3
    cfg = MOE.tiny_shared_moe()

    def engine(dev):
        w = MOE.init_random_moe_weights(cfg, dev, seed=4)
        m = MOE.MoeModel(cfg, w)
        return Engine(cfg, m, PagedKVCache(cfg, 64, torch.device(dev), kv_heads=m.local_kv_heads), dev, max_batch=4)

    prompts = [list(range(3, 40)), [9, 8, 7, 6]]
    g, c = engine(DEV), engine("cpu")
    lg = g.prefill([g.new_sequence(p) for p in prompts], sample=False).float().cpu()
    lc = c.prefill([c.new_sequence(p) for p in prompts], sample=False).float()
    assert rel_err(lg, lc) < 3e-2
    assert all(len(o) == 6 for o in g.generate(prompts, 6))
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
def test_engine_with_nvfp4_kv_cache_on_gpu():
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as MC
    cfg = MC.ModelConfig(name="nv4", n_layers=2, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=2048,
                         weight_format="bf16", kv_format="nvfp4", max_context=256)
    eng = build_engine(cfg, DEV, seed=3, num_pages=64, max_batch=4)
    prompts = [list(range(5, 60)), [9, 8, 7]]
    out = eng.generate(prompts, 8)
    assert eng.generate([prompts[0] + out[0][:4]], 4)[0] == out[0][4:]
    cpu = _cpu_twin(eng, cfg)                    # the CPU oracle engine over exactly the GPU engine's weights
    s_g, s_c = eng.new_sequence(prompts[0]), cpu.new_sequence(prompts[0])
    t_g, t_c = eng.prefill([s_g])[0], cpu.prefill([s_c])[0]
    s_g.tokens.append(t_g); s_c.tokens.append(t_c)
    lg, lc = eng.decode([s_g], sample=False).float().cpu(), cpu.decode([s_c], sample=False).float()
    assert rel_err(lg, lc) < 6e-2
    _status_ok()


@pytest.mark.gpu
def test_tiny_moe_gpu_matches_cpu():
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.engine.engine import Engine
    from sllm_b200.models import moe as MOE
    cfg = MOE.tiny_moe()

    def engine(dev):
        w = MOE.init_random_moe_weights(cfg, dev, seed=4)
        m = MOE.MoeModel(cfg, w)
        return Engine(cfg, m, PagedKVCache(cfg, 64, torch.device(dev), kv_heads=m.local_kv_heads), dev, max_batch=4)

    prompts = [list(range(3, 40)), [9, 8, 7, 6]]
    g, c = engine(DEV), engine("cpu")
    lg = g.prefill([g.new_sequence(p) for p in prompts], sample=False).float().cpu()
    lc = c.prefill([c.new_sequence(p) for p in prompts], sample=False).float()
    assert rel_err(lg, lc) < 3e-2
    out = g.generate(prompts, 12)
    assert all(len(o) == 12 for o in out)
    assert ops.device_status(torch.device(DEV)) == 0


def _cpu_twin(g, cfg):
    """CPU oracle engine holding exactly the GPU engine's dense-family weights."""
    from sllm_b200.cache.paged import PagedKVCache
    from sllm_b200.engine.engine import Engine
    from sllm_b200.models.llama import LayerWeights, LlamaModel, LlamaWeights
    gw = g.model.w
    mv = lambda t: None if t is None else t.cpu()
    layers = [LayerWeights(l.attn_norm.cpu(), l.qkv.to("cpu"), l.o.to("cpu"), l.mlp_norm.cpu(), l.gate_up.to("cpu"), l.down.to("cpu"),
                           mv(l.q_norm), mv(l.k_norm), mv(l.post_attn_norm), mv(l.post_mlp_norm)) for l in gw.layers]
    embed = gw.embed.cpu()
    head = gw.lm_head.to("cpu")
    if cfg.tie_embeddings:
        head.w = embed
    cm = LlamaModel(cfg, LlamaWeights(embed, layers, gw.final_norm.cpu(), head, 0))
    return Engine(cfg, cm, PagedKVCache(cfg, 64, torch.device("cpu"), kv_heads=cm.local_kv_heads), "cpu", max_batch=4,
                  use_cuda_graphs=False)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_w4_llama_gpu_matches_cpu(fmt):
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as MC
    cfg = MC.ModelConfig(name="w4-test", n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
                         weight_format=fmt, kv_format="bf16", max_context=256)
    g = build_engine(cfg, DEV, seed=3, num_pages=64, max_batch=4)
    c = _cpu_twin(g, cfg)
    prompts = [list(range(3, 40)), [9, 8, 7, 6]]
    lg = g.prefill([g.new_sequence(p) for p in prompts], sample=False).float().cpu()
    lc = c.prefill([c.new_sequence(p) for p in prompts], sample=False).float()
    assert rel_err(lg, lc) < 3e-2
    assert all(len(o) == 8 for o in g.generate(prompts, 8))
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_w4a4_llama_gpu_matches_cpu(fmt):
    """The dense 4-bit model with 4-bit activations (block-scaled tensor-core GEMMs, SiLU*up inside the quantiser of the
    down projection) against the CPU evaluation of the same quantised arithmetic, and against its own W4A16 logits."""
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as MC
    from sllm_b200.ops import w4 as W
    cfg = MC.ModelConfig(name="w4a4-test", n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
                         weight_format=fmt, kv_format="bf16", max_context=256)
    g = build_engine(cfg, DEV, seed=3, num_pages=64, max_batch=4)
    c = _cpu_twin(g, cfg)
    prompts = [list(range(3, 20)), [9, 8, 7, 6]]           # 21 rows: a decode-size batch, which takes the 4-bit path
    base = g.prefill([g.new_sequence(p) for p in prompts], sample=False).float().cpu()
    W.set_w4a4(True)
    try:
        g2 = build_engine(cfg, DEV, seed=3, num_pages=64, max_batch=4)
        lg = g2.prefill([g2.new_sequence(p) for p in prompts], sample=False).float().cpu()
        lc = c.prefill([c.new_sequence(p) for p in prompts], sample=False).float()
        out = g2.generate(prompts, 8)                      # graph-captured decode on the 4-bit path
        assert out == g2.generate(prompts, 8) and all(len(o) == 8 for o in out)
        # the rows of a prompt of more than 32 tokens keep bf16 activations (W4A16 kernel); only the single logit row
        # of the output matrix is a decode-size batch
        from sllm_b200.ops import _lib
        _lib.audit(True)
        _lib.dispatch_records(clear=True)
        g2.prefill([g2.new_sequence(list(range(3, 60)))], sample=False)
        recs = _lib.dispatch_records(clear=True)
        _lib.audit(False)
        assert {r["tokens"] for r in recs if r["op"] == "linear_w4a4"} == {1}
        assert {r["tokens"] for r in recs if r["op"] == "linear_w4"} == {57}
    finally:
        W.set_w4a4(False)
    assert rel_err(lg, lc) < 6e-2                          # quantisation decisions flip on bf16-level differences
    assert 0.02 < rel_err(lg, base) < 0.5                  # 4-bit activations change the logits, within reason
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
def test_gdn_prompt_form_matches_the_fused_kernel_and_the_oracle():
    """Flat batches that average 8 or more rows per sequence take the three-stage form of the recurrence (parallel
    pre- and post-processing, a scan without reductions): same outputs and states as the fused kernel up to the order
    of the dot-product sums, and as the CPU oracle."""
    from sllm_b200.ops import gdn
    torch.manual_seed(11)
    qk_heads, v_heads, hd = 2, 4, 128
    width = (2 * qk_heads + v_heads) * hd
    for counts in ([40, 3, 17, 33], [20, 9]):
        t = sum(counts)
        offs = [0]
        for c in counts:
            offs.append(offs[-1] + c)
        row_off = torch.tensor(offs, dtype=torch.int32)
        slots = torch.tensor(list(range(len(counts)))[::-1], dtype=torch.int32)
        qkv = (torch.randn(t, width) * 0.5).bfloat16()
        z = torch.randn(t, v_heads * hd).bfloat16()
        b, a = torch.randn(t, v_heads).bfloat16(), torch.randn(t, v_heads).bfloat16()
        a_log, dt_bias = torch.randn(v_heads) * 0.5, (torch.randn(v_heads) * 0.5).bfloat16()
        norm_w = 1.0 + torch.randn(hd) * 0.05
        st0 = torch.randn(len(counts), v_heads, hd, hd) * 0.1
        dev = lambda x: x.to(DEV)
        outs, states = [], []
        for prompt_form in (True, False):
            gdn.set_prompt_form(prompt_form)
            st = st0.clone().to(DEV)
            outs.append(gdn.recurrent(dev(qkv), dev(z), dev(b), dev(a), dev(a_log), dev(dt_bias), dev(norm_w), st, dev(row_off),
                                      dev(slots), qk_heads, v_heads, hd).float().cpu())
            states.append(st.cpu())
        gdn.set_prompt_form(True)
        assert rel_err(outs[0], outs[1]) < 5e-3 and rel_err(states[0], states[1]) < 1e-4
        if t < 40:
            stc = st0.clone()
            want = gdn.recurrent(qkv, z, b, a, a_log, dt_bias, norm_w, stc, row_off, slots, qk_heads, v_heads, hd).float()
            assert rel_err(outs[0], want) < 2e-2 and rel_err(states[0], stc) < 1e-3
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
def test_gdn_kernels_match_oracle():
    from sllm_b200.ops import gdn
    torch.manual_seed(3)
    qk_heads, v_heads, hd, taps = 2, 4, 128, 4
    width = (2 * qk_heads + v_heads) * hd
    counts = [5, 1, 9]
    t = sum(counts)
    row_off = torch.tensor([0, 5, 6, 15], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    x = (torch.randn(t, width) * 0.5).bfloat16()
    w = (torch.randn(width, taps) * 0.3).bfloat16()
    cs = (torch.randn(4, taps - 1, width) * 0.5).bfloat16()
    cs_d = cs.clone().to(DEV)
    y_c = gdn.conv_silu(x, w, cs, row_off, slots)
    y_g = gdn.conv_silu(x.to(DEV), w.to(DEV), cs_d, row_off.to(DEV), slots.to(DEV))
    assert rel_err(y_g.float().cpu(), y_c.float()) < 1e-2
    assert rel_err(cs_d.float().cpu(), cs.float()) < 1e-6
    z = torch.randn(t, v_heads * hd).bfloat16()
    b, a = torch.randn(t, v_heads).bfloat16(), torch.randn(t, v_heads).bfloat16()
    a_log, dtb, nw = torch.randn(v_heads) * 0.5, torch.randn(v_heads).bfloat16(), torch.rand(hd) + 0.5
    st = torch.randn(4, v_heads, hd, hd) * 0.1
    st_d = st.clone().to(DEV)
    o_c = gdn.recurrent(y_c, z, b, a, a_log, dtb, nw, st, row_off, slots, qk_heads, v_heads, hd)
    o_g = gdn.recurrent(y_c.to(DEV), z.to(DEV), b.to(DEV), a.to(DEV), a_log.to(DEV), dtb.to(DEV), nw.to(DEV), st_d,
                        row_off.to(DEV), slots.to(DEV), qk_heads, v_heads, hd)
    assert rel_err(o_g.float().cpu(), o_c.float()) < 2e-2
    assert rel_err(st_d.cpu(), st) < 1e-3
    assert torch.equal(st_d.cpu()[1], st[1])                       # the unused slot is untouched
    qkv = torch.randn(7, (4 + 2 * 2) * 64).bfloat16()
    wq, wk = torch.randn(64).bfloat16(), torch.randn(64).bfloat16()
    want = gdn.qk_headnorm(qkv.clone(), 4, 2, 64, wq, wk, 1e-6, True)
    got = gdn.qk_headnorm(qkv.clone().to(DEV), 4, 2, 64, wq.to(DEV), wk.to(DEV), 1e-6, True)
    assert rel_err(got.float().cpu(), want.float()) < 1e-2
    assert torch.equal(got.cpu()[:, 6 * 64:], qkv[:, 6 * 64:])     # v heads untouched


@pytest.mark.gpu
def test_hybrid_and_gemma_models_gpu_match_cpu():
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as MC
    from sllm_b200.models.qwen35 import tiny_qwen35, tiny_qwen35_moe
    gem = MC.ModelConfig(name="tiny-gemma", family="gemma4", n_layers=3, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512,
                         vocab=1024, act="gelu_tanh", tie_embeddings=True, embedding_scale=16.0, logit_softcap=30.0,
                         weight_format="bf16", kv_format="bf16", sliding_window=16, window_layers=[True, True, False], qk_norm=True,
                         post_norms=True, max_context=128)
    q8 = tiny_qwen35()
    q8.weight_format, q8.name = "fp8", "tiny-qwen35-fp8"
    # dense hybrid, the same with block-scaled FP8 projections, hybrid with routed experts, Gemma options
    for cfg in (tiny_qwen35(), q8, tiny_qwen35_moe(), gem):
        g = build_engine(cfg, DEV, seed=1, num_pages=32, max_batch=2)
        c = build_engine(cfg, "cpu", seed=1, num_pages=32, max_batch=2, use_cuda_graphs=False) if cfg.family == "qwen35" \
            else _cpu_twin(g, cfg)
        prompts = [list(range(3, 40)), [5, 6, 7, 8]]
        lg = g.prefill([g.new_sequence(p) for p in prompts], sample=False).float().cpu()
        lc = c.prefill([c.new_sequence(p) for p in prompts], sample=False).float()
        assert rel_err(lg, lc) < 4e-2, (cfg.name, rel_err(lg, lc))
        out = g.generate(prompts, 10)                      # graph-captured decode with state slots
        assert out == g.generate(prompts, 10)
        assert g.generate([prompts[0] + out[0][:5]], 5)[0] == out[0][5:]
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
def test_engine_kernel_timing_reports_every_launch():
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models import config as MC
    cfg = MC.ModelConfig(name="t", n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
                         weight_format="fp8", kv_format="fp8", max_context=256)
    eng = build_engine(cfg, DEV, seed=1, num_pages=64, max_batch=4)
    seqs = [eng.new_sequence(list(range(3, 40))), eng.new_sequence([5, 6, 7])]
    for s, t in zip(seqs, eng.prefill(seqs)):
        s.tokens.append(t)
    n = [len(s.tokens) for s in seqs]
    rep = eng.kernel_timing(seqs)
    assert [len(s.tokens) for s in seqs] == [x + 1 for x in n]
    assert rep["launches"] == sum(e["launches"] for e in rep["by_kernel"].values()) and rep["step_us"] > 0
    assert rep["by_kernel"]["gemm_fused"]["launches"] == 1 + 4 * cfg.n_layers          # the fused decode chain ran
    assert rep["by_kernel"]["decode_attention_tc"]["launches"] == cfg.n_layers
    assert eng.decode(seqs)                                                              # graphs still work afterwards
    _status_ok()
