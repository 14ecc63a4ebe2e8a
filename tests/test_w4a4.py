"""W4A4 path: 4-bit activations (NVFP4 / MXFP4) times 4-bit weights on the block-scaled tensor-core kinds.

CPU: the activation quantiser's oracle, the native tile layout (swizzled code image + scale atoms) against the file
layout, and the CPU form of the GEMM.  GPU: the quantiser kernel bit for bit against the oracle, structured probes that
isolate each scale mapping (weight row, weight K block, token row, activation K block), and random dense / grouped /
split-K cases against an fp32 evaluation of the same quantised operands.
(Reference: native/hip/src/matmul_kernel.hip.cpp:343,396,457,562 - activation quantisers and W4A4 dots.)"""
import numpy as np
import pytest
import torch

from sllm_b200 import ops
from sllm_b200.ops import reference as R
from sllm_b200.ops.w4 import W4Weight, act_quant_fp4, linear_w4, linear_w4a4, sf_compact, sf_padded

DEV = "cuda"


def rel(a, b):
    return ((a - b).norm() / (b.norm() + 1e-9)).item()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_activation_quantiser_oracle(fmt):
    torch.manual_seed(0)
    x = (torch.randn(6, 200) * torch.logspace(-3, 2, 6).view(6, 1)).to(torch.bfloat16)
    x[2] = 0
    x[4, 7] = float("nan")
    codes, sf, outer = R.quant_act_fp4(x, fmt)
    block = 32 if fmt == "mxfp4" else 16
    assert codes.shape == (6, 128) and sf.shape == (6, 256 // block) and outer.shape == (6,)
    back = R.dequant_act_fp4(codes, sf, outer, fmt)
    assert torch.equal(back[2], torch.zeros(256)) and torch.equal(back[:, 200:], torch.zeros(6, 56))
    for r in (0, 1, 3, 5):                       # every magnitude range keeps the 4-bit relative error
        assert rel(back[r, :200], x[r].float()) < 0.16
    assert torch.isfinite(back).all()            # the NaN element became a zero code
    if fmt == "nvfp4":
        assert torch.allclose(outer[0], x[0].float().abs().max() / 2688.0) and outer[2] == 1.0
    else:
        assert torch.equal(outer, torch.ones(6))


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_native_tiles_hold_the_file_layout(fmt):
    torch.manual_seed(1)
    w = W4Weight.quantize(fmt, torch.randn(2, 130, 200) * 0.1)
    nt = w.native_tiles()
    g, rt, kb, width = nt.shape
    atoms = 4 if fmt == "nvfp4" else 2
    assert (g, rt, kb, width) == (2, 2, 1, 16384 + 512 * atoms) and w.native_tiles() is nt
    img = nt[..., :16384].view(g, rt, kb, 128, 8, 16)
    rr = (torch.arange(128) & 7).view(128, 1)
    src = (torch.arange(8).view(1, 8) ^ rr).view(1, 1, 1, 128, 8, 1)
    rows = torch.gather(img, 4, src.expand(g, rt, kb, 128, 8, 16)).reshape(g, rt, kb, 128, 128)
    rows = rows.permute(0, 1, 3, 2, 4).reshape(g, rt * 128, kb * 128)
    for gi in range(g):
        packed, scales = w.to_file_layout(gi)
        assert np.array_equal(rows[gi, :130, :100].numpy(), packed)
        at = nt[gi, ..., 16384:].view(rt, kb, atoms, 32, 4, 4)                 # [atom][r][j][s]: scale s of row r + 32 j
        sc = at.permute(0, 4, 3, 1, 2, 5).reshape(rt * 128, kb * atoms * 4)
        assert np.array_equal(sc[:130, :scales.shape[1]].numpy(), scales)


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_cpu_form_tracks_the_w4a16_result(fmt):
    torch.manual_seed(2)
    w = W4Weight.quantize(fmt, torch.randn(96, 320) * 0.1)
    x = torch.randn(5, 320).to(torch.bfloat16)
    a16 = linear_w4(x, w).float()
    a4 = linear_w4a4(x, w).float()
    assert 0.02 < rel(a4, a16) < 0.16            # 4-bit activations cost about a tenth, and are not a no-op
    q = act_quant_fp4(x, fmt)
    assert torch.equal(sf_compact(q[1]), R.quant_act_fp4(x, fmt)[1]) and torch.equal(sf_padded(sf_compact(q[1])), q[1])
    assert torch.equal(linear_w4a4(x, w, quantized=q), linear_w4a4(x, w))


# ---------------------------------------------------------------------------------------------------- GPU
def _oracle(q, w, t, tok_off=None, tok_scale=None, residual=None):
    xf = R.dequant_act_fp4(q[0], sf_compact(q[1].cpu()), q[2], w.fmt)[:, :w.k]
    out = torch.zeros((t, w.n))
    offs = [0, t] if tok_off is None else tok_off.cpu().tolist()
    for g in range(w.groups):
        a, b = offs[g], offs[g + 1]
        if b > a:
            out[a:b] = xf[a:b] @ w.dequantized(g).t()
    if tok_scale is not None:
        out = out * tok_scale.cpu().float()[:, None]
    if residual is not None:
        out = out + residual.float().cpu()
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_quantiser_kernel_is_bit_exact(fmt):
    torch.manual_seed(3)
    x = (torch.randn(9, 2880) * torch.logspace(-2, 1, 9).view(9, 1)).to(torch.bfloat16)
    x[3] = 0
    def same(got, want):
        assert torch.equal(got[0].cpu(), want[0]) and torch.equal(got[2].cpu(), want[2])
        assert torch.equal(sf_compact(got[1].cpu()), want[1])          # four scale bytes, then four the kernel ignores

    same(act_quant_fp4(x.to(DEV), fmt), R.quant_act_fp4(x, fmt))
    # gathered rows: token t reads source row src_row[t]
    src = torch.tensor([8, 0, 0, 5], dtype=torch.int32, device=DEV)
    same(act_quant_fp4(x.to(DEV), fmt, src_row=src), R.quant_act_fp4(x[[8, 0, 0, 5]], fmt))
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("kind", ["ones", "w_row", "w_k", "x_row", "x_k"])
def test_scale_mappings_one_at_a_time(fmt, kind):
    """All codes are 1.0; one family of scales varies, so a wrong lane, column or byte of the scale layout in tensor
    memory changes the (exactly representable) result."""
    block = 32 if fmt == "mxfp4" else 16
    n, k, t = 128, 512, 32
    sc = (lambda e: 127 + e) if fmt == "mxfp4" else (lambda e: 0x38 + 8 * e)
    wp, ws = np.full((n, k // 2), 0x22, dtype=np.uint8), np.full((n, k // block), sc(0), dtype=np.uint8)
    xp, xs = torch.full((t, k // 2), 0x22, dtype=torch.uint8), torch.full((t, k // block), sc(0), dtype=torch.uint8)
    if kind == "w_row":
        for m in range(n):
            ws[m, :] = sc(m % 4)
    elif kind == "w_k":
        for b in range(k // block):
            ws[:, b] = sc(b % 5)
    elif kind == "x_row":
        for m in range(t):
            xs[m, :] = sc(m % 3)
    elif kind == "x_k":
        for b in range(k // block):
            xs[:, b] = sc(b % 5)
    w = W4Weight.from_file_layout(fmt, wp, ws, k, None, DEV)
    q = (xp.to(DEV), sf_padded(xs).to(DEV), torch.ones(t, device=DEV))
    y = linear_w4a4(None, w, quantized=q).float().cpu()
    assert torch.equal(y, _oracle(q, w, t))
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("t,n,k,groups,splits", [(1, 256, 512, 1, 0), (7, 300, 2880, 1, 0), (32, 1024, 4096, 1, 2),
                                                  (32, 512, 8192, 1, 0), (100, 384, 1024, 1, 0), (40, 256, 2048, 8, 0),
                                                  (130, 256, 1024, 3, 0),
                                                  # dense decode schedule: runs of K blocks that cross row tiles unevenly
                                                  (3, 640, 3328, 1, 0), (32, 2944, 4096, 1, 0), (16, 8192, 8192, 1, 0),
                                                  (16, 8192, 8192, 1, 1)])
def test_gemm_fp4_against_fp32_of_the_same_operands(fmt, t, n, k, groups, splits):
    torch.manual_seed(t + n)
    w = W4Weight.quantize(fmt, torch.randn(groups, n, k) * 0.1, DEV, keep_file=False)
    x = torch.randn(t, k).to(torch.bfloat16).to(DEV)
    tok_off = ts = mg = res = None
    if groups > 1:
        cuts = sorted(torch.randint(0, t + 1, (groups - 1,)).tolist())
        offs = [0] + cuts + [t]
        tok_off = torch.tensor(offs, dtype=torch.int32, device=DEV)
        mg = max(b - a for a, b in zip(offs, offs[1:]))
        ts = torch.rand(t, device=DEV)
    else:
        res = torch.randn(t, n).to(torch.bfloat16).to(DEV)
    q = act_quant_fp4(x, fmt)
    y = linear_w4a4(x, w, residual=res, tok_off=tok_off, tok_scale=ts, max_group_tokens=mg, splits=splits, quantized=q)
    want = _oracle(q, w, t, tok_off, ts, res)
    assert rel(y.float().cpu(), want) < 4e-3
    if t > 32:
        # the wide token tiles (scales staged through shared memory, K split through the workspace)
        for bn in (64, 128):
            yw = linear_w4a4(x, w, residual=res, tok_off=tok_off, tok_scale=ts, max_group_tokens=mg, quantized=q, bn=bn)
            assert rel(yw.float().cpu(), want) < 4e-3
    # the whole path (quantise + multiply) stays within the 4-bit activation error of the bf16-activation kernel
    if groups == 1:
        a16 = linear_w4(x, w, residual=res).float().cpu()
        assert rel(y.float().cpu(), a16) < 0.16
    assert ops.device_status(torch.device(DEV)) == 0


def test_expert_mlp_with_4bit_activations_cpu():
    """The routed expert MLP in its W4A4 form (quantiser reads the routed rows, SiLU*up inside the second quantiser)
    tracks the bf16-activation form within the 4-bit error, and the switch really changes the path."""
    from sllm_b200.ops import moe as M
    from sllm_b200.ops import w4 as W
    torch.manual_seed(5)
    E, d, F, t, k = 8, 256, 128, 6, 2
    gate_up = W4Weight.quantize("mxfp4", torch.randn(E, 2 * F, d) * 0.1)
    down = W4Weight.quantize("mxfp4", torch.randn(E, d, F) * 0.1)
    x = torch.randn(t, d).to(torch.bfloat16)
    idx, rw = M.route(torch.randn(t, E), k)
    base, perm = M.experts_forward(x, idx, rw, gate_up, down, "silu", 0, E)
    W.set_w4a4(True)
    try:
        a4, perm4 = M.experts_forward(x, idx, rw, gate_up, down, "silu", 0, E)
    finally:
        W.set_w4a4(False)
    assert torch.equal(perm, perm4) and a4.shape == base.shape
    assert 0.02 < rel(a4.float(), base.float()) < 0.25


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_gated_quantiser_and_expert_mlp_gpu(fmt):
    from sllm_b200.ops import moe as M
    from sllm_b200.ops import w4 as W
    torch.manual_seed(6)
    # SiLU*up inside the quantiser: within the 4-bit step of quantising the stand-alone kernel's output
    gu = torch.randn(5, 2 * 384).to(torch.bfloat16)
    q = act_quant_fp4(gu.to(DEV), fmt, gated="silu")
    want = R.round_bf16(R.gated_act(gu, "silu"))
    got = R.dequant_act_fp4(q[0], sf_compact(q[1].cpu()), q[2], fmt)[:, :384]
    assert rel(got, want) < 0.16
    ref = R.dequant_act_fp4(*[a if i != 1 else a for i, a in enumerate(R.quant_act_fp4(want, fmt))], fmt)[:, :384]
    assert rel(got, ref) < 0.03                       # the same quantiser up to the device's exp()
    # RMSNorm inside the quantiser
    h = torch.randn(7, 640).to(torch.bfloat16)
    nw = (torch.randn(640) * 0.1).to(torch.bfloat16)
    for off1 in (False, True):
        qn = act_quant_fp4(h.to(DEV), fmt, norm=(nw.to(DEV), 1e-5, off1))
        wantn = R.round_bf16(R.rmsnorm(h, nw, 1e-5, off1))
        gotn = R.dequant_act_fp4(qn[0], sf_compact(qn[1].cpu()), qn[2], fmt)[:, :640]
        refn = R.dequant_act_fp4(*R.quant_act_fp4(wantn, fmt), fmt)[:, :640]
        assert rel(gotn, wantn) < 0.16 and rel(gotn, refn) < 0.03
    # the routed expert MLP, GPU against the CPU form of the same W4A4 arithmetic
    E, d, F, t, k = 8, 256, 256, 40, 2
    wgu, wdn = torch.randn(E, 2 * F, d) * 0.1, torch.randn(E, d, F) * 0.1
    x = torch.randn(t, d).to(torch.bfloat16)
    idx, rw = M.route(torch.randn(t, E), k)
    W.set_w4a4(True)
    try:
        want, _ = M.experts_forward(x, idx, rw, W4Weight.quantize(fmt, wgu), W4Weight.quantize(fmt, wdn), "silu", 0, E)
        got, _ = M.experts_forward(x.to(DEV), idx.to(DEV), rw.to(DEV), W4Weight.quantize(fmt, wgu, DEV, keep_file=False),
                                   W4Weight.quantize(fmt, wdn, DEV, keep_file=False), "silu", 0, E)
        # a scatter-free combine of both gives the layer output; rows past the routed ones are not compared
        n = t * k
        assert rel(got[:n].float().cpu(), want[:n].float()) < 0.05
        # dense form through the switch: decode-size batches take the 4-bit path, prompt-size ones keep bf16 activations
        w = W4Weight.quantize(fmt, torch.randn(192, d) * 0.1, DEV, keep_file=False)
        y4 = linear_w4(x[:32].to(DEV), w)
        y4_prompt = linear_w4(x.to(DEV), w)
    finally:
        W.set_w4a4(False)
    y16 = linear_w4(x.to(DEV), w)
    assert 0.02 < rel(y4.float(), y16[:32].float()) < 0.16
    assert torch.equal(y4_prompt, y16)
    assert ops.device_status(torch.device(DEV)) == 0


@pytest.mark.gpu
def test_scatter_epilogue_places_rows_by_address():
    """row_ptr: result row t is stored at the bf16 row whose address is row_ptr[t] (the expert-parallel combine hands
    addresses in the token owner's memory); here the addresses permute the rows of a local buffer."""
    torch.manual_seed(8)
    t, n, k, groups = 24, 256, 512, 4
    w = W4Weight.quantize("mxfp4", torch.randn(groups, n, k) * 0.1, DEV, keep_file=False)
    x = torch.randn(t, k).to(torch.bfloat16).to(DEV)
    tok_off = torch.tensor([0, 5, 5, 17, 24], dtype=torch.int32, device=DEV)
    ts = torch.rand(t, device=DEV)
    q = act_quant_fp4(x, "mxfp4")
    plain = linear_w4a4(None, w, tok_off=tok_off, tok_scale=ts, max_group_tokens=12, quantized=q)
    buf = torch.zeros((t, n), dtype=torch.bfloat16, device=DEV)
    perm = torch.randperm(t)
    row_ptr = torch.tensor([buf.data_ptr() + int(p) * n * 2 for p in perm], dtype=torch.int64, device=DEV)
    assert linear_w4a4(None, w, tok_off=tok_off, tok_scale=ts, max_group_tokens=12, quantized=q, row_ptr=row_ptr) is None
    torch.cuda.synchronize()
    assert torch.equal(buf[perm.to(DEV)], plain)
    assert ops.device_status(torch.device(DEV)) == 0
