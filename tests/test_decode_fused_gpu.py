"""Fused decode kernel: every phase kind against an fp32 PyTorch restatement, at tile-edge shapes and with grids
that force tiles to be split over several CTAs; then whole decode steps against the per-op path."""
import math

import pytest
import torch

from sllm_b200 import ops
from sllm_b200.ops import fused_decode as fd
from sllm_b200.ops import reference as ref
from sllm_b200.ops.core import KVLayer, LinearWeight

pytestmark = pytest.mark.gpu
DEV = "cuda"
IMPLS = ["persistent", "cluster"]      # one persistent kernel for all phases / one cluster split-K GEMM per phase


def _status_ok():
    assert ops.device_status(torch.device(DEV)) == 0


def close(got, want, rtol=2e-2, atol_frac=6e-3, name=""):
    """Per-element check: |got - want| <= rtol |want| + atol_frac * max|want|, and a tight norm-relative error."""
    got, want = got.float().cpu(), want.float().cpu()
    tol = rtol * want.abs() + atol_frac * want.abs().max()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{name}: {int(bad.sum())} elements off, worst {(got - want).abs().max().item():.4g}"
    assert ((got - want).norm() / (want.norm() + 1e-12)).item() < 6e-3, name


def _weights(n_rows, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n_rows, k, generator=g) * 0.03).bfloat16()
    w[:, :128] *= 4
    lw = LinearWeight.from_dense(w, "fp8").to(DEV)
    return lw


def _acts(rows, k, bn, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, k, generator=g) * 1.5).bfloat16()
    x[:, -128:] *= 12
    q, s_t = ref.quant_fp8_1x128(x)
    s = torch.zeros((k // 128, bn), dtype=torch.float32)
    s[:, :rows] = s_t
    return q.to(DEV), s.to(DEV)


@pytest.mark.parametrize("rows,n,k,grid", [(1, 128, 128, 1), (5, 384, 512, 3), (16, 1000, 256, 7), (17, 640, 1024, 148),
                                           (32, 4096, 4096, 148), (32, 128, 2048, 148), (31, 2052, 384, 0),
                                           (8, 256, 14336, 148)])
@pytest.mark.parametrize("impl", IMPLS)
def test_plain_phase(impl, rows, n, k, grid):
    bn = 16 if rows <= 16 else 32
    lw = _weights(n, k, n + k)
    xq, xs = _acts(rows, k, bn, rows)
    res = (torch.randn(rows, n) * 0.5).bfloat16().to(DEV)
    y = torch.zeros((rows, n), dtype=torch.bfloat16, device=DEV)
    ph = fd.phase(fd.PLAIN, lw.w, lw.scale_t, xq, xs, n=n, k=k, y=y, ldy=n, residual=res)
    for _ in range(2):      # the second call runs on the counters and the barrier word the first one left
        y.zero_()
        fd.launch([ph], rows, torch.device(DEV), grid=grid, impl=impl)
    want = fd.ref_plain(lw.w, lw.scale_t, xq, xs, rows, residual=res)
    close(y, want, name="plain")
    _status_ok()


@pytest.mark.parametrize("rows,d,k,grid", [(1, 256, 512, 5), (16, 512, 256, 148), (32, 4096, 4096, 148), (20, 1024, 1792, 37)])
@pytest.mark.parametrize("impl", IMPLS)
def test_resid_quant_phase(impl, rows, d, k, grid):
    bn = 16 if rows <= 16 else 32
    lw = _weights(d, k, d * 3 + k)
    xq, xs = _acts(rows, k, bn, rows + 1)
    h = (torch.randn(rows, d) * 0.7).bfloat16().to(DEV)
    h0 = h.clone()
    q = torch.zeros((rows, d), dtype=torch.uint8, device=DEV)
    s = torch.zeros((d // 128, bn), dtype=torch.float32, device=DEV)
    ssq = torch.zeros((d // 128, bn), dtype=torch.float32, device=DEV)
    ph = fd.phase(fd.RESID_QUANT, lw.w, lw.scale_t, xq, xs, n=d, k=k, y=h, ldy=d, residual=h, q_out=q, s_out=s,
                  ssq_out=ssq, ld_s_out=bn)
    fd.launch([ph], rows, torch.device(DEV), grid=grid, impl=impl)
    want = fd.ref_plain(lw.w, lw.scale_t, xq, xs, rows, residual=h0)
    close(h, want, name="residual stream")
    # the quantised form and the statistics describe the bf16 values the kernel itself wrote
    hv, q_ref, s_ref, ssq_ref = fd.ref_quant_rows(h.float().cpu())
    assert torch.equal(q.cpu(), q_ref)
    assert torch.allclose(s.cpu()[:, :rows], s_ref, rtol=1e-6, atol=0)
    assert torch.allclose(ssq.cpu()[:, :rows], ssq_ref, rtol=1e-4, atol=1e-6)
    _status_ok()


@pytest.mark.parametrize("rows,ffn,k,grid,act", [(3, 256, 256, 4, 0), (16, 1792, 512, 148, 0), (32, 14336, 4096, 148, 0),
                                                 (32, 384, 1024, 9, 1)])
@pytest.mark.parametrize("impl", IMPLS)
def test_silu_quant_phase(impl, rows, ffn, k, grid, act):
    bn = 16 if rows <= 16 else 32
    lw = _weights(2 * ffn, k, ffn + k)
    xq, xs = _acts(rows, k, bn, rows + 2)
    ssq_in = (torch.rand((k // 128, bn)) * 200 + 10).to(DEV)
    q = torch.zeros((rows, ffn), dtype=torch.uint8, device=DEV)
    s = torch.zeros((ffn // 128, bn), dtype=torch.float32, device=DEV)
    ph = fd.phase(fd.SILU_QUANT, lw.w, lw.scale_t, xq, xs, n=ffn, k=k, dual_off=ffn, ssq_in=ssq_in, norm_dim=k, eps=1e-5,
                  act=act, q_out=q, s_out=s, ld_s_out=bn)
    il = [fd.interleave_gate_up(lw.w, lw.scale_t, ffn)]
    fd.launch([ph], rows, torch.device(DEV), grid=grid, impl=impl, interleaved=il)
    norm = fd.ref_norm_factor(ssq_in, rows, k, 1e-5)
    want = fd.ref_silu(lw.w, lw.scale_t, xq, xs, rows, ffn, ffn, norm, act)
    got = ref.dequant_fp8_1x128(q.cpu(), s.cpu()[:, :rows].contiguous())
    # E4M3 carries 3 mantissa bits: half a step of 1/8 relative to the block maximum
    tol = 0.07 * want.abs() + 0.04 * want.abs().view(rows, -1, 128).amax(dim=-1, keepdim=True).expand(-1, -1, 128).reshape(rows, ffn)
    assert ((got - want).abs() <= tol + 1e-6).all()
    assert ((got - want).norm() / want.norm()).item() < 4e-2
    _status_ok()


@pytest.mark.parametrize("rows,hq,hkv,rd,fp8,grid", [(1, 4, 2, 128, True, 6), (16, 8, 2, 128, True, 148), (32, 32, 8, 128, True, 148),
                                                     (7, 4, 4, 64, False, 11), (9, 2, 1, 128, True, 1)])
@pytest.mark.parametrize("impl", IMPLS)
def test_rope_kv_phase(impl, rows, hq, hkv, rd, fp8, grid):
    hd, d, page = 128, 512, 16
    bn = 16 if rows <= 16 else 32
    n = (hq + 2 * hkv) * hd
    lw = _weights(n, d, n + rows)
    xq, xs = _acts(rows, d, bn, rows + 3)
    ssq_in = (torch.rand((d // 128, bn)) * 300 + 20).to(DEV)
    g = torch.Generator().manual_seed(rows)
    positions = torch.randint(0, 200, (rows,), generator=g, dtype=torch.int32)
    seq_index = torch.arange(rows, dtype=torch.int32)
    max_blocks = 16
    block_table = torch.randperm(rows * max_blocks, generator=g).view(rows, max_blocks).to(torch.int32)
    num_pages = rows * max_blocks
    theta = 10000.0

    def make_kv(device):
        if fp8:
            return KVLayer(torch.zeros((num_pages, hkv, page, hd), dtype=torch.uint8, device=device),
                           torch.zeros((num_pages, hkv, page, hd), dtype=torch.uint8, device=device),
                           torch.zeros((num_pages, hkv, page), dtype=torch.float32, device=device),
                           torch.zeros((num_pages, hkv, page), dtype=torch.float32, device=device), True, page)
        return KVLayer(torch.zeros((num_pages, hkv, page, hd), dtype=torch.bfloat16, device=device),
                       torch.zeros((num_pages, hkv, page, hd), dtype=torch.bfloat16, device=device), None, None, False, page)

    kv = make_kv(DEV)
    qout = torch.zeros((rows, hq * hd), dtype=torch.bfloat16, device=DEV)
    ph = fd.phase(fd.ROPE_KV, lw.w, lw.scale_t, xq, xs, n=n, k=d, ssq_in=ssq_in, norm_dim=d, eps=1e-6, y=qout, ldy=hq * hd,
                  ld_s_out=bn)
    # the descriptor holds raw addresses: the device copies must outlive the launch
    d_pos, d_seq, d_table = positions.to(DEV), seq_index.to(DEV), block_table.to(DEV)
    rope = fd.rope_desc(d_pos, d_seq, d_table, kv, hq, hkv, rd, theta)
    fd.launch([ph], rows, torch.device(DEV), rope, grid=grid, impl=impl)
    # reference: projection (fp32), norm factor, then the per-op rotary + append on CPU tensors
    norm = fd.ref_norm_factor(ssq_in, rows, d, 1e-6)
    qkv = fd.ref_plain(lw.w, lw.scale_t, xq, xs, rows, norm=norm)
    kv_ref = make_kv("cpu")
    q_ref = ops.rope_kv_append(qkv.clone(), positions, seq_index, block_table, kv_ref, hq, hkv, hd, theta, rd)
    close(qout, q_ref, name="q")
    blk = block_table[seq_index.long(), (positions // page).long()].long()
    off = (positions % page).long()
    if fp8:
        for name, got_v, got_s, want_v, want_s in (("k", kv.k, kv.k_scale, kv_ref.k, kv_ref.k_scale),
                                                   ("v", kv.v, kv.v_scale, kv_ref.v, kv_ref.v_scale)):
            gv = ref.from_e4m3(got_v.cpu()[blk, :, off]) * got_s.cpu()[blk, :, off].unsqueeze(-1)
            wv = ref.from_e4m3(want_v[blk, :, off]) * want_s[blk, :, off].unsqueeze(-1)
            assert torch.allclose(got_s.cpu()[blk, :, off], want_s[blk, :, off], rtol=2e-2), name
            amax = wv.abs().amax(dim=-1, keepdim=True)
            assert ((gv - wv).abs() <= 0.07 * wv.abs() + 0.04 * amax).all(), name
        # nothing outside the addressed slots was touched
        mask = torch.ones((num_pages, page), dtype=torch.bool)
        mask[blk, off] = False
        assert not kv.k.cpu().permute(0, 2, 1, 3)[mask].any()
    else:
        close(kv.k.cpu()[blk, :, off], kv_ref.k[blk, :, off], name="k pages")
        close(kv.v.cpu()[blk, :, off], kv_ref.v[blk, :, off], name="v pages")
    _status_ok()


@pytest.mark.parametrize("rows,grid", [(4, 148), (32, 148), (32, 5)])
@pytest.mark.parametrize("impl", IMPLS)
def test_four_phase_chain_matches_sequential_reference(impl, rows, grid):
    """o-proj -> gate/up -> down -> head as one launch: outputs of each phase feed the next through the grid barrier."""
    _chain(impl, rows, grid)


def _chain(impl, rows, grid):
    d, qs, ffn, vocab = 512, 256, 768, 1000
    bn = 16 if rows <= 16 else 32
    wo, wgu, wd, wh = _weights(d, qs, 1), _weights(2 * ffn, d, 2), _weights(d, ffn, 3), _weights(vocab, d, 4)
    aq, a_s = _acts(rows, qs, bn, 5)
    dev = torch.device(DEV)
    z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=DEV)
    h = (torch.randn(rows, d) * 0.8).bfloat16().to(DEV)
    h0 = h.clone()
    hq, hs, ssq = z((rows, d), torch.uint8), z((d // 128, bn), torch.float32), z((d // 128, bn), torch.float32)
    actq, acts = z((rows, ffn), torch.uint8), z((ffn // 128, bn), torch.float32)
    logits = z((rows, vocab), torch.bfloat16)
    eps = 1e-5
    phases = [
        fd.phase(fd.RESID_QUANT, wo.w, wo.scale_t, aq, a_s, n=d, k=qs, y=h, ldy=d, residual=h, q_out=hq, s_out=hs, ssq_out=ssq, ld_s_out=bn),
        fd.phase(fd.SILU_QUANT, wgu.w, wgu.scale_t, hq, hs, n=ffn, k=d, dual_off=ffn, ssq_in=ssq, norm_dim=d, eps=eps, q_out=actq, s_out=acts, ld_s_out=bn),
        fd.phase(fd.RESID_QUANT, wd.w, wd.scale_t, actq, acts, n=d, k=ffn, y=h, ldy=d, residual=h, q_out=hq, s_out=hs, ssq_out=ssq, ld_s_out=bn),
        fd.phase(fd.PLAIN, wh.w, wh.scale_t, hq, hs, n=vocab, k=d, ssq_in=ssq, norm_dim=d, eps=eps, y=logits, ldy=vocab, ld_s_out=bn),
    ]
    il = [None, fd.interleave_gate_up(wgu.w, wgu.scale_t, ffn), None, None]
    fd.launch(phases, rows, dev, grid=grid, impl=impl, interleaved=il)
    got_logits = logits.clone()
    # sequential reference with the kernel's rounding points
    h1 = ref.round_bf16(fd.ref_plain(wo.w, wo.scale_t, aq, a_s, rows, residual=h0))
    _, q1, s1, ssq1 = fd.ref_quant_rows(h1)
    n1 = torch.rsqrt(ssq1.sum(dim=0) / d + eps)
    act = ref.round_bf16(fd.ref_silu(wgu.w, wgu.scale_t, q1, s1, rows, ffn, ffn, n1))
    _, q2, s2, _ = fd.ref_quant_rows(act)
    h2 = ref.round_bf16(fd.ref_plain(wd.w, wd.scale_t, q2, s2, rows, residual=h1))
    _, q3, s3, ssq3 = fd.ref_quant_rows(h2)
    n3 = torch.rsqrt(ssq3.sum(dim=0) / d + eps)
    want = fd.ref_plain(wh.w, wh.scale_t, q3, s3, rows, norm=n3)
    close(h, h2, rtol=3e-2, atol_frac=1.5e-2, name="final residual stream")
    got, wantf = got_logits.float().cpu(), want
    assert ((got - wantf).norm() / wantf.norm()).item() < 3e-2
    # replays are bit-identical (fixed summation order of split tiles)
    h.copy_(h0)
    fd.launch(phases, rows, dev, grid=grid, impl=impl, interleaved=il)
    assert torch.equal(logits, got_logits)
    _status_ok()


def test_embed_quant():
    rows, d, vocab = 9, 512, 300
    table = (torch.randn(vocab, d) * 0.05).bfloat16().to(DEV)
    ids = torch.randint(0, vocab, (rows,), dtype=torch.int32).to(DEV)
    h = torch.zeros((rows, d), dtype=torch.bfloat16, device=DEV)
    q = torch.zeros((rows, d), dtype=torch.uint8, device=DEV)
    s = torch.zeros((d // 128, 16), dtype=torch.float32, device=DEV)
    ssq = torch.zeros((d // 128, 16), dtype=torch.float32, device=DEV)
    fd.embed_quant(table, ids, h, q, s, ssq)
    want = table[ids.long()]
    assert torch.equal(h, want)
    _, q_ref, s_ref, ssq_ref = fd.ref_quant_rows(want.float().cpu())
    assert torch.equal(q.cpu(), q_ref)
    assert torch.allclose(s.cpu()[:, :rows], s_ref, rtol=1e-6)
    assert torch.allclose(ssq.cpu()[:, :rows], ssq_ref, rtol=1e-5)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("batch", [1, 3, 16, 32])
def test_engine_decode_fused_matches_per_op_path(batch, impl, monkeypatch):
    """Whole decode steps: the fused chain and the per-op path produce the same greedy tokens and close logits."""
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.models.config import ModelConfig
    cfg = ModelConfig(name="t", n_layers=3, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
                      weight_format="fp8", kv_format="fp8", max_context=256)
    g = torch.Generator().manual_seed(batch)
    prompts = torch.randint(0, cfg.vocab, (batch, 40), generator=g).tolist()

    def run(fused: bool):
        monkeypatch.setenv("SLLM_FUSED_DECODE", "1" if fused else "0")
        monkeypatch.setenv("SLLM_FD_BACKEND", impl)
        eng = build_engine(cfg, DEV, seed=3, max_batch=32, use_cuda_graphs=False)
        seqs = [eng.new_sequence(p) for p in prompts]
        for s, t in zip(seqs, eng.prefill(seqs)):
            s.tokens.append(t)
        lg = eng.decode(seqs, sample=False).float().cpu().clone()
        toks = []
        for _ in range(6):
            out = eng.decode(seqs)
            toks.append(out)
            for s, t in zip(seqs, out):
                s.tokens.append(t)
        used = bool(eng.model._fused)
        for s in seqs:
            eng.free_sequence(s)
        return lg, toks, used

    lg_f, tok_f, used_f = run(True)
    lg_u, tok_u, used_u = run(False)
    assert used_f and not used_u
    # the two paths quantise at different points (before / after the norm factor), so they agree to FP8 noise, row by row
    row_err = (lg_f - lg_u).norm(dim=-1) / lg_u.norm(dim=-1)
    assert row_err.max().item() < 0.08, row_err
    top2 = lg_u.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.1 * lg_u.abs().max()
    assert torch.equal(lg_f.argmax(-1)[clear], lg_u.argmax(-1)[clear])
    _status_ok()
