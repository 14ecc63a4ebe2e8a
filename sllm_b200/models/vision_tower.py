"""Vision tower of a Qwen-VL-class multimodal model: patch embedding, learned position table, a stack of
pre-LayerNorm transformer blocks with 2-D rotary attention over the patches of one image, and the 2 x 2 patch
merger that projects into the language model's width.

Tensor inventory per the reference's 297-tensor manifest (crates/sllm-core/src/qwen_vision.rs): patch embedding
(weight, bias), position table, 24 blocks x 12 tensors (norm1, norm2, attn.qkv, attn.proj, mlp.linear_fc1,
mlp.linear_fc2, each weight + bias), merger (norm, linear_fc1, linear_fc2, each weight + bias).  As in the
reference's executor (crates/sllm-core/src/qwen_vision_execution.rs:1-8) the dense projections run through the
GEMM op of the device (tcgen05 on a GPU) and the small transforms (LayerNorm, bias, GELU, the per-image softmax)
are plain tensor code: an image is encoded once per request, off the decode path.

`assemble_multimodal` splices the merged patch rows into the token embeddings at the image placeholder tokens and
returns the 3-axis (temporal, height, width) position ids of the whole prompt.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..ops.core import LinearWeight


@dataclass
class VisionConfig:
    depth: int = 24
    hidden: int = 1024
    heads: int = 16
    intermediate: int = 4096
    out_hidden: int = 2560
    patch: int = 16
    temporal_patch: int = 2
    merge: int = 2
    in_channels: int = 3
    position_grid: int = 48            # the learned table covers position_grid x position_grid patches
    ln_eps: float = 1e-6
    rope_theta: float = 10000.0

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch * self.patch * self.patch

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


def tiny_vision() -> VisionConfig:
    return VisionConfig(depth=2, hidden=64, heads=4, intermediate=128, out_hidden=256, position_grid=8)


@dataclass
class VisionBlock:
    norm1_w: torch.Tensor
    norm1_b: torch.Tensor
    norm2_w: torch.Tensor
    norm2_b: torch.Tensor
    qkv: LinearWeight
    qkv_b: torch.Tensor
    proj: LinearWeight
    proj_b: torch.Tensor
    fc1: LinearWeight
    fc1_b: torch.Tensor
    fc2: LinearWeight
    fc2_b: torch.Tensor


@dataclass
class VisionWeights:
    patch_w: LinearWeight              # [hidden, patch_dim] (the 3-D convolution with stride = kernel, flattened)
    patch_b: torch.Tensor
    pos_table: torch.Tensor            # [position_grid ** 2, hidden]
    blocks: list = field(default_factory=list)
    merger_norm_w: Optional[torch.Tensor] = None
    merger_norm_b: Optional[torch.Tensor] = None
    merger_fc1: Optional[LinearWeight] = None      # [merge^2 * hidden, merge^2 * hidden]
    merger_fc1_b: Optional[torch.Tensor] = None
    merger_fc2: Optional[LinearWeight] = None      # [out_hidden, merge^2 * hidden]
    merger_fc2_b: Optional[torch.Tensor] = None

    def tensor_count(self) -> int:
        return 3 + 12 * len(self.blocks) + 6


def init_random_vision_weights(cfg: VisionConfig, device, seed: int = 0, dtype=torch.bfloat16) -> VisionWeights:
    gen = torch.Generator().manual_seed(seed)
    dev = torch.device(device)

    def rnd(shape, std):
        return (torch.randn(shape, generator=gen) * std).to(dtype).to(dev).contiguous()

    def lin(n, k):
        return LinearWeight("dense", rnd((n, k), 1.0 / math.sqrt(k))), rnd((n,), 0.02)

    def ln():
        return (1.0 + 0.05 * torch.randn((cfg.hidden,), generator=gen)).to(dtype).to(dev), rnd((cfg.hidden,), 0.02)

    pw, pb = lin(cfg.hidden, cfg.patch_dim)
    w = VisionWeights(pw, pb, rnd((cfg.position_grid ** 2, cfg.hidden), 0.02))
    for _ in range(cfg.depth):
        n1w, n1b = ln()
        n2w, n2b = ln()
        qkv, qkv_b = lin(3 * cfg.hidden, cfg.hidden)
        proj, proj_b = lin(cfg.hidden, cfg.hidden)
        fc1, fc1_b = lin(cfg.intermediate, cfg.hidden)
        fc2, fc2_b = lin(cfg.hidden, cfg.intermediate)
        w.blocks.append(VisionBlock(n1w, n1b, n2w, n2b, qkv, qkv_b, proj, proj_b, fc1, fc1_b, fc2, fc2_b))
    m = cfg.merge * cfg.merge * cfg.hidden
    w.merger_norm_w, w.merger_norm_b = ln()
    w.merger_fc1, w.merger_fc1_b = lin(m, m)
    w.merger_fc2, w.merger_fc2_b = lin(cfg.out_hidden, m)
    return w


def patch_rows_cols(grid_thw: tuple, merge: int):
    """(row, column) of every patch in the preprocessor's order: merge blocks row-major, patches of a block
    row-major inside it (frontend.vision.process_image), repeated per temporal slice."""
    t, gh, gw = grid_thw
    br, bc, mr, mc = np.meshgrid(np.arange(gh // merge), np.arange(gw // merge), np.arange(merge), np.arange(merge),
                                 indexing="ij")
    rows = (br * merge + mr).reshape(-1)
    cols = (bc * merge + mc).reshape(-1)
    return np.tile(rows, t), np.tile(cols, t)


class VisionTower:
    def __init__(self, cfg: VisionConfig, weights: VisionWeights):
        if cfg.head_dim % 4:
            raise ValueError("2-D rotary attention needs a head size divisible by 4")
        self.cfg, self.w = cfg, weights

    # ------------------------------------------------------------------ pieces
    def _linear(self, x: torch.Tensor, w: LinearWeight, b: torch.Tensor) -> torch.Tensor:
        return ops.linear(x.contiguous(), w) + b

    def _positions(self, rows: np.ndarray, cols: np.ndarray, gh: int, gw: int, device, dtype) -> torch.Tensor:
        """Bilinear interpolation of the learned position_grid x position_grid table at the patch centres of a
        gh x gw grid (the table was trained on one grid size; other aspect ratios sample it)."""
        g = self.cfg.position_grid
        table = self.w.pos_table.float().view(g, g, -1)
        fr = torch.tensor(rows, dtype=torch.float32, device=device) * ((g - 1) / max(gh - 1, 1))
        fc = torch.tensor(cols, dtype=torch.float32, device=device) * ((g - 1) / max(gw - 1, 1))
        r0, c0 = fr.floor().long().clamp(0, g - 1), fc.floor().long().clamp(0, g - 1)
        r1, c1 = (r0 + 1).clamp(max=g - 1), (c0 + 1).clamp(max=g - 1)
        ar, ac = (fr - r0).unsqueeze(1), (fc - c0).unsqueeze(1)
        out = (table[r0, c0] * (1 - ar) * (1 - ac) + table[r0, c1] * (1 - ar) * ac
               + table[r1, c0] * ar * (1 - ac) + table[r1, c1] * ar * ac)
        return out.to(dtype)

    def _rope(self, rows: np.ndarray, cols: np.ndarray, device):
        """cos / sin [N, head_dim / 2]: the first quarter of the rotary pairs turns with the patch row, the
        second with the column (split-half pairing: channel j rotates with channel j + head_dim / 2)."""
        hd = self.cfg.head_dim
        q = hd // 4
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(q, dtype=torch.float32, device=device) / q))
        r = torch.tensor(rows, dtype=torch.float32, device=device).unsqueeze(1) * inv
        c = torch.tensor(cols, dtype=torch.float32, device=device).unsqueeze(1) * inv
        ang = torch.cat([r, c], dim=1)                    # [N, hd / 2]
        return ang.cos(), ang.sin()

    @staticmethod
    def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """x [N, heads, hd] in fp32."""
        half = x.shape[-1] // 2
        a, b = x[..., :half], x[..., half:]
        c, s = cos.unsqueeze(1), sin.unsqueeze(1)
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    # ------------------------------------------------------------------ forward
    def forward(self, patches: torch.Tensor, grid_thw: tuple) -> torch.Tensor:
        """patches [N, patch_dim] of ONE image in the preprocessor's order -> merged visual rows
        [N / merge^2, out_hidden].  Attention is full (not causal) over the patches of the image."""
        cfg, w = self.cfg, self.w
        t, gh, gw = grid_thw
        n = t * gh * gw
        if patches.shape != (n, cfg.patch_dim):
            raise ValueError(f"expected patches [{n}, {cfg.patch_dim}], got {tuple(patches.shape)}")
        dt = w.patch_b.dtype
        dev = patches.device
        rows, cols = patch_rows_cols(grid_thw, cfg.merge)
        x = self._linear(patches.to(dt), w.patch_w, w.patch_b)
        x = x + self._positions(rows, cols, gh, gw, dev, dt)
        cos, sin = self._rope(rows, cols, dev)
        h, hd = cfg.heads, cfg.head_dim
        for blk in w.blocks:
            y = F.layer_norm(x.float(), (cfg.hidden,), blk.norm1_w.float(), blk.norm1_b.float(), cfg.ln_eps).to(dt)
            qkv = self._linear(y, blk.qkv, blk.qkv_b).float().view(n, 3, h, hd)
            q, k, v = self._rotate(qkv[:, 0], cos, sin), self._rotate(qkv[:, 1], cos, sin), qkv[:, 2]
            att = torch.einsum("qhd,khd->hqk", q, k) * (1.0 / math.sqrt(hd))
            o = torch.einsum("hqk,khd->qhd", att.softmax(dim=-1), v).reshape(n, cfg.hidden).to(dt)
            x = x + self._linear(o, blk.proj, blk.proj_b)
            y = F.layer_norm(x.float(), (cfg.hidden,), blk.norm2_w.float(), blk.norm2_b.float(), cfg.ln_eps).to(dt)
            y = F.gelu(self._linear(y, blk.fc1, blk.fc1_b).float(), approximate="tanh").to(dt)
            x = x + self._linear(y, blk.fc2, blk.fc2_b)
        y = F.layer_norm(x.float(), (cfg.hidden,), w.merger_norm_w.float(), w.merger_norm_b.float(), cfg.ln_eps).to(dt)
        y = y.view(n // (cfg.merge * cfg.merge), cfg.merge * cfg.merge * cfg.hidden)   # 4 consecutive patches = 1 block
        y = F.gelu(self._linear(y, w.merger_fc1, w.merger_fc1_b).float()).to(dt)
        return self._linear(y, w.merger_fc2, w.merger_fc2_b)


def reference_forward(cfg: VisionConfig, w: VisionWeights, patches: torch.Tensor, grid_thw: tuple) -> torch.Tensor:
    """The same network in fp32 torch.nn.functional calls on the CPU (the oracle of the tests)."""
    def f(t):
        return t.detach().float().cpu()

    def lin(x, lw, b):
        return F.linear(x, f(lw.w), f(b))
    tower = VisionTower(cfg, w)
    t, gh, gw = grid_thw
    n = t * gh * gw
    rows, cols = patch_rows_cols(grid_thw, cfg.merge)
    x = lin(f(patches), w.patch_w, w.patch_b) + f(tower._positions(rows, cols, gh, gw, w.pos_table.device, torch.float32))
    cos, sin = (f(z) for z in tower._rope(rows, cols, w.pos_table.device))
    h, hd = cfg.heads, cfg.head_dim
    for blk in w.blocks:
        y = F.layer_norm(x, (cfg.hidden,), f(blk.norm1_w), f(blk.norm1_b), cfg.ln_eps)
        qkv = lin(y, blk.qkv, blk.qkv_b).view(n, 3, h, hd)
        q, k, v = tower._rotate(qkv[:, 0], cos, sin), tower._rotate(qkv[:, 1], cos, sin), qkv[:, 2]
        o = F.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1)).transpose(0, 1)
        x = x + lin(o.reshape(n, cfg.hidden), blk.proj, blk.proj_b)
        y = F.layer_norm(x, (cfg.hidden,), f(blk.norm2_w), f(blk.norm2_b), cfg.ln_eps)
        x = x + lin(F.gelu(lin(y, blk.fc1, blk.fc1_b), approximate="tanh"), blk.fc2, blk.fc2_b)
    y = F.layer_norm(x, (cfg.hidden,), f(w.merger_norm_w), f(w.merger_norm_b), cfg.ln_eps)
    y = y.view(n // (cfg.merge * cfg.merge), -1)
    return lin(F.gelu(lin(y, w.merger_fc1, w.merger_fc1_b)), w.merger_fc2, w.merger_fc2_b)


def assemble_multimodal(tokens: list, image_token_id: int, token_embeds: torch.Tensor, images: list, merge: int = 2):
    """Splices visual rows into a prompt.

    tokens        prompt ids; every image occupies one run of `image_token_id` as long as its merged grid
    token_embeds  [T, d] embeddings of `tokens` (placeholder rows are overwritten)
    images        [(visual_rows [n_i, d], grid_thw)] in prompt order
    Returns (embeds [T, d], positions int32 [3, T]): text tokens advance the temporal, height and width axes
    together; the tokens of an image share the temporal index and enumerate the merged grid; text after an image
    continues from the largest index used so far + 1 (the reference's multimodal prompt assembly,
    crates/sllm-core/src/qwen_vision_execution.rs)."""
    t_total = len(tokens)
    if token_embeds.shape[0] != t_total:
        raise ValueError("one embedding row per token is required")
    out = token_embeds.clone()
    pos = np.zeros((3, t_total), dtype=np.int32)
    i, nxt, img = 0, 0, 0
    while i < t_total:
        if tokens[i] != image_token_id:
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        if img >= len(images):
            raise ValueError("more image placeholder runs than images")
        rows, (t, gh, gw) = images[img]
        mh, mw = gh // merge, gw // merge
        n = t * mh * mw
        if rows.shape[0] != n or tokens[i:i + n] != [image_token_id] * n:
            raise ValueError(f"image {img}: the placeholder run does not match its {n} visual tokens")
        if i + n < t_total and tokens[i + n] == image_token_id:
            raise ValueError(f"image {img}: the placeholder run is longer than its {n} visual tokens")
        out[i:i + n] = rows.to(out.dtype)
        tt = np.repeat(np.arange(t, dtype=np.int32), mh * mw)
        hh = np.tile(np.repeat(np.arange(mh, dtype=np.int32), mw), t)
        ww = np.tile(np.arange(mw, dtype=np.int32), t * mh)
        pos[0, i:i + n], pos[1, i:i + n], pos[2, i:i + n] = nxt + tt, nxt + hh, nxt + ww
        nxt += max(t, mh, mw)
        i += n
        img += 1
    if img != len(images):
        raise ValueError("fewer image placeholder runs than images")
    return out, pos


IMAGE_MARKER = "<|image_pad|>"


def encode_with_images(tokenizer, text: str, image_token_id: int) -> list:
    """Token ids of `text` in which every IMAGE_MARKER becomes one `image_token_id` (tokenizers that do not know
    the marker as a special token would otherwise spell it out)."""
    parts = text.split(IMAGE_MARKER)
    ids = []
    for i, part in enumerate(parts):
        if i:
            ids.append(image_token_id)
        if part:
            ids.extend(tokenizer.encode(part))
    return ids


class MultimodalPrompt:
    """A prompt with images, ready for the engine: `tokens` carries one placeholder run per image (as long as the
    image's merged grid), and calling the object with the engine returns (embeds [T, d], rope_pos3 int32 [3, T])
    for `Engine.prefill`.  The tower runs when the request is scheduled, on the engine's device."""

    def __init__(self, tower: VisionTower, images: list, prompt_ids: list, image_token_id: int):
        merge2 = tower.cfg.merge * tower.cfg.merge
        if sum(1 for t in prompt_ids if t == image_token_id) != len(images):
            raise ValueError("the prompt needs exactly one image placeholder per image")
        self.tower, self.images, self.image_token_id = tower, images, image_token_id
        self.tokens, k = [], 0
        for t in prompt_ids:
            if t == image_token_id:
                g = images[k].grid_thw
                self.tokens.extend([image_token_id] * (g[0] * g[1] * g[2] // merge2))
                k += 1
            else:
                self.tokens.append(t)

    def __call__(self, engine):
        dev = engine.device
        w = engine.model.w
        rows = []
        for img in self.images:
            patches = torch.from_numpy(np.ascontiguousarray(img.patches)).to(dev)
            rows.append((self.tower.forward(patches, img.grid_thw), img.grid_thw))
        # the placeholder id may lie outside the embedding table: embed a harmless id there, the rows are overwritten
        ids = [0 if t == self.image_token_id else t for t in self.tokens]
        emb = ops.embedding(w.embed, torch.tensor(ids, dtype=torch.int32, device=dev), engine.cfg.embedding_scale)
        embeds, pos3 = assemble_multimodal(self.tokens, self.image_token_id, emb, rows, self.tower.cfg.merge)
        return embeds.contiguous(), torch.from_numpy(pos3).to(dev)
