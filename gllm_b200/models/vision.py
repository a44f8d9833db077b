"""SigLIP-style vision tower: patch embedding, learned 2-D positions, pre-LN transformer encoder, projector into
the language model's hidden size.

Reference parity: SigLIP ViT graph ops ``PatchEmbed`` / ``LearnedPos2D`` (CLAUDE.md:996-1007;
src/compat/vision_forward.rs). Compute only; images arrive as tensors (no decoding / graphics API here).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops


@dataclass
class VisionConfig:
    image_size: int = 224
    patch_size: int = 14
    channels: int = 3
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    mlp: int = 3072
    eps: float = 1e-6
    out_hidden: int = 0        # projector width (LLM hidden); 0 = no projector
    pool: int = 1              # average-pool factor over the patch grid before projecting

    @property
    def grid(self) -> int:
        return self.image_size // self.patch_size

    @property
    def num_patches(self) -> int:
        return self.grid * self.grid


class VisionWeights:
    """Random-init weights of the tower (deterministic), or a dict of tensors with the same names."""

    def __init__(self, cfg: VisionConfig, device="cpu", dtype=torch.float32, seed=0, tensors: Optional[dict] = None):
        g = torch.Generator().manual_seed(seed)
        mk = lambda *s, std=0.02: (torch.randn(*s, generator=g) * std).to(device, dtype)
        H = cfg.hidden
        # supplied tensors move to the tower's device; matrices take its dtype, norm weights and biases stay as they are
        t = {k: (v.to(device, dtype) if v.dim() >= 2 else v.to(device)) for k, v in (tensors or {}).items()}
        pd = cfg.channels * cfg.patch_size * cfg.patch_size
        self.patch_w = t.get("patch_embed.weight", mk(H, pd))
        self.patch_b = t.get("patch_embed.bias", torch.zeros(H, device=device, dtype=torch.float32))
        self.pos = t.get("pos_embed", mk(cfg.num_patches, H))
        self.layers = []
        for l in range(cfg.layers):
            p = f"layers.{l}."
            self.layers.append({
                "ln1_w": t.get(p + "ln1.weight", torch.ones(H, device=device)), "ln1_b": t.get(p + "ln1.bias", torch.zeros(H, device=device)),
                "qkv_w": t.get(p + "qkv.weight", mk(3 * H, H)), "qkv_b": t.get(p + "qkv.bias", torch.zeros(3 * H, device=device)),
                "o_w": t.get(p + "o.weight", mk(H, H)), "o_b": t.get(p + "o.bias", torch.zeros(H, device=device)),
                "ln2_w": t.get(p + "ln2.weight", torch.ones(H, device=device)), "ln2_b": t.get(p + "ln2.bias", torch.zeros(H, device=device)),
                "fc1_w": t.get(p + "fc1.weight", mk(cfg.mlp, H)), "fc1_b": t.get(p + "fc1.bias", torch.zeros(cfg.mlp, device=device)),
                "fc2_w": t.get(p + "fc2.weight", mk(H, cfg.mlp)), "fc2_b": t.get(p + "fc2.bias", torch.zeros(H, device=device)),
            })
        self.post_w = t.get("post_ln.weight", torch.ones(H, device=device))
        self.post_b = t.get("post_ln.bias", torch.zeros(H, device=device))
        self.proj_w = t.get("proj.weight", mk(cfg.out_hidden, H)) if cfg.out_hidden else None


def siglip_tensors(cfg: VisionConfig, get, has=None, prefix: str = "vision_model.") -> dict:
    """Checkpoint tensors of a SigLIP / CLIP style vision tower under their Hugging Face names -> the names
    ``VisionWeights`` reads: the convolutional patch embedding [H, C, p, p] becomes a [H, C * p * p] matrix, the three
    attention projections of a layer are stacked into one qkv matrix. ``get(name)`` returns a tensor, ``has(name)``
    (optional) says whether it exists. Reference: SigLIP tower weights behind the multimodal projector
    (src/arch/auto_graph_fragments/build_graph.inc.rs vision branch, src/loader/name_map.rs)."""
    has = has or (lambda n: True)
    t = {}
    pe = get(prefix + "embeddings.patch_embedding.weight")
    t["patch_embed.weight"] = pe.reshape(pe.shape[0], -1)
    if has(prefix + "embeddings.patch_embedding.bias"):
        t["patch_embed.bias"] = get(prefix + "embeddings.patch_embedding.bias").float()
    t["pos_embed"] = get(prefix + "embeddings.position_embedding.weight")
    for l in range(cfg.layers):
        src, dst = f"{prefix}encoder.layers.{l}.", f"layers.{l}."
        t[dst + "ln1.weight"], t[dst + "ln1.bias"] = get(src + "layer_norm1.weight"), get(src + "layer_norm1.bias")
        t[dst + "ln2.weight"], t[dst + "ln2.bias"] = get(src + "layer_norm2.weight"), get(src + "layer_norm2.bias")
        t[dst + "qkv.weight"] = torch.cat([get(src + f"self_attn.{n}_proj.weight") for n in "qkv"], 0)
        t[dst + "qkv.bias"] = torch.cat([get(src + f"self_attn.{n}_proj.bias") for n in "qkv"], 0)
        t[dst + "o.weight"], t[dst + "o.bias"] = get(src + "self_attn.out_proj.weight"), get(src + "self_attn.out_proj.bias")
        t[dst + "fc1.weight"], t[dst + "fc1.bias"] = get(src + "mlp.fc1.weight"), get(src + "mlp.fc1.bias")
        t[dst + "fc2.weight"], t[dst + "fc2.bias"] = get(src + "mlp.fc2.weight"), get(src + "mlp.fc2.bias")
    t["post_ln.weight"], t["post_ln.bias"] = get(prefix + "post_layernorm.weight"), get(prefix + "post_layernorm.bias")
    for cand in ("multi_modal_projector.linear.weight", "multi_modal_projector.mm_input_projection_weight"):
        if cfg.out_hidden and has(cand):
            w = get(cand)
            t["proj.weight"] = w if w.shape[0] == cfg.out_hidden else w.t().contiguous()
            break
    return t


def patchify(images: torch.Tensor, patch: int) -> torch.Tensor:
    """[B, C, H, W] -> [B, patches, C*patch*patch] (row-major patch grid; conv with stride = kernel as a GEMM)."""
    B, C, H, W = images.shape
    x = images.reshape(B, C, H // patch, patch, W // patch, patch).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(B, (H // patch) * (W // patch), C * patch * patch)


def _linear(x, w, b):
    y = ops.gemm(x.reshape(-1, x.shape[-1]).contiguous(), w, out_dtype=x.dtype, bias=b.float() if b is not None else None)
    return y[:, :w.shape[0]].reshape(*x.shape[:-1], w.shape[0])


class VisionTower:
    def __init__(self, cfg: VisionConfig, weights: VisionWeights):
        self.cfg, self.w = cfg, weights

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        """images [B, C, H, W] in [-1, 1] -> [B, tokens, out_hidden or hidden]."""
        c, w = self.cfg, self.w
        dt = w.patch_w.dtype
        x = _linear(patchify(images.to(dt), c.patch_size), w.patch_w, w.patch_b) + w.pos[None].to(dt)
        B, N, H = x.shape
        hd = H // c.heads
        for lw in w.layers:
            h = F.layer_norm(x.float(), (H,), lw["ln1_w"].float(), lw["ln1_b"].float(), c.eps).to(dt)
            qkv = _linear(h, lw["qkv_w"], lw["qkv_b"]).reshape(B, N, 3, c.heads, hd).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])            # bidirectional
            x = x + _linear(a.transpose(1, 2).reshape(B, N, H), lw["o_w"], lw["o_b"])
            h = F.layer_norm(x.float(), (H,), lw["ln2_w"].float(), lw["ln2_b"].float(), c.eps).to(dt)
            h = F.gelu(_linear(h, lw["fc1_w"], lw["fc1_b"]).float(), approximate="tanh").to(dt)
            x = x + _linear(h, lw["fc2_w"], lw["fc2_b"])
        x = F.layer_norm(x.float(), (H,), w.post_w.float(), w.post_b.float(), c.eps).to(dt)
        if c.pool > 1:
            g = c.grid
            x = F.avg_pool2d(x.reshape(B, g, g, H).permute(0, 3, 1, 2).float(), c.pool).flatten(2).transpose(1, 2).to(dt)
        if w.proj_w is not None:
            x = _linear(x, w.proj_w, None)
        return x
