"""Vision-language support: a ViT image tower (Qwen2-VL and Qwen2.5-VL layouts), the image
pre-processor that turns pictures into flattened patches, multimodal rotary position ids
(M-RoPE), and the wrapper that splices image features into the decoder's token embeddings.

Reference behaviour: the reference trains VLMs through HF ``AutoModelForImageTextToText``
(``areal/engine/fsdp_engine.py:375-560``), computes M-RoPE ids per sample
(``areal/models/transformers/qwen2_vl.py``, ``qwen3_vl.py``) and carries the pixel data as
``multi_modal_input`` entries of the trajectory (``areal/workflow/vision_rlvr.py``). Here the
tower is part of the model zoo; its parameter names are the HF ones (``visual.*``), so
checkpoints map one to one.

Layout facts this file relies on (they define checkpoint compatibility):

* patches arrive flattened as ``[N, C * Tp * P * P]`` in the order (frame, h-block, w-block,
  h-in-block, w-in-block): the ``m x m`` patches that the merger fuses are adjacent rows;
* 2-D rotary embedding: half of each head's rotary pairs turn with the patch's row index, the
  other half with its column index;
* Qwen2-VL blocks: LayerNorm, biased QKV / proj, QuickGELU MLP, full attention inside a frame;
  Qwen2.5-VL blocks: RMSNorm, SwiGLU MLP with biases, attention inside ``window_size`` pixel
  windows except on the ``fullatt_block_indexes`` layers (tokens are re-ordered window by
  window once, and the merger's output is put back in raster order);
* the merger normalises, concatenates each ``m x m`` group and projects to the decoder width.

The tower's attention runs on ``scaled_dot_product_attention`` (head size 80 is outside the
64 / 128 the flash kernels cover); its linear layers use the framework's GEMM kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class VisionConfig:
    arch: str = "qwen2_vl"              # qwen2_vl | qwen2_5_vl | qwen3_vl
    depth: int = 32
    embed_dim: int = 1280
    num_heads: int = 16
    mlp_hidden: int = 5120
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    window_size: int = 0                # pixels; 0 = full attention everywhere
    fullatt_block_indexes: list[int] = field(default_factory=list)
    # qwen3_vl: learned position table (a square grid, bilinearly resampled to the image grid) and
    # "deep stack" taps: the outputs of these blocks are merged and added to the hidden states of
    # the first decoder layers at the image positions
    num_position_embeddings: int = 0
    deepstack_visual_indexes: list[int] = field(default_factory=list)

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2

    @classmethod
    def from_hf_dict(cls, d: dict, llm_hidden: int, arch: str) -> "VisionConfig":
        if arch == "qwen3_vl":
            return cls(arch=arch, depth=d.get("depth", 27), embed_dim=d.get("hidden_size", 1152), num_heads=d.get("num_heads", 16),
                       mlp_hidden=d.get("intermediate_size", 4304), in_channels=d.get("in_channels", d.get("in_chans", 3)),
                       patch_size=d.get("patch_size", 16), temporal_patch_size=d.get("temporal_patch_size", 2),
                       spatial_merge_size=d.get("spatial_merge_size", 2), out_hidden_size=d.get("out_hidden_size", llm_hidden),
                       num_position_embeddings=d.get("num_position_embeddings", 2304),
                       deepstack_visual_indexes=list(d.get("deepstack_visual_indexes", [8, 16, 24])))
        if arch == "qwen2_5_vl":
            return cls(arch=arch, depth=d.get("depth", 32), embed_dim=d.get("hidden_size", 1280), num_heads=d.get("num_heads", 16),
                       mlp_hidden=d.get("intermediate_size", 3420), in_channels=d.get("in_chans", d.get("in_channels", 3)),
                       patch_size=d.get("patch_size", 14), temporal_patch_size=d.get("temporal_patch_size", 2),
                       spatial_merge_size=d.get("spatial_merge_size", 2), out_hidden_size=d.get("out_hidden_size", llm_hidden),
                       window_size=d.get("window_size", 112), fullatt_block_indexes=list(d.get("fullatt_block_indexes", [7, 15, 23, 31])))
        e = d.get("embed_dim", 1280)
        return cls(arch="qwen2_vl", depth=d.get("depth", 32), embed_dim=e, num_heads=d.get("num_heads", 16),
                   mlp_hidden=int(e * d.get("mlp_ratio", 4)), in_channels=d.get("in_chans", d.get("in_channels", 3)),
                   patch_size=d.get("patch_size", 14), temporal_patch_size=d.get("temporal_patch_size", 2),
                   spatial_merge_size=d.get("spatial_merge_size", 2), out_hidden_size=d.get("hidden_size", llm_hidden))

    def to_hf_dict(self) -> dict:
        if self.arch == "qwen3_vl":
            return dict(depth=self.depth, hidden_size=self.embed_dim, intermediate_size=self.mlp_hidden, num_heads=self.num_heads,
                        in_channels=self.in_channels, patch_size=self.patch_size, temporal_patch_size=self.temporal_patch_size,
                        spatial_merge_size=self.spatial_merge_size, out_hidden_size=self.out_hidden_size, hidden_act="gelu_pytorch_tanh",
                        num_position_embeddings=self.num_position_embeddings, deepstack_visual_indexes=list(self.deepstack_visual_indexes),
                        model_type="qwen3_vl")
        if self.arch == "qwen2_5_vl":
            return dict(depth=self.depth, hidden_size=self.embed_dim, intermediate_size=self.mlp_hidden, num_heads=self.num_heads,
                        in_chans=self.in_channels, patch_size=self.patch_size, temporal_patch_size=self.temporal_patch_size,
                        spatial_merge_size=self.spatial_merge_size, out_hidden_size=self.out_hidden_size, window_size=self.window_size,
                        fullatt_block_indexes=list(self.fullatt_block_indexes), model_type="qwen2_5_vl")
        return dict(depth=self.depth, embed_dim=self.embed_dim, mlp_ratio=self.mlp_hidden / self.embed_dim, num_heads=self.num_heads,
                    in_chans=self.in_channels, patch_size=self.patch_size, temporal_patch_size=self.temporal_patch_size,
                    spatial_merge_size=self.spatial_merge_size, hidden_size=self.out_hidden_size, model_type="qwen2_vl")


# --------------------------------------------------------------------------- image -> patches
def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    """Size (multiples of ``factor``) closest to the input whose area lies in the pixel budget."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def preprocess_images(images: Sequence, cfg: Optional[VisionConfig] = None, min_pixels: int = 56 * 56,
                      max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[torch.Tensor, torch.Tensor]:
    """PIL images (or ``[H, W, 3]`` uint8 arrays) -> (``pixel_values [N, C*Tp*P*P]`` fp32,
    ``image_grid_thw [n, 3]``): resize to a multiple of ``patch * merge``, scale to [0, 1],
    normalise with the CLIP statistics, repeat the frame ``Tp`` times, cut into patches in
    merge-block order."""
    cfg = cfg or VisionConfig()
    P, m, Tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    # Qwen3-VL checkpoints were trained with 0.5 / 0.5 normalisation, the earlier families with the CLIP statistics
    mean = np.asarray((0.5, 0.5, 0.5) if cfg.arch == "qwen3_vl" else CLIP_MEAN, dtype=np.float32).reshape(1, 1, 3)
    std = np.asarray((0.5, 0.5, 0.5) if cfg.arch == "qwen3_vl" else CLIP_STD, dtype=np.float32).reshape(1, 1, 3)
    outs, grids = [], []
    for im in images:
        if not isinstance(im, np.ndarray):
            im = im.convert("RGB")
            h, w = smart_resize(im.height, im.width, P * m, min_pixels, max_pixels)
            from PIL import Image

            arr = np.asarray(im.resize((w, h), resample=Image.BICUBIC), dtype=np.float32)
        else:
            from PIL import Image

            h, w = smart_resize(im.shape[0], im.shape[1], P * m, min_pixels, max_pixels)
            arr = np.asarray(Image.fromarray(im.astype(np.uint8)).resize((w, h), resample=Image.BICUBIC), dtype=np.float32)
        arr = (arr / 255.0 - mean) / std                                       # [h, w, 3]
        chw = np.ascontiguousarray(arr.transpose(2, 0, 1))                     # [C, h, w]
        frames = np.stack([chw] * Tp, axis=0)[None]                            # [grid_t = 1, Tp, C, h, w]
        gh, gw = h // P, w // P
        x = frames.reshape(1, Tp, cfg.in_channels, gh // m, m, P, gw // m, m, P)
        x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                             # t, hb, wb, mh, mw, C, Tp, P, P
        outs.append(torch.from_numpy(np.ascontiguousarray(x).reshape(gh * gw, cfg.patch_dim)))
        grids.append([1, gh, gw])
    if not outs:
        return torch.zeros(0, cfg.patch_dim), torch.zeros(0, 3, dtype=torch.long)
    return torch.cat(outs, 0), torch.tensor(grids, dtype=torch.long)


def num_image_tokens(grid_thw: torch.Tensor, merge: int = 2) -> list[int]:
    """Placeholder tokens each image occupies in the text sequence."""
    return [int(t * h * w) // (merge * merge) for t, h, w in grid_thw.tolist()]


# --------------------------------------------------------------------------- M-RoPE
def mrope_position_ids(input_ids: torch.Tensor, grid_thw: Optional[torch.Tensor], image_token_id: int, merge: int = 2,
                       video_token_id: Optional[int] = None, image_positions: Optional[list] = None) -> tuple[torch.Tensor, int]:
    """Three position streams (temporal, height, width) for ONE sequence. Text tokens advance all
    three together; a run of image placeholders takes (frame, row, column) of its merged grid,
    offset by the position reached so far; the text after it continues from the largest index
    used plus one. Returns (``[3, L]`` int64, ``delta``) where ``delta + L`` is the position of
    the next generated token. Placeholder ids beyond the given grids (a model may *generate* one)
    count as text. ``image_positions``, when given, receives the indices that hold image features."""
    ids = input_ids.tolist()
    L = len(ids)
    pos = torch.zeros(3, L, dtype=torch.long)
    grids = grid_thw.tolist() if grid_thw is not None else []
    special = {image_token_id} | ({video_token_id} if video_token_id is not None else set())
    i, nxt, img = 0, 0, 0
    while i < L:
        if ids[i] in special and img < len(grids):
            t, h, w = grids[img]
            lh, lw = h // merge, w // merge
            n = t * lh * lw
            if i + n > L:
                raise ValueError("image placeholder run is shorter than its grid")
            tt = torch.arange(t).repeat_interleave(lh * lw)
            hh = torch.arange(lh).repeat_interleave(lw).repeat(t)
            ww = torch.arange(lw).repeat(t * lh)
            pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            if image_positions is not None:
                image_positions.extend(range(i, i + n))
            nxt = int(pos[:, i:i + n].max()) + 1
            i += n
            img += 1
        else:
            j = i
            while j < L and not (ids[j] in special and img < len(grids)):
                j += 1
            pos[:, i:j] = torch.arange(nxt, nxt + (j - i))
            nxt += j - i
            i = j
    return pos, nxt - L


def mrope_tables(pos3: torch.Tensor, head_dim: int, theta: float, sections: Sequence[int], device,
                 interleaved: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token cos / sin rows ``[T, head_dim / 2]``: frequency ``f`` turns with the temporal,
    height or width stream according to the section it falls in (``sum(sections) = head_dim / 2``).
    ``interleaved`` (Qwen3-VL): the streams alternate t, h, w, t, h, w, ... over the first
    ``3 * sections[1]`` (height) / ``3 * sections[2]`` (width) frequencies instead of forming three
    contiguous runs; everything else turns with the temporal stream."""
    half = head_dim // 2
    if sum(sections) != half:
        raise ValueError(f"mrope sections {list(sections)} must sum to {half}")
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64, device=device) * 2 / head_dim))
    if interleaved:
        which = torch.zeros(half, dtype=torch.long, device=device)
        which[1:3 * sections[1]:3] = 1
        which[2:3 * sections[2]:3] = 2
    else:
        which = torch.repeat_interleave(torch.arange(3, device=device), torch.tensor(list(sections), device=device))
    p = pos3.to(device=device, dtype=torch.float64)[which]                        # [half, T]
    ang = (p * inv[:, None]).t()
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


# --------------------------------------------------------------------------- tower
class _Lin(nn.Module):
    def __init__(self, i: int, o: int, dtype, device, bias: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        if x.is_cuda and x.shape[0] > 0 and x.shape[-1] % 64 == 0 and self.weight.shape[0] % 64 == 0 and x.dtype == torch.bfloat16:
            y = OF.linear(x.contiguous(), self.weight)
            return y if self.bias is None else y + self.bias
        return F.linear(x, self.weight, self.bias)


class _Norm(nn.Module):
    def __init__(self, dim: int, rms: bool, dtype, device, eps: float = 1e-6):
        super().__init__()
        self.rms, self.eps = rms, eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = None if rms else nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        if self.rms:
            xf = x.float()
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight
        return F.layer_norm(x, (x.shape[-1],), self.weight, self.bias, self.eps)


class _PatchEmbed(nn.Module):
    """``Conv3d(C, E, kernel = stride = (Tp, P, P))`` on non-overlapping patches is one matmul on the
    flattened patch; the weight keeps the conv shape so checkpoints load unchanged."""

    def __init__(self, cfg: VisionConfig, dtype, device):
        super().__init__()
        self.proj = nn.Module()
        self.proj.weight = nn.Parameter(torch.empty(cfg.embed_dim, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size,
                                                    cfg.patch_size, dtype=dtype, device=device))
        self.proj.bias = nn.Parameter(torch.zeros(cfg.embed_dim, dtype=dtype, device=device)) if cfg.arch == "qwen3_vl" else None

    def forward(self, x):
        return F.linear(x.to(self.proj.weight.dtype), self.proj.weight.view(self.proj.weight.shape[0], -1), self.proj.bias)


class _VisionAttention(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device):
        super().__init__()
        self.nh, self.hd = cfg.num_heads, cfg.head_dim
        self.qkv = _Lin(cfg.embed_dim, 3 * cfg.embed_dim, dtype, device)
        self.proj = _Lin(cfg.embed_dim, cfg.embed_dim, dtype, device)

    def forward(self, x, cos, sin, bounds: list[int]):
        N = x.shape[0]
        q, k, v = self.qkv(x).view(N, 3, self.nh, self.hd).unbind(1)

        def rot(t):
            tf = t.float()
            a, b = tf[..., : self.hd // 2], tf[..., self.hd // 2:]
            return (tf * cos[:, None, :] + torch.cat([-b, a], -1) * sin[:, None, :]).to(t.dtype)

        q, k = rot(q), rot(k)
        outs = []
        for a, b in zip(bounds[:-1], bounds[1:]):        # attention never crosses a frame / window
            o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None], v[a:b].transpose(0, 1)[None])
            outs.append(o[0].transpose(0, 1))
        return self.proj(torch.cat(outs, 0).reshape(N, self.nh * self.hd))


class _VisionMLP(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device):
        super().__init__()
        self.gated = cfg.arch == "qwen2_5_vl"
        self.tanh_gelu = cfg.arch == "qwen3_vl"
        if self.tanh_gelu:
            self.linear_fc1 = _Lin(cfg.embed_dim, cfg.mlp_hidden, dtype, device)
            self.linear_fc2 = _Lin(cfg.mlp_hidden, cfg.embed_dim, dtype, device)
        elif self.gated:
            self.gate_proj = _Lin(cfg.embed_dim, cfg.mlp_hidden, dtype, device)
            self.up_proj = _Lin(cfg.embed_dim, cfg.mlp_hidden, dtype, device)
            self.down_proj = _Lin(cfg.mlp_hidden, cfg.embed_dim, dtype, device)
        else:
            self.fc1 = _Lin(cfg.embed_dim, cfg.mlp_hidden, dtype, device)
            self.fc2 = _Lin(cfg.mlp_hidden, cfg.embed_dim, dtype, device)

    def forward(self, x):
        if self.tanh_gelu:
            return self.linear_fc2(F.gelu(self.linear_fc1(x), approximate="tanh"))
        if self.gated:
            return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))
        h = self.fc1(x)
        return self.fc2(h * torch.sigmoid(1.702 * h))     # QuickGELU


class _VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device):
        super().__init__()
        rms = cfg.arch == "qwen2_5_vl"
        self.norm1 = _Norm(cfg.embed_dim, rms, dtype, device)
        self.norm2 = _Norm(cfg.embed_dim, rms, dtype, device)
        self.attn = _VisionAttention(cfg, dtype, device)
        self.mlp = _VisionMLP(cfg, dtype, device)

    def forward(self, x, cos, sin, bounds):
        x = x + self.attn(self.norm1(x), cos, sin, bounds)
        return x + self.mlp(self.norm2(x))


class _Merger(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device):
        super().__init__()
        self.unit = cfg.embed_dim * cfg.spatial_merge_size ** 2
        self.ln_q = _Norm(cfg.embed_dim, cfg.arch == "qwen2_5_vl", dtype, device)
        self.mlp = nn.ModuleList([_Lin(self.unit, self.unit, dtype, device), nn.GELU(), _Lin(self.unit, cfg.out_hidden_size, dtype, device)])

    def forward(self, x):
        x = self.ln_q(x).view(-1, self.unit)
        return self.mlp[2](self.mlp[1](self.mlp[0](x)))


class _Merger3(nn.Module):
    """Qwen3-VL merger: LayerNorm over one patch (main merger) or over the whole merge unit
    (deep-stack mergers), then a two-layer GELU MLP on the unit."""

    def __init__(self, cfg: VisionConfig, post_shuffle: bool, dtype, device):
        super().__init__()
        self.unit = cfg.embed_dim * cfg.spatial_merge_size ** 2
        self.post_shuffle = post_shuffle
        self.norm = _Norm(self.unit if post_shuffle else cfg.embed_dim, False, dtype, device)
        self.linear_fc1 = _Lin(self.unit, self.unit, dtype, device)
        self.linear_fc2 = _Lin(self.unit, cfg.out_hidden_size, dtype, device)

    def forward(self, x):
        x = self.norm(x.view(-1, self.unit) if self.post_shuffle else x).view(-1, self.unit)
        return self.linear_fc2(F.gelu(self.linear_fc1(x)))


class VisionTower(nn.Module):
    """``forward(pixel_values [N, patch_dim], grid_thw [n, 3]) -> [N / m^2, out_hidden_size]``."""

    def __init__(self, cfg: VisionConfig, dtype=torch.bfloat16, device="cpu", init_std: float = 0.02, seed: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = _PatchEmbed(cfg, dtype, device)
        self.blocks = nn.ModuleList([_VisionBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        if cfg.arch == "qwen3_vl":
            self.pos_embed = nn.Module()
            self.pos_embed.weight = nn.Parameter(torch.empty(cfg.num_position_embeddings, cfg.embed_dim, dtype=dtype, device=device))
            self.merger = _Merger3(cfg, False, dtype, device)
            self.deepstack_merger_list = nn.ModuleList([_Merger3(cfg, True, dtype, device) for _ in cfg.deepstack_visual_indexes])
        else:
            self.merger = _Merger(cfg, dtype, device)
        gen = None
        if seed is not None:
            gen = torch.Generator(device=device)
            gen.manual_seed(seed + 1)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if n.endswith("bias"):
                    p.zero_()
                elif ("norm" in n or "ln_q" in n) and n.endswith("weight"):
                    p.fill_(1.0)
                else:
                    p.copy_((torch.randn(p.shape, device=p.device, dtype=torch.float32, generator=gen) * init_std).to(p.dtype))

    # ---- index helpers (host side, small)
    def _rot_pos(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """(row, column) of every patch in merge-block order, ``[N, 2]``."""
        m = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            wp = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            out.append(torch.stack([hp, wp], -1).repeat(t, 1))
        return torch.cat(out, 0)

    def _window_index(self, grid_thw: torch.Tensor) -> tuple[torch.Tensor, list[int]]:
        """Order of the merged tokens that makes every attention window contiguous, and the
        window boundaries in patch units."""
        m, P = self.cfg.spatial_merge_size, self.cfg.patch_size
        win = self.cfg.window_size // m // P          # window edge in merged tokens
        order, bounds, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            lh, lw = h // m, w // m
            idx = torch.arange(t * lh * lw).view(t, lh, lw)
            ph, pw = (-lh) % win, (-lw) % win
            idx = F.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (lh + ph) // win, (lw + pw) // win
            idx = idx.view(t, nh, win, nw, win).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, win * win)
            for row in idx:
                keep = row[row >= 0]
                if keep.numel():
                    order.append(keep + base)
                    bounds.append(bounds[-1] + int(keep.numel()) * m * m)
            base += t * lh * lw
        return torch.cat(order), bounds

    def _interpolated_pos_embed(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """Rows of the learned ``side x side`` position table resampled bilinearly to every image's
        ``h x w`` patch grid (corners aligned), repeated per frame, in merge-block order: ``[N, E]``."""
        cfg, m = self.cfg, self.cfg.spatial_merge_size
        table = self.pos_embed.weight
        side = int(cfg.num_position_embeddings ** 0.5)
        out = []
        for t, h, w in grid_thw.tolist():
            hi, wi = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            h0, w0 = hi.int(), wi.int()
            h1, w1 = (h0 + 1).clip(max=side - 1), (w0 + 1).clip(max=side - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            acc = 0
            for hh, ww, wt in ((h0, w0, (1 - dh) * (1 - dw)), (h0, w1, (1 - dh) * dw), (h1, w0, dh * (1 - dw)), (h1, w1, dh * dw)):
                idx = (hh[:, None] * side + ww[None, :]).reshape(-1).long().to(table.device)
                acc = acc + table[idx] * wt.reshape(-1, 1).to(device=table.device, dtype=table.dtype)
            pe = acc.repeat(t, 1).view(t, h // m, m, w // m, m, -1).permute(0, 1, 3, 2, 4, 5).reshape(t * h * w, -1)
            out.append(pe)
        return torch.cat(out, 0)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor, return_deepstack: bool = False):
        cfg = self.cfg
        dev = self.patch_embed.proj.weight.device
        grid_thw = grid_thw.cpu().long()
        x = self.patch_embed(pixel_values.to(dev))
        if cfg.arch == "qwen3_vl":
            x = x + self._interpolated_pos_embed(grid_thw)
        N, m2 = x.shape[0], cfg.spatial_merge_size ** 2
        rp = self._rot_pos(grid_thw)
        quarter = cfg.head_dim // 4
        inv = 1.0 / (10000.0 ** (torch.arange(0, quarter, dtype=torch.float32) * 2 / (cfg.head_dim // 2)))
        ang = torch.cat([rp[:, 0:1].float() * inv, rp[:, 1:2].float() * inv], -1)            # [N, head_dim / 2]
        ang = torch.cat([ang, ang], -1).to(dev)
        cos, sin = ang.cos(), ang.sin()
        frame_bounds = [0]
        for t, h, w in grid_thw.tolist():
            for _ in range(t):
                frame_bounds.append(frame_bounds[-1] + h * w)
        windowed = cfg.window_size > 0
        if windowed:
            widx, win_bounds = self._window_index(grid_thw)
            widx = widx.to(dev)
            x = x.view(N // m2, m2, -1)[widx].reshape(N, -1)
            cos = cos.view(N // m2, m2, -1)[widx].reshape(N, -1)
            sin = sin.view(N // m2, m2, -1)[widx].reshape(N, -1)
        taps = []
        for i, blk in enumerate(self.blocks):
            bounds = win_bounds if (windowed and i not in cfg.fullatt_block_indexes) else frame_bounds
            x = blk(x, cos, sin, bounds)
            if i in cfg.deepstack_visual_indexes:
                taps.append(self.deepstack_merger_list[cfg.deepstack_visual_indexes.index(i)](x))
        y = self.merger(x)
        if windowed:
            y = y[torch.argsort(widx)]
        return (y, taps) if return_deepstack else y


def vision_param_names(cfg: VisionConfig) -> list[str]:
    """Parameter names of the tower (identical to the HF checkpoint names after ``visual.``)."""
    names = ["patch_embed.proj.weight"]
    rms = cfg.arch == "qwen2_5_vl"
    v3 = cfg.arch == "qwen3_vl"
    if v3:
        names += ["patch_embed.proj.bias", "pos_embed.weight"]
    for i in range(cfg.depth):
        b = f"blocks.{i}."
        names += [b + "norm1.weight", b + "norm2.weight"] + ([] if rms else [b + "norm1.bias", b + "norm2.bias"])
        names += [b + "attn.qkv.weight", b + "attn.qkv.bias", b + "attn.proj.weight", b + "attn.proj.bias"]
        mlp = ["linear_fc1", "linear_fc2"] if v3 else (["gate_proj", "up_proj", "down_proj"] if rms else ["fc1", "fc2"])
        for n in mlp:
            names += [b + f"mlp.{n}.weight", b + f"mlp.{n}.bias"]
    if v3:
        for pre in ["merger."] + [f"deepstack_merger_list.{j}." for j in range(len(cfg.deepstack_visual_indexes))]:
            names += [pre + n for n in ("norm.weight", "norm.bias", "linear_fc1.weight", "linear_fc1.bias", "linear_fc2.weight", "linear_fc2.bias")]
        return names
    names += ["merger.ln_q.weight"] + ([] if rms else ["merger.ln_q.bias"])
    names += ["merger.mlp.0.weight", "merger.mlp.0.bias", "merger.mlp.2.weight", "merger.mlp.2.bias"]
    return names
