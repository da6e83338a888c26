"""Vision-language causal LM: the decoder of ``decoder.py`` plus the image tower of
``vision.py``. Image features replace the embeddings of the image placeholder tokens and the
rotary tables are built per token from the three M-RoPE position streams.

Reference behaviour: ``areal/engine/fsdp_engine.py:1997-2056`` (multi-modal inputs gathered per
micro-batch, position ids from the model's ``get_rope_index``) and
``areal/models/transformers/qwen2_vl.py``.
"""
from __future__ import annotations

import copy
from typing import Any, Optional

import torch

from ..ops import functional as OF
from .config import ModelConfig
from .decoder import CausalLM, PackedBatch
from .vision import VisionTower, mrope_position_ids, mrope_tables, num_image_tokens


def collect_multi_modal(mm_list: Optional[list]) -> Optional[dict[str, Any]]:
    """Per-sequence ``multi_modal_input`` entries (dicts with ``pixel_values`` / ``image_grid_thw``,
    or ``None`` for text-only samples) -> one dict for the packed batch, images in sequence order;
    ``images_per_seq`` says how many grids each sequence owns."""
    if not mm_list:
        return None
    px, grids, per_seq = [], [], []
    for m in mm_list:
        if not m or m.get("pixel_values") is None:
            per_seq.append(0)
            continue
        g = torch.as_tensor(m["image_grid_thw"]).view(-1, 3).long()
        px.append(torch.as_tensor(m["pixel_values"]))
        grids.append(g)
        per_seq.append(g.shape[0])
    if not px:
        return None
    return {"pixel_values": torch.cat(px, 0), "image_grid_thw": torch.cat(grids, 0), "images_per_seq": per_seq}


class VisionLanguageModel(CausalLM):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", init_std: float = 0.02, seed: Optional[int] = None):
        super().__init__(cfg, dtype=dtype, device=device, init_std=init_std, seed=seed)
        self.vcfg = cfg.vision_config()
        self.visual = VisionTower(self.vcfg, dtype=dtype, device=device, init_std=init_std, seed=seed)

    def packed_mrope(self, ids_cpu: torch.Tensor, cu: list[int], grid_thw: Optional[torch.Tensor],
                     images_per_seq: Optional[list[int]] = None) -> tuple[torch.Tensor, list[int], torch.Tensor]:
        """M-RoPE streams ``[3, T]`` for a packed batch, the per-sequence deltas, and the token
        indices that hold image features. Images are consumed in order; a sequence owns
        ``images_per_seq[i]`` grids (without that list: as many as its placeholder tokens account for)."""
        cfg = self.cfg
        m = self.vcfg.spatial_merge_size
        T = ids_cpu.shape[0]
        pos = torch.zeros(3, T, dtype=torch.long)
        per_image = num_image_tokens(grid_thw, m) if grid_thw is not None else []
        img, deltas, where = 0, [], []
        for si, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
            seq = ids_cpu[a:b]
            if images_per_seq is not None:
                k = images_per_seq[si] if si < len(images_per_seq) else 0
            else:
                want = int(((seq == cfg.image_token_id) | (seq == cfg.video_token_id)).sum())
                k = 0
                while want > 0 and img + k < len(per_image):
                    want -= per_image[img + k]
                    k += 1
                if want != 0:
                    raise ValueError("image placeholder tokens do not match the image grids of this sequence")
            g = grid_thw[img:img + k] if k else None
            local: list[int] = []
            p, d = mrope_position_ids(seq, g, cfg.image_token_id, m, cfg.video_token_id, image_positions=local)
            if len(local) != sum(per_image[img:img + k]):
                raise ValueError(f"sequence {si}: {len(local)} placeholder tokens for {sum(per_image[img:img + k])} image features")
            pos[:, a:b] = p
            deltas.append(d)
            where += [a + x for x in local]
            img += k
        return pos, deltas, torch.tensor(where, dtype=torch.long)

    vision_sp = None     # (group, size, rank) set by the train engine: the pictures of a micro-batch are split over the group

    def _image_features(self, px: torch.Tensor, grid: torch.Tensor):
        """Features of all pictures ``[n_tokens, H]`` (+ deep-stack taps). Under sequence parallelism every rank of
        the group runs the tower on a contiguous share of the pictures (balanced by patch count) and the features are
        all-gathered; the backward pass sums the feature gradients of all ranks onto the rank that made them (role of
        the reference's ``vision_sp_shard.py``, which all-gathers the tower's outputs over the SP group)."""
        want_taps = bool(self.vcfg.deepstack_visual_indexes)

        def tower(p, g):
            if want_taps:
                return self.visual(p, g, return_deepstack=True)
            return self.visual(p, g), None
        sp = self.vision_sp
        n_img = int(grid.shape[0])
        if sp is None or sp[1] <= 1 or n_img < 2:
            return tower(px, grid)
        from ..parallel.cp import _AllGatherCat

        group, size, rank = sp
        patches = grid.long().prod(-1).tolist()
        merge = self.vcfg.spatial_merge_size ** 2
        # contiguous shares with about equal patch counts
        total, bounds, acc = sum(patches), [0], 0
        for i, n in enumerate(patches):
            acc += n
            while len(bounds) < size and acc >= total * len(bounds) / size:
                bounds.append(i + 1)
        bounds += [n_img] * (size + 1 - len(bounds))
        bounds[-1] = n_img
        tok = [sum(patches[bounds[r]:bounds[r + 1]]) // merge for r in range(size)]
        i0, i1 = bounds[rank], bounds[rank + 1]
        pa = sum(patches[:i0])
        H = self.embed_tokens.shape[1]
        if i1 > i0:
            f, t = tower(px[pa:pa + sum(patches[i0:i1])], grid[i0:i1])
        else:
            # no picture for this rank: an empty slice of a parameter keeps the gather below inside this rank's autograd
            # graph, so its backward (a collective) runs here as it does on the peers
            f = self.embed_tokens[:0]
            t = [self.embed_tokens[:0] for _ in self.vcfg.deepstack_visual_indexes] if want_taps else None
        Lmax = max(tok)

        def gather(x):
            pad = x.new_zeros(Lmax, x.shape[1])
            pad = torch.cat([x, pad[: Lmax - x.shape[0]]], 0) if x.shape[0] < Lmax else x
            full = _AllGatherCat.apply(pad.contiguous(), group)
            return torch.cat([full[r * Lmax: r * Lmax + tok[r]] for r in range(size)], 0)
        return gather(f), ([gather(x) for x in t] if want_taps else None)

    def embed_multimodal(self, input_ids: torch.Tensor, mm: dict[str, Any], positions: Optional[torch.Tensor] = None,
                         with_deepstack: bool = False):
        feats, taps = self._image_features(mm["pixel_values"].to(self.embed_tokens.dtype), mm["image_grid_thw"])
        h = OF.embedding(input_ids, self.embed_tokens)
        if positions is None:
            mask = (input_ids == self.cfg.image_token_id) | (input_ids == self.cfg.video_token_id)
            positions = mask.nonzero(as_tuple=True)[0]
        positions = positions.to(input_ids.device)
        if positions.numel() != feats.shape[0]:
            raise ValueError(f"{positions.numel()} placeholder tokens for {feats.shape[0]} image features")
        out = h.index_copy(0, positions, feats.to(h.dtype))
        return (out, (positions, taps) if taps else None) if with_deepstack else out

    def forward_hidden(self, input_ids: torch.Tensor, pb: PackedBatch, attn_fns=None, mm: Optional[dict[str, Any]] = None,
                       row_slice: Optional[slice] = None, **kw) -> torch.Tensor:
        """``row_slice`` (sequence parallelism): ``input_ids`` holds ALL tokens of the micro-batch, the layers run on
        rows ``row_slice`` only. Embeddings, image features and the per-token rotary tables are made for the whole
        micro-batch on every rank (the image tower is small beside the language model) and cut to the rows; ``pb`` is
        the local batch descriptor (full ``cu_seqlens``)."""
        sl = row_slice
        if mm is None or mm.get("pixel_values") is None or mm["pixel_values"].numel() == 0:
            # text only: the three streams coincide and M-RoPE is ordinary RoPE
            return super().forward_hidden(input_ids if sl is None else input_ids[sl], pb, attn_fns, **kw)
        T = input_ids.shape[0]
        pos3, where = mm.get("mrope_position_ids"), mm.get("image_positions")
        if pos3 is None:
            cu = pb.cu_seqlens.tolist()
            pos3, _, where = self.packed_mrope(input_ids.cpu().long(), cu, mm["image_grid_thw"].cpu().long(), mm.get("images_per_seq"))
        sections = self.cfg.mrope_section or [self.cfg.head_dim // 2, 0, 0]
        cos, sin = mrope_tables(pos3, self.cfg.head_dim, self.cfg.rope_theta, sections, input_ids.device, self.cfg.mrope_interleaved)
        pb2 = copy.copy(pb)
        rows = torch.arange(T, dtype=torch.int32, device=input_ids.device)   # row t of the per-token tables
        embeds, deep = self.embed_multimodal(input_ids, mm, where, with_deepstack=True)
        if sl is not None:
            rows, embeds, input_ids = rows[sl], embeds[sl], input_ids[sl]
            if deep is not None:
                idx, feats = deep
                keep = (idx >= sl.start) & (idx < sl.stop)
                deep = (idx[keep] - sl.start, [f[keep] for f in feats])
        pb2.position_ids = rows
        return super().forward_hidden(input_ids, pb2, attn_fns, inputs_embeds=embeds, rope=(cos, sin), deepstack=deep)
