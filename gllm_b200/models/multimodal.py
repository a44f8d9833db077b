"""Routing of image / audio virtual tokens: placeholder token ids in the prompt are replaced by encoder outputs
before the first decoder layer.

Reference parity: token routing of image / audio virtual tokens (src/compat/multimodal.rs),
``generate_with_multimodal`` (src/engine/executor_api.rs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


@dataclass
class MultimodalSpec:
    image_token_id: int = -1
    audio_token_id: int = -1


def expand_placeholders(token_ids: Sequence[int], spec: MultimodalSpec, n_image_tokens: Sequence[int] = (),
                        n_audio_tokens: Sequence[int] = ()) -> Tuple[List[int], List[Tuple[str, int, int, int]]]:
    """Each single placeholder becomes a run of the right length. Returns (ids, spans) with spans
    (kind, item index, start, length)."""
    out, spans, ii, ai = [], [], 0, 0
    for t in token_ids:
        if t == spec.image_token_id and ii < len(n_image_tokens):
            spans.append(("image", ii, len(out), n_image_tokens[ii]))
            out.extend([t] * n_image_tokens[ii])
            ii += 1
        elif t == spec.audio_token_id and ai < len(n_audio_tokens):
            spans.append(("audio", ai, len(out), n_audio_tokens[ai]))
            out.extend([t] * n_audio_tokens[ai])
            ai += 1
        else:
            out.append(int(t))
    if ii != len(n_image_tokens) or ai != len(n_audio_tokens):
        raise ValueError("fewer placeholders in the prompt than media items")
    return out, spans


def splice_embeddings(text_embeds: torch.Tensor, spans, image_feats: Sequence[torch.Tensor] = (),
                      audio_feats: Sequence[torch.Tensor] = ()) -> torch.Tensor:
    """text_embeds [T, H] (placeholders embedded as ordinary tokens) -> rows of each span overwritten."""
    x = text_embeds.clone()
    for kind, idx, start, n in spans:
        f = (image_feats if kind == "image" else audio_feats)[idx]
        if f.shape[0] != n or f.shape[1] != x.shape[1]:
            raise ValueError(f"{kind} {idx}: features {tuple(f.shape)} do not fit span of {n} x {x.shape[1]}")
        x[start:start + n] = f.to(x.dtype)
    return x


class MultimodalEncoder:
    """What ``Client.set_multimodal_encoder`` takes: turns raw media into feature rows of the LLM's width."""

    def __init__(self, vision=None, audio=None, spec: MultimodalSpec = MultimodalSpec()):
        self.vision, self.audio, self.spec = vision, audio, spec

    @classmethod
    def from_checkpoint(cls, keys, get, hf_config: dict, llm_hidden: int, device="cpu", dtype=torch.float32):
        """Build the image side from a multimodal checkpoint: ``keys`` are its tensor names, ``get(name)`` reads one,
        ``hf_config`` is the parsed config.json (its ``vision_config`` sizes the tower, ``image_token_index`` /
        ``image_token_id`` is the placeholder, ``mm_tokens_per_image`` gives the pooling factor). Returns None when the
        checkpoint has no SigLIP / CLIP style tower. Reference: vision branch of the model graph
        (src/arch/auto_graph_fragments/build_graph.inc.rs), tower weights by name (src/loader/name_map.rs)."""
        from .vision import VisionConfig, VisionTower, VisionWeights, siglip_tensors
        keys = set(keys)
        mark = "embeddings.patch_embedding.weight"
        hit = next((k for k in keys if k.endswith("vision_model." + mark)), None)
        vc = hf_config.get("vision_config") or {}
        if hit is None or not vc:
            return None
        prefix = hit[:-len(mark)]
        outer = prefix[:-len("vision_model.")]                      # "", "vision_tower.", "model.vision_tower." ...
        outer = outer[:-len("vision_tower.")] if outer.endswith("vision_tower.") else outer
        cfg = VisionConfig(image_size=int(vc.get("image_size", 224)), patch_size=int(vc.get("patch_size", 14)),
                           channels=int(vc.get("num_channels", 3)), hidden=int(vc["hidden_size"]),
                           layers=int(vc["num_hidden_layers"]), heads=int(vc["num_attention_heads"]),
                           mlp=int(vc["intermediate_size"]), eps=float(vc.get("layer_norm_eps", 1e-6)),
                           out_hidden=llm_hidden)
        per_image = int(hf_config.get("mm_tokens_per_image", 0) or 0)
        if per_image:
            side = int(round(per_image ** 0.5))
            cfg.pool = max(1, cfg.grid // max(side, 1))

        def find(name):        # the projector sits beside the tower, under the same outer prefix or at the top level
            return next((c for c in (outer + name, "model." + name, name) if c in keys), None)
        has = lambda n: (n in keys) or (n.startswith("multi_modal_projector.") and find(n) is not None)
        rd = lambda n: get(n if n in keys else find(n))
        t = siglip_tensors(cfg, rd, has, prefix=prefix)
        if "proj.weight" not in t:
            cfg.out_hidden = 0
        tok = hf_config.get("image_token_index", hf_config.get("image_token_id", -1))
        return cls(vision=VisionTower(cfg, VisionWeights(cfg, device=device, dtype=dtype, tensors=t)),
                   spec=MultimodalSpec(image_token_id=int(tok)))

    def encode_images(self, images: torch.Tensor) -> List[torch.Tensor]:
        return list(self.vision.forward(images)) if self.vision is not None and images is not None else []

    def encode_audio(self, waves: torch.Tensor) -> List[torch.Tensor]:
        return list(self.audio.forward(waves)) if self.audio is not None and waves is not None else []

    def prepare(self, token_ids, embed_table: torch.Tensor, images=None, waves=None):
        """-> (expanded ids, input embeddings [T, H]) ready for the decoder's ``hidden_in``."""
        imgs, auds = self.encode_images(images), self.encode_audio(waves)
        ids, spans = expand_placeholders(token_ids, self.spec, [f.shape[0] for f in imgs], [f.shape[0] for f in auds])
        emb = embed_table[torch.tensor(ids, dtype=torch.long, device=embed_table.device)]
        return ids, splice_embeddings(emb, spans, imgs, auds)
