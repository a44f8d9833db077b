"""Single-sequence generation outside the batcher: a private KV cache, one prefill (token ids or prepared input
embeddings), then token-by-token decode. Used for prompts that carry image / audio features and by diagnostics.

Reference parity: ``generate_with_multimodal`` and ``generate_single_sequence``
(src/engine/executor_api.rs:19-860; src/engine/mega_kernel/executor_ops.inc.rs:84-1496).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .batch import ForwardBatch

PAGE = 16


def generate_single(model, token_ids: Sequence[int], max_new_tokens: int, *, input_embeds: Optional[torch.Tensor] = None,
                    temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, eos_ids: Sequence[int] = (), seed: int = 0) -> List[int]:
    dev = model.device
    T = len(token_ids)
    if input_embeds is not None and input_embeds.shape[0] != T:
        raise ValueError("input_embeds must have one row per prompt token")
    pages = (T + max_new_tokens + PAGE - 1) // PAGE + 1
    kv = model.alloc_kv_cache(pages)
    bt = torch.arange(pages, dtype=torch.int32, device=dev)[None]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    V = model.cfg.vocab_size
    gen = torch.Generator().manual_seed(seed)

    def pick(logits_row: torch.Tensor) -> int:
        if temperature <= 0:
            return int(logits_row[:V].argmax())
        params = torch.tensor([[temperature, float(top_k), top_p, 0.0]], dtype=torch.float32, device=logits_row.device)
        out = ops.sample(logits_row[None, :V].float().contiguous(), params, vocab=V, seed=seed,
                         step_offsets=torch.zeros(1, dtype=torch.int64, device=logits_row.device), generator=gen)
        return int(out[0])

    batch = ForwardBatch(token_ids=i32(list(token_ids)), positions=torch.arange(T, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), block_tables=bt, ctx_lens=i32([T]),
                         q_start=i32([0]), q_len=i32([T]), max_q_len=T,
                         logits_rows=torch.tensor([T - 1], dtype=torch.int64, device=dev))
    hid = None if input_embeds is None else input_embeds.to(dev, model.dtype).contiguous()
    logits = model.forward(batch, kv, hidden_in=hid)
    out: List[int] = []
    tok = pick(logits[0])
    pos = T
    while True:
        out.append(tok)
        if tok in eos_ids or len(out) >= max_new_tokens:
            break
        b = ForwardBatch(token_ids=i32([tok]), positions=i32([pos]), slot_mapping=i32([pos]), block_tables=bt,
                         ctx_lens=i32([pos + 1]), is_decode=True)
        tok = pick(model.forward(b, kv)[0])
        pos += 1
    return out
