"""Verification of drafted tokens and the KV commit / rollback instructions that follow.

Invariants (EqSpec): greedy verification yields exactly the tokens plain greedy decoding would; stochastic
verification (rejection sampling with residual resampling) leaves the output distribution equal to the target's.

Reference parity: src/speculative/verify.rs:14-285 (``KvCommitInstruction``,
``generate_kv_commit_instructions``); MTP verify (src/engine/mtp_executor.rs:15-425).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .tree import SpecTree


def verify_greedy(draft: Sequence[int], target_argmax: Sequence[int]) -> Tuple[int, int]:
    """``target_argmax[i]`` is the target's choice AFTER consuming draft[:i] (so it has len(draft)+1 entries).
    Returns (accepted count, next token) where next token is the correction or the bonus token."""
    n = 0
    while n < len(draft) and int(draft[n]) == int(target_argmax[n]):
        n += 1
    return n, int(target_argmax[n])


def verify_stochastic(draft: Sequence[int], q_probs: torch.Tensor, p_probs: torch.Tensor,
                      generator: Optional[torch.Generator] = None) -> Tuple[int, int]:
    """q_probs [n, V] draft distributions, p_probs [n+1, V] target distributions. Accept token i with probability
    min(1, p/q); on rejection sample from normalise(max(p - q, 0))."""
    n = len(draft)
    for i in range(n):
        t = int(draft[i])
        p, q = float(p_probs[i, t]), float(q_probs[i, t])
        u = float(torch.rand((), generator=generator))
        if q <= 0 or u >= min(1.0, p / q):
            resid = (p_probs[i] - q_probs[i]).clamp_min(0)
            s = resid.sum()
            dist = resid / s if s > 0 else p_probs[i]
            return i, int(torch.multinomial(dist, 1, generator=generator))
    return n, int(torch.multinomial(p_probs[n], 1, generator=generator))


def verify_tree_greedy(tree: SpecTree, target_argmax_at_node: Sequence[int], root_argmax: int) -> Tuple[List[int], int]:
    """Walk the tree from the root following the target's greedy choices. ``root_argmax`` is the target's token
    after the committed context; ``target_argmax_at_node[i]`` its token after node i. Returns (accepted node ids,
    next token)."""
    accepted, want, parent = [], int(root_argmax), -1
    while True:
        nxt = next((i for i, n in enumerate(tree.nodes) if n.parent == parent and n.token == want), None)
        if nxt is None:
            return accepted, want
        accepted.append(nxt)
        parent, want = nxt, int(target_argmax_at_node[nxt])


class KvOp(enum.Enum):
    KEEP = 0
    MOVE = 1
    DROP = 2


@dataclass
class KvCommitInstruction:
    op: KvOp
    src_slot: int
    dst_slot: int = -1


def generate_kv_commit_instructions(base_len: int, node_slots: Sequence[int], accepted_nodes: Sequence[int]) -> List[KvCommitInstruction]:
    """Draft node i wrote its KV at ``node_slots[i]`` (token index past ``base_len``). After verification the
    accepted nodes must occupy base_len, base_len+1, ... in order; everything else is dropped."""
    out = []
    acc = list(accepted_nodes)
    for rank, node in enumerate(acc):
        src, dst = node_slots[node], base_len + rank
        out.append(KvCommitInstruction(KvOp.KEEP if src == dst else KvOp.MOVE, src, dst))
    keep = set(acc)
    for i, s in enumerate(node_slots):
        if i not in keep:
            out.append(KvCommitInstruction(KvOp.DROP, s))
    return out


def check_eqspec_invariants(committed_before: Sequence[int], committed_after: Sequence[int], accepted: int, next_token: int,
                            draft: Sequence[int]) -> None:
    """Raises AssertionError when a verify step broke an invariant."""
    assert list(committed_after[:len(committed_before)]) == list(committed_before), "committed prefix changed"
    grown = list(committed_after[len(committed_before):])
    assert grown == list(draft[:accepted]) + [next_token], "commit must be accepted drafts + exactly one new token"
    assert 0 <= accepted <= len(draft)
