"""Draft trees for speculative decoding: prompt-lookup (PLD) spine, n-gram branches, and the tree attention mask.

Reference parity: ``SpecTree`` PLD spine + n-gram branches and ``tree_attention_mask_csr``
(src/speculative/tree.rs:93-340), ``NgramIndex`` (:394-452).
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


class NgramIndex:
    """Maps every n-gram (n in [min_n, max_n]) of the running token stream to the positions that follow it."""

    def __init__(self, min_n: int = 2, max_n: int = 4):
        self.min_n, self.max_n = min_n, max_n
        self.tokens: List[int] = []
        self.index: Dict[Tuple[int, ...], List[int]] = defaultdict(list)

    def extend(self, toks: Sequence[int]):
        for t in toks:
            self.tokens.append(int(t))
            end = len(self.tokens) - 1          # the n-gram ENDS at end-1; position `end` follows it
            for n in range(self.min_n, self.max_n + 1):
                if end - n >= 0:
                    self.index[tuple(self.tokens[end - n:end])].append(end)

    def lookup(self, max_len: int, top: int = 1) -> List[List[int]]:
        """Continuations (token lists up to ``max_len``) following the longest matching suffix, newest first."""
        out = []
        for n in range(self.max_n, self.min_n - 1, -1):
            if len(self.tokens) < n:
                continue
            key = tuple(self.tokens[-n:])
            for pos in reversed(self.index.get(key, [])):
                cont = self.tokens[pos:pos + max_len]
                if cont and cont not in out:
                    out.append(cont)
                    if len(out) >= top:
                        return out
            if out:
                return out
        return out


@dataclass
class TreeNode:
    token: int
    parent: int          # index into nodes, -1 for children of the root (the last accepted token)
    depth: int
    children: List[int] = field(default_factory=list)


class SpecTree:
    def __init__(self):
        self.nodes: List[TreeNode] = []

    def add_path(self, tokens: Sequence[int]) -> List[int]:
        """Insert a root-anchored path, sharing existing prefixes. Returns the node ids along the path."""
        parent, ids = -1, []
        for d, tok in enumerate(tokens):
            sibs = [i for i, n in enumerate(self.nodes) if n.parent == parent]
            hit = next((i for i in sibs if self.nodes[i].token == tok), None)
            if hit is None:
                self.nodes.append(TreeNode(int(tok), parent, d))
                hit = len(self.nodes) - 1
                if parent >= 0:
                    self.nodes[parent].children.append(hit)
            ids.append(hit)
            parent = hit
        return ids

    @staticmethod
    def build(spine: Sequence[int], branches: Sequence[Sequence[int]] = (), max_nodes: int = 64) -> "SpecTree":
        t = SpecTree()
        t.add_path(spine[:max_nodes])
        for b in branches:
            if len(t.nodes) + len(b) > max_nodes:
                break
            t.add_path(b)
        return t

    def tokens(self) -> List[int]:
        return [n.token for n in self.nodes]

    def depths(self) -> List[int]:
        return [n.depth for n in self.nodes]

    def ancestors(self, i: int) -> List[int]:
        out = []
        while i >= 0:
            out.append(i)
            i = self.nodes[i].parent
        return out[::-1]

    def paths(self) -> List[List[int]]:
        leaves = [i for i, n in enumerate(self.nodes) if not n.children]
        return [self.ancestors(i) for i in leaves]


def tree_attention_mask_csr(tree: SpecTree) -> Tuple[List[int], List[int]]:
    """CSR (row_ptr, col_idx): node i attends to itself and its ancestors (plus, implicitly, the whole committed
    context)."""
    row_ptr, cols = [0], []
    for i in range(len(tree.nodes)):
        cols.extend(tree.ancestors(i))
        row_ptr.append(len(cols))
    return row_ptr, cols


def tree_attention_mask_dense(tree: SpecTree):
    import torch
    n = len(tree.nodes)
    m = torch.zeros(n, n, dtype=torch.bool)
    rp, ci = tree_attention_mask_csr(tree)
    for i in range(n):
        m[i, ci[rp[i]:rp[i + 1]]] = True
    return m
