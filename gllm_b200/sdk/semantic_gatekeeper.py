"""Semantic gatekeeper: watches a mid-layer query signal during generation; when it matches a pre-computed
knowledge key strongly enough, the matching knowledge is injected (as a residual vector or as retrieved text).

Reference parity: src/semantic_gatekeeper/* — ``SemanticLevel`` L1-L3 keys pre-computed at load (descriptor text
-> embed -> detect-layer projection), ``GatekeeperRingBuffer`` Q-tap (ring_buffer.rs:34), ``SgSharedMemory``
detect / knowledge vectors (sg_shared_memory.rs:22), traits ``KnowledgeProvider / AstSentinel / TokenizerLookup``
(mod.rs:141-180), ``SemanticGatekeeperConfig`` (:204), retrieve callback slot 0
(src/engine/mega_kernel_callback.rs:17-60). Detect layer = L/2.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Protocol, Sequence

import torch


class SemanticLevel(enum.IntEnum):
    L1_TOPIC = 1      # coarse domain
    L2_ENTITY = 2     # specific entity / API
    L3_FACT = 3       # exact fact


class KnowledgeProvider(Protocol):
    def retrieve(self, key_id: int, query: torch.Tensor) -> str: ...


class AstSentinel(Protocol):
    def in_code_context(self, text: str) -> bool: ...


@dataclass
class SemanticGatekeeperConfig:
    detect_layer: Optional[int] = None
    thresholds: Dict[SemanticLevel, float] = field(default_factory=lambda: {SemanticLevel.L1_TOPIC: 0.55,
                                                                            SemanticLevel.L2_ENTITY: 0.7,
                                                                            SemanticLevel.L3_FACT: 0.8})
    ring_capacity: int = 32
    cooldown_tokens: int = 16
    inject_scale: float = 1.0


class GatekeeperRingBuffer:
    """Last N query taps (one vector per generated token)."""

    def __init__(self, capacity: int):
        self.buf: Deque[torch.Tensor] = deque(maxlen=capacity)

    def push(self, q: torch.Tensor):
        self.buf.append(q.detach().float().cpu())

    def mean(self, last: int = 4) -> Optional[torch.Tensor]:
        if not self.buf:
            return None
        return torch.stack(list(self.buf)[-last:]).mean(0)


@dataclass
class KnowledgeKey:
    key_id: int
    level: SemanticLevel
    descriptor: str
    vector: torch.Tensor


class SgSharedMemory:
    """Detect vectors (keys) and knowledge vectors side by side, as one matrix each, for a single GEMV probe."""

    def __init__(self):
        self.keys: List[KnowledgeKey] = []
        self.detect: Optional[torch.Tensor] = None
        self.knowledge: Dict[int, torch.Tensor] = {}

    def add(self, key: KnowledgeKey, knowledge_vec: Optional[torch.Tensor] = None):
        self.keys.append(key)
        v = torch.nn.functional.normalize(key.vector.float(), dim=-1)
        self.detect = v[None] if self.detect is None else torch.cat([self.detect, v[None]])
        if knowledge_vec is not None:
            self.knowledge[key.key_id] = knowledge_vec.float()

    def match(self, q: torch.Tensor):
        if self.detect is None:
            return None, 0.0
        sims = self.detect @ torch.nn.functional.normalize(q.float(), dim=-1)
        i = int(sims.argmax())
        return self.keys[i], float(sims[i])


class SemanticGatekeeper:
    def __init__(self, client, cfg: SemanticGatekeeperConfig = SemanticGatekeeperConfig(),
                 provider: Optional[KnowledgeProvider] = None, sentinel: Optional[AstSentinel] = None):
        self.client, self.cfg, self.provider, self.sentinel = client, cfg, provider, sentinel
        n = client._st().model.cfg.num_layers
        self.layer = cfg.detect_layer if cfg.detect_layer is not None else n // 2
        self.mem = SgSharedMemory()
        self.ring = GatekeeperRingBuffer(cfg.ring_capacity)
        self._cool = 0
        self.fired: List[tuple] = []

    def register(self, descriptor: str, level: SemanticLevel, knowledge_text: Optional[str] = None) -> int:
        """Pre-compute the key: descriptor text -> hidden state at the detect layer."""
        kid = len(self.mem.keys)
        vec = self.client.encode_to_layer([descriptor], self.layer, "mean")[0]
        kvec = self.client.encode_to_layer([knowledge_text], self.layer, "mean")[0] if knowledge_text else None
        self.mem.add(KnowledgeKey(kid, level, descriptor, vec), kvec)
        return kid

    def tap(self, text_so_far: str):
        """Feed the current context; returns (key, similarity, payload) when a key fires."""
        q = self.client.encode_to_layer([text_so_far], self.layer, "mean")[0]
        self.ring.push(q)
        if self._cool > 0:
            self._cool -= 1
            return None
        if self.sentinel is not None and self.sentinel.in_code_context(text_so_far):
            return None
        key, sim = self.mem.match(self.ring.mean())
        if key is None or sim < self.cfg.thresholds[key.level]:
            return None
        self._cool = self.cfg.cooldown_tokens
        payload = self.provider.retrieve(key.key_id, q) if self.provider else self.mem.knowledge.get(key.key_id)
        self.fired.append((key.key_id, sim))
        return key, sim, payload

    def as_callback(self, device=None, dtype=torch.float32) -> "SgDetectInjectCallback":
        """The detect / inject pair as one layer callback on the model's device: the detect matrix and the knowledge
        vectors move there once; per forward it costs one GEMV and, when a key fires, one row update."""
        return SgDetectInjectCallback(self.layer, self.mem, self.cfg, device=device, dtype=dtype)

    def injection_vector(self, key_id: int) -> Optional[torch.Tensor]:
        v = self.mem.knowledge.get(key_id)
        return None if v is None else self.cfg.inject_scale * v


from ..engine.callbacks import CallbackAction, CallbackResult, LayerCallback  # noqa: E402


class SgDetectInjectCallback(LayerCallback):
    """SgDetect + SgInject on the residual stream (the reference runs them as ops inside its layer loop: detect at
    layer L / 2 against the pre-computed keys, injection of the matching knowledge vector into the same stream,
    src/semantic_gatekeeper/mod.rs, src/engine/mega_kernel_callback.rs:119-201). Here: after the detect layer the last
    row's hidden state is compared (cosine) with every key in one matrix-vector product on the device; when the best
    key passes its level's threshold and the cool-down has run out, its knowledge vector (scaled) is added to that row."""
    priority = 4

    def __init__(self, layer: int, mem: SgSharedMemory, cfg: SemanticGatekeeperConfig, device=None, dtype=torch.float32):
        self.layers = [layer]
        self.cfg = cfg
        self.keys = list(mem.keys)
        dev = device or "cpu"
        self.detect = (mem.detect if mem.detect is not None else torch.zeros(0, 1)).to(dev, dtype)
        self.thresholds = torch.tensor([cfg.thresholds[k.level] for k in self.keys], dtype=torch.float32, device=dev)
        width = self.detect.shape[1] if self.detect.numel() else 1
        self.knowledge = torch.zeros((len(self.keys), width), dtype=dtype, device=dev)
        self.has_knowledge = torch.zeros(len(self.keys), dtype=torch.bool, device=dev)
        for i, k in enumerate(self.keys):
            v = mem.knowledge.get(k.key_id)
            if v is not None:
                self.knowledge[i] = v.to(dev, dtype)
                self.has_knowledge[i] = True
        self._cool = 0
        self.fired: List[tuple] = []

    def post_layer(self, layer, hidden):
        if not self.keys:
            return CallbackResult()
        if self._cool > 0:
            self._cool -= 1
            return CallbackResult()
        q = torch.nn.functional.normalize(hidden[-1].to(self.detect.dtype), dim=-1)
        sims = self.detect @ q                                   # [keys]
        margin = sims.float() - self.thresholds
        i = int(torch.argmax(margin))
        if float(margin[i]) < 0:
            return CallbackResult(info={"sg_best": float(sims[i])})
        self._cool = self.cfg.cooldown_tokens
        key = self.keys[i]
        self.fired.append((key.key_id, float(sims[i])))
        info = {"sg_fired": key.key_id, "sg_similarity": float(sims[i])}
        if not bool(self.has_knowledge[i]):
            return CallbackResult(info=info)
        h = hidden.clone()
        h[-1] = (h[-1].float() + self.cfg.inject_scale * self.knowledge[i].float()).to(h.dtype)
        return CallbackResult(CallbackAction.REPLACE, h, info)
