"""Layer callbacks: observers / editors of the residual stream at chosen layers, chained by priority.

Reference parity: ``LayerCallback`` + ``CallbackChain`` (pre/post node, priority)
(src/graph/layer_callback.rs:31-295); concrete callbacks early-exit, gate-skip, mid-layer encode, MoE dispatch,
RAG inject, residual-bus bridge (src/engine/callbacks/*); port layers: RAG injection L/2, early-exit recall
0.786 L, intent recall 0.75 L, guardrail L-2 (src/engine/executor_builder.rs:9-13,287-304); the 8-slot C-ABI
callback table (src/engine/mega_kernel_callback.rs:17-100).

``DecoderModel.forward(callbacks=chain)`` runs the chain on the residual stream before / after the layers it names
(the eager forward, never inside a captured CUDA graph); ``LLMEngine`` takes a chain in ``EngineConfig.callbacks``.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch


class CallbackAction(enum.Enum):
    CONTINUE = 0
    EXIT_EARLY = 1        # stop the layer loop, go to the head
    VETO = 2              # abort the request
    REPLACE = 3           # the callback returned a new hidden state


@dataclass
class CallbackResult:
    action: CallbackAction = CallbackAction.CONTINUE
    hidden: Optional[torch.Tensor] = None
    info: dict = field(default_factory=dict)


class LayerCallback:
    priority: int = 0
    layers: Optional[List[int]] = None      # None = every layer

    def wants(self, layer: int) -> bool:
        return self.layers is None or layer in self.layers

    def pre_layer(self, layer: int, hidden: torch.Tensor) -> CallbackResult:
        return CallbackResult()

    def post_layer(self, layer: int, hidden: torch.Tensor) -> CallbackResult:
        return CallbackResult()


class CallbackChain:
    def __init__(self, callbacks: Optional[List[LayerCallback]] = None):
        self.callbacks: List[LayerCallback] = sorted(callbacks or [], key=lambda c: -c.priority)

    def add(self, cb: LayerCallback):
        self.callbacks.append(cb)
        self.callbacks.sort(key=lambda c: -c.priority)

    def layers_of_interest(self, num_layers: int) -> List[int]:
        out = set()
        for c in self.callbacks:
            out |= set(range(num_layers)) if c.layers is None else set(c.layers)
        return sorted(out)

    def run(self, when: str, layer: int, hidden: torch.Tensor) -> CallbackResult:
        final = CallbackResult()
        for c in self.callbacks:
            if not c.wants(layer):
                continue
            r = c.pre_layer(layer, hidden) if when == "pre" else c.post_layer(layer, hidden)
            if r.action == CallbackAction.REPLACE and r.hidden is not None:
                hidden = r.hidden
                final = CallbackResult(CallbackAction.REPLACE, hidden, {**final.info, **r.info})
            elif r.action in (CallbackAction.EXIT_EARLY, CallbackAction.VETO):
                r.info = {**final.info, **r.info}
                if final.hidden is not None and r.hidden is None:
                    r.hidden = final.hidden
                return r
            else:
                final.info.update(r.info)
        return final


def port_layers(num_layers: int) -> Dict[str, int]:
    L = num_layers
    return {"rag_inject": L // 2, "early_exit": int(0.786 * L), "intent": int(0.75 * L), "guardrail": max(0, L - 2),
            "sg_detect": L // 2}


class EarlyExitCallback(LayerCallback):
    """Exit when consecutive hidden states stop changing direction (cosine) or magnitude (delta rho)."""
    priority = 10

    def __init__(self, layer: int, cos_threshold: float = 0.999, rho_threshold: float = 0.02):
        self.layers = [layer - 1, layer]
        self.cos_threshold, self.rho_threshold = cos_threshold, rho_threshold
        self.prev: Optional[torch.Tensor] = None

    def post_layer(self, layer, hidden):
        h = hidden.float()
        if layer == self.layers[0] or self.prev is None:
            self.prev = h.clone()
            return CallbackResult()
        cos = torch.nn.functional.cosine_similarity(h, self.prev, dim=-1).min().item()
        rho = ((h - self.prev).norm(dim=-1) / self.prev.norm(dim=-1).clamp_min(1e-9)).max().item()
        self.prev = None
        if cos > self.cos_threshold and rho < self.rho_threshold:
            return CallbackResult(CallbackAction.EXIT_EARLY, info={"exit_layer": layer, "cos": cos, "rho": rho})
        return CallbackResult(info={"cos": cos, "rho": rho})


class MidLayerEncodeCallback(LayerCallback):
    """Copies the hidden state of one layer out (intent / head-routing consumers)."""
    priority = 5

    def __init__(self, layer: int):
        self.layers = [layer]
        self.captured: Optional[torch.Tensor] = None

    def post_layer(self, layer, hidden):
        self.captured = hidden.detach().clone()
        return CallbackResult()


class RagInjectCallback(LayerCallback):
    """Late-fusion RAG: add a (scaled) knowledge vector to the residual stream of the last token."""
    priority = 3

    def __init__(self, layer: int, vector: torch.Tensor, scale: float = 1.0):
        self.layers, self.vector, self.scale = [layer], vector, scale

    def pre_layer(self, layer, hidden):
        h = hidden.clone()
        h[-1] = (h[-1].float() + self.scale * self.vector.to(h.device).float()).to(h.dtype)
        return CallbackResult(CallbackAction.REPLACE, h, {"rag_injected": True})


class GateSkipCallback(LayerCallback):
    """Records which layers the epilogue telemetry marked as skippable and replaces their output with the input."""
    priority = 1

    def __init__(self, skip_layers: List[int]):
        self.layers = list(skip_layers)
        self._saved: Dict[int, torch.Tensor] = {}

    def pre_layer(self, layer, hidden):
        self._saved[layer] = hidden.clone()
        return CallbackResult()

    def post_layer(self, layer, hidden):
        return CallbackResult(CallbackAction.REPLACE, self._saved.pop(layer), {"skipped": layer})


class LayerTelemetryCallback(LayerCallback):
    """Feeds the epilogue aggregator: per layer the relative change of the residual stream (delta rho = ||x_out -
    x_in|| / ||x_in||, on the device through ``ops.telemetry.layer_telemetry`` when the rows live there). The
    aggregator's advice names the layers that barely move the stream (candidates for ``GateSkipCallback``) and
    whether drafts are likely to be accepted. Reference: epilogue telemetry signals and their consumers
    (src/jit/epilogue.rs, src/engine/executor_step.rs:265-393)."""
    priority = 50
    layers = None

    def __init__(self, aggregator):
        self.agg = aggregator
        self._in: Dict[int, torch.Tensor] = {}

    def pre_layer(self, layer, hidden):
        self._in[layer] = hidden.clone()
        return CallbackResult()

    def post_layer(self, layer, hidden):
        from ...runtime.epilogue import EpilogueSignal, signals_from_tensors
        x_in = self._in.pop(layer, None)
        if x_in is None:
            return CallbackResult()
        if hidden.is_cuda:
            from ...ops.telemetry import layer_telemetry
            sig = EpilogueSignal(layer, delta_rho=float(layer_telemetry(x_in, hidden)["delta_rho"]))
        else:
            sig = signals_from_tensors(layer, x_in, hidden)
        self.agg.push(sig)
        return CallbackResult()


class ProbeVetoCallback(LayerCallback):
    """Linear probe on a mid-layer hidden state; vetoes the request when the score crosses the threshold."""
    priority = 20

    def __init__(self, layer: int, weight: torch.Tensor, bias: float = 0.0, threshold: float = 0.5):
        self.layers, self.w, self.b, self.threshold = [layer], weight, bias, threshold

    def post_layer(self, layer, hidden):
        score = torch.sigmoid(hidden[-1].float() @ self.w.to(hidden.device).float() + self.b).item()
        if score > self.threshold:
            return CallbackResult(CallbackAction.VETO, info={"probe_score": score})
        return CallbackResult(info={"probe_score": score})


# ---- C-ABI style slot table -----------------------------------------------------------------------
SLOT_SG_KNOWLEDGE_RETRIEVE, SLOT_GUARDRAIL, SLOT_KV_DECOMPRESS, SLOT_EARLY_EXIT, SLOT_MOE_DISPATCH, SLOT_RAG_INJECT, \
    SLOT_INTENT, SLOT_USER = range(8)


class CallbackTable:
    """Eight fixed slots, as the device-side ABI of the reference; a slot holds a Python callable here."""

    def __init__(self):
        self.slots: List[Optional[Callable]] = [None] * 8

    def register(self, slot: int, fn: Callable):
        if not 0 <= slot < 8:
            raise IndexError("callback slots are 0..7")
        self.slots[slot] = fn

    def call(self, slot: int, *args):
        fn = self.slots[slot]
        return None if fn is None else fn(*args)
