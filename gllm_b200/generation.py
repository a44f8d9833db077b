"""Generation-side API objects: builder, response, token stream, hooks.

Reference parity: ``GenerationBuilder`` defaults ``max_tokens=256, temperature=0.7, top_k=0, top_p=1.0``
(src/generation.rs:447-461), ``GenerationOutput/Stream/Response`` (:428-695), hooks ``GenerationHook /
HookDecision`` Continue / Veto / Terminate (:16-65), ``thinking_budget``, ``split_thinking_content`` (:857).
The reference "streams" by generating everything first and re-yielding (:219-289); here ``stream()`` yields
tokens as the engine samples them.
"""
from __future__ import annotations

import enum
import queue
import threading
from dataclasses import dataclass, field
from typing import Callable, Iterator, List, Optional


class HookDecision(str, enum.Enum):
    CONTINUE = "continue"
    VETO = "veto"            # drop this token and finish the request
    TERMINATE = "terminate"  # keep this token and finish the request


class GenerationHook:
    """Called after every sampled token: ``post_step(token_id, generated_so_far) -> HookDecision``."""

    def post_step(self, token_id: int, n_generated: int) -> HookDecision:
        return HookDecision.CONTINUE


class StopStringHook(GenerationHook):
    """Ends a request once its decoded text contains one of ``strings`` (``GenerationBuilder.stop``): the token that
    completed the stop string is kept by the engine, the response text is cut before the string with ``cut``."""

    def __init__(self, decode: Callable[[List[int]], str], strings):
        self.decode, self.strings = decode, [s for s in strings if s]
        self.tokens: List[int] = []
        self.hit = False

    def _first(self, text: str) -> int:
        return min((i for i in (text.find(s) for s in self.strings) if i >= 0), default=-1)

    def post_step(self, token_id: int, n_generated: int) -> HookDecision:
        self.tokens.append(int(token_id))
        if self._first(self.decode(self.tokens)) >= 0:
            self.hit = True
            return HookDecision.TERMINATE
        return HookDecision.CONTINUE

    def cut(self, text: str) -> str:
        at = self._first(text)
        return text if at < 0 else text[:at]


@dataclass
class GenerationResponse:
    text: str
    token_ids: List[int]
    finish_reason: str = "length"
    thinking: str = ""
    prompt_tokens: int = 0
    cached_prefix_tokens: int = 0
    ttft_ms: float = 0.0
    tpot_ms: float = 0.0
    mtp_stats: Optional[dict] = None

    def __str__(self):
        return self.text


def split_thinking_content(text: str, open_tag: str = "<think>", close_tag: str = "</think>"):
    """-> (thinking, answer). Handles a missing opening tag (the template may have consumed it)."""
    if close_tag in text:
        head, tail = text.split(close_tag, 1)
        return head.replace(open_tag, "").strip(), tail.lstrip()
    if open_tag in text:
        return text.split(open_tag, 1)[1].strip(), ""
    return "", text


class GenerationStream:
    """Iterator over decoded text pieces while generation runs on a worker thread."""

    def __init__(self):
        self._q: "queue.Queue" = queue.Queue()
        self.response: Optional[GenerationResponse] = None
        self.error: Optional[BaseException] = None

    def _push(self, piece):
        self._q.put(piece)

    def _finish(self, response=None, error=None):
        self.response, self.error = response, error
        self._q.put(None)

    def __iter__(self) -> Iterator[str]:
        while True:
            item = self._q.get()
            if item is None:
                if self.error is not None:
                    raise self.error
                return
            yield item


class GenerationBuilder:
    def __init__(self, client, prompt):
        self._client, self._prompt = client, prompt
        self._max_tokens, self._temperature, self._top_k, self._top_p = 256, 0.7, 0, 1.0
        self._session_id: Optional[str] = None
        self._stream = False
        self._hooks: List[GenerationHook] = []
        self._thinking_budget: Optional[int] = None
        self._reasoning = False
        self._images: list = []
        self._audio: list = []
        self._stop: List[int] = []
        self._stop_strings: List[str] = []
        self._callbacks = None

    def callbacks(self, chain):
        """Run an ``engine.callbacks.CallbackChain`` on the residual stream while this request is generated (RAG or
        knowledge injection, probes that veto, early exit). The call then runs alone and eagerly."""
        self._callbacks = chain
        return self

    def max_tokens(self, n: int):
        self._max_tokens = int(n)
        return self

    def temperature(self, t: float):
        self._temperature = float(t)
        return self

    def top_k(self, k: int):
        self._top_k = int(k)
        return self

    def top_p(self, p: float):
        self._top_p = float(p)
        return self

    def session_id(self, sid: str):
        self._session_id = sid
        return self

    def stream(self, on: bool = True):
        self._stream = on
        return self

    def hook(self, h: GenerationHook):
        self._hooks.append(h)
        return self

    def thinking_budget(self, n: int):
        self._thinking_budget = int(n)
        return self

    def reasoning(self, on: bool = True):
        self._reasoning = on
        return self

    def image(self, img):
        self._images.append(img)
        return self

    def audio(self, wav):
        self._audio.append(wav)
        return self

    def stop_token_ids(self, ids):
        self._stop = [int(i) for i in ids]
        return self

    def stop(self, strings):
        """Stop strings: generation ends when the text contains one; the response holds the text before it
        (``finish_reason = "stop"``)."""
        self._stop_strings = [strings] if isinstance(strings, str) else [str(s) for s in strings]
        return self

    # ------------------------------------------------------------------------------------------
    def generate(self):
        if self._stream:
            return self._client._execute_generation_stream(self)
        return self._client._execute_generation(self)
