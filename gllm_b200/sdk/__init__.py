"""SDKs layered on the Client: chain-of-thought, guardrail, head routing, intent, semantic gatekeeper, stream
guard, late-fusion RAG / residual bus."""
from .cot import CotConfig, CotReasoner, CotTrace  # noqa: F401
from .guardrail import Guardrail, GuardrailVerdict  # noqa: F401
from .head_routing import HeadRouter  # noqa: F401
from .intent import IntentClassifier, IntentTracker, IntentTrackerCell  # noqa: F401
from .probes import LinearProbe  # noqa: F401
from .qwen3_guard import Risk, StreamGuard  # noqa: F401
from .rag import LateFusionRag, ResidualBus  # noqa: F401
from .semantic_gatekeeper import (GatekeeperRingBuffer, SemanticGatekeeper, SemanticGatekeeperConfig, SemanticLevel,  # noqa: F401
                                  SgSharedMemory)
