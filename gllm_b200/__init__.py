"""gllm_b200: a Blackwell (sm_100a) native LLM inference engine with the capabilities of gllm.

Layers (top to bottom): ``client`` (Client / builders) -> ``engine`` (executor, CUDA-graph step runner)
-> ``scheduler`` (C++ paged scheduler, prefix index, continuous batcher) / ``models`` / ``loader``
-> ``ops`` (hand-written sm_100a kernels behind a C ABI) / ``parallel`` (TP/PP/EP/CP over NVLink).
"""
__version__ = "0.1.0"

_LAZY = {
    "Client": "client", "ClientBuilder": "client", "AsyncClient": "client", "GllmError": "client",
    "GenerateRequest": "engine.batch", "ModelKind": "models.registry",
    "LLMEngine": "engine.executor", "EngineConfig": "engine.executor", "ServingLoop": "engine.serving",
    "ReplicaRouter": "engine.serving", "DecoderModel": "models.decoder", "ModelConfig": "models.config",
}


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(name)
    import importlib
    return getattr(importlib.import_module(f"{__name__}.{mod}"), name)
