"""Public client surface: ``Client`` / ``ClientBuilder`` / ``AsyncClient`` and the embed / rerank / classify
builders.

Reference parity: ``Client::{new_chat,new_embedding,new_classifier,builder}``, ``load_model / unload_model /
swap_model``, ``generate / embed / rerank / classify / generate_batch / encode / decode``
(src/client_fragments/client_impl.inc.rs:119-2010), ``ClientBuilder`` (builder.inc.rs:22-325), error enum
(error_config.inc.rs:6-25), ``AsyncClient`` thread offload (async_client.inc.rs:41-48), ``EmbeddingsBuilder``
with ``normalize / dimension`` (Matryoshka) / ``rerank_query / top_n`` (src/embeddings.rs:31-181),
``RerankBuilder`` (src/rerank.rs:27-58), classify = softmax + argmax on the host
(client_impl.inc.rs:1363-1403), pipelines embed->rerank and RAG embed->rerank->generate (:1415-1573).
"""
from __future__ import annotations

import concurrent.futures as cf
import math
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .engine.batch import GenerateRequest, GenerateResult
from .generation import (GenerationBuilder, GenerationHook, GenerationResponse, GenerationStream, HookDecision, StopStringHook,
                         split_thinking_content)
from .models.registry import ModelKind


class GllmError(Exception):
    pass


class ModelNotFoundError(GllmError):
    pass


class BackendError(GllmError):
    pass


class OutOfMemoryError(GllmError):
    pass


class InvalidModelTypeError(GllmError):
    pass


class NoModelLoadedError(GllmError):
    pass


class RuntimeGllmError(GllmError):
    pass


ClientError = GllmError


@dataclass
class ClientConfig:
    """Per-client execution settings (error_config.inc.rs:96-131)."""
    max_num_seqs: int = 64
    max_model_len: int = 4096
    max_batch_tokens: int = 4096
    enable_prefix_cache: bool = True
    use_cuda_graphs: bool = True
    compute_dtype: str = "bf16"
    intent: str = "throughput"       # latency | throughput (arbiter input)
    seed: int = 0
    kv_cache_dtype: str = "auto"     # bf16 | fp8 | auto (the KV decision matrix picks from what fits in HBM)
    kv_scale: float = 0.05           # per-tensor scale of an fp8 KV cache
    # How the dense projections are held on the device. "bf16": a quantised checkpoint (GGUF K-quants, AWQ, GPTQ, fp8
    # blocks ...) is dequantised at load and runs the fused bf16 layer. "mxfp8" / "nvfp4": the projections are
    # (re)quantised to block-scaled operands and every GEMM of the fused layer runs block-scaled on the tensor cores.
    # "auto": nvfp4 for a checkpoint quantised to 4-5 bits, mxfp8 for 6-8 bits, bf16 otherwise (on a GPU, when the model
    # has the shapes of the fused layer).
    weight_quant: str = "bf16"
    # MoE models with weight paging enabled (ClientBuilder.weight_paging_enabled): experts of every layer kept on the
    # device, the rest are paged in from pinned host memory per step. 0 = max(4 * experts per token, experts / 4).
    expert_slots: int = 0
    debug: bool = False              # ClientBuilder.debug_jit(): eager steps with per-layer NaN / Inf checks


@dataclass
class _State:
    model_id: str
    kind: ModelKind
    loaded: object
    model: object
    engine: Optional[object]
    tokenizer: object
    backend: object


class ClientBuilder:
    def __init__(self):
        self._model: Optional[str] = None
        self._kind: Optional[ModelKind] = None
        self._backend: Optional[str] = None
        self._cfg = ClientConfig()
        self._distributed = None
        self._reranker: Optional[str] = None
        self._generator: Optional[str] = None
        self._gguf_filter: Optional[str] = None
        self._debug = False
        self._weight_paging = False

    def model(self, model_id: str):
        self._model = model_id
        return self

    def kind(self, kind):
        self._kind = ModelKind(kind) if not isinstance(kind, ModelKind) else kind
        return self

    def backend(self, name: str):
        self._backend = name
        return self

    def intent(self, intent: str):
        self._cfg.intent = intent
        return self

    def distributed(self, cfg):
        self._distributed = cfg
        return self

    def compute_dtype(self, dt: str):
        self._cfg.compute_dtype = dt
        return self

    def reranker(self, model_id: str):
        self._reranker = model_id
        return self

    def generator(self, model_id: str):
        self._generator = model_id
        return self

    def gguf_file_filter(self, pattern: str):
        self._gguf_filter = pattern
        return self

    def debug_jit(self, on: bool = True):
        """Debug serving. The reference dumps its JIT's instruction stream here; this engine has no JIT, so the switch
        turns on what debugging a forward needs instead: eager steps and a non-finite check after every layer."""
        self._debug = on
        self._cfg.debug = bool(on)
        return self

    def weight_paging_enabled(self, on: bool = True):
        self._weight_paging = on
        return self

    def config(self, **kw):
        for k, v in kw.items():
            setattr(self._cfg, k, v)
        return self

    def build(self) -> "Client":
        if not self._model:
            raise GllmError("ClientBuilder: model() is required")
        c = Client(self._cfg, backend=self._backend, distributed=self._distributed, gguf_filter=self._gguf_filter,
                   weight_paging=self._weight_paging)
        c.load_model(self._model, self._kind)
        if self._reranker:
            c._aux["reranker"] = Client(self._cfg, backend=self._backend)
            c._aux["reranker"].load_model(self._reranker, ModelKind.RERANKER)
        if self._generator:
            c._aux["generator"] = Client(self._cfg, backend=self._backend)
            c._aux["generator"].load_model(self._generator, ModelKind.CHAT)
        return c


class Client:
    def __init__(self, config: Optional[ClientConfig] = None, backend: Optional[str] = None, distributed=None,
                 gguf_filter: Optional[str] = None, weight_paging: bool = False):
        self.config = config or ClientConfig()
        self._weight_paging = bool(weight_paging)
        self._backend_name, self._distributed, self._gguf_filter = backend, distributed, gguf_filter
        self._state: Optional[_State] = None
        self._lock = threading.RLock()
        self._aux: Dict[str, "Client"] = {}
        self._multimodal_encoder = None

    # ---- constructors ---------------------------------------------------------------------------
    @staticmethod
    def builder() -> ClientBuilder:
        return ClientBuilder()

    @staticmethod
    def new_chat(model_id: str, **kw) -> "Client":
        return ClientBuilder().model(model_id).kind(ModelKind.CHAT).config(**kw).build()

    @staticmethod
    def new_embedding(model_id: str, **kw) -> "Client":
        return ClientBuilder().model(model_id).kind(ModelKind.EMBEDDING).config(**kw).build()

    @staticmethod
    def new_reranker(model_id: str, **kw) -> "Client":
        return ClientBuilder().model(model_id).kind(ModelKind.RERANKER).config(**kw).build()

    @staticmethod
    def new_classifier(model_id: str, **kw) -> "Client":
        return ClientBuilder().model(model_id).kind(ModelKind.CLASSIFIER).config(**kw).build()

    @staticmethod
    def from_model(cfg, weights, tokenizer=None, kind=ModelKind.CHAT, device=None, dtype=None, distributed=None,
                   weight_paging: bool = False, **kw) -> "Client":
        """Build a client around in-memory weights (synthetic models, tests)."""
        c = Client(ClientConfig(**kw), distributed=distributed, weight_paging=weight_paging)
        c._install(model_id="<memory>", kind=kind, loaded=None, cfg=cfg, weights=weights, tokenizer=tokenizer,
                   device=device, dtype=dtype)
        return c

    # ---- model lifecycle ------------------------------------------------------------------------
    def load_model(self, model_id: str, kind: Optional[ModelKind] = None):
        from .loader import Loader, LoaderConfig, ModelNotFound
        lc = LoaderConfig.from_env()
        lc.gguf_file_filter = self._gguf_filter
        try:
            loaded = Loader.from_source_with_config(model_id, lc).load()
        except ModelNotFound as e:
            raise ModelNotFoundError(str(e)) from e
        k = kind or ModelKind(loaded.config.kind if loaded.config.kind in ModelKind._value2member_map_ else "chat")
        self._install(model_id, k, loaded, loaded.config, loaded.weights, loaded.tokenizer)
        self._attach_checkpoint_encoder(loaded)

    def _attach_checkpoint_encoder(self, loaded):
        """A multimodal SafeTensors checkpoint (a ``vision_config`` in its config.json and a SigLIP / CLIP style tower
        among its tensors) gets its image encoder without a ``set_multimodal_encoder`` call."""
        import json
        from pathlib import Path
        raw = getattr(loaded.weights, "model", None)
        root = Path(loaded.path) if Path(loaded.path).is_dir() else Path(loaded.path).parent
        cj = root / "config.json"
        if raw is None or not hasattr(raw, "keys") or not cj.exists() or not loaded.config.causal:
            return
        try:
            hf = json.loads(cj.read_text())
        except ValueError:
            return
        if not hf.get("vision_config"):
            return
        from .models.multimodal import MultimodalEncoder
        model = self._st().model
        enc = MultimodalEncoder.from_checkpoint(list(raw.keys()), raw.tensor, hf, loaded.config.hidden_size,
                                                device=model.device, dtype=model.dtype)
        if enc is not None:
            self._multimodal_encoder = enc

    def _install(self, model_id, kind, loaded, cfg, weights, tokenizer, device=None, dtype=None):
        from .backend import detect_backend
        from .engine.executor import EngineConfig, LLMEngine
        from .models.decoder import DecoderModel
        from .models.encoder import EncoderModel
        from .tokenizer import TokenizerHandle
        be = detect_backend(self._backend_name)
        dev = torch.device(device) if device is not None else be.device
        dt = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        tokenizer = tokenizer or TokenizerHandle.byte_level()
        with self._lock:
            try:
                if cfg.causal:
                    if kind in (ModelKind.EMBEDDING, ModelKind.RERANKER, ModelKind.CLASSIFIER) and cfg.num_labels == 0 \
                            and kind != ModelKind.EMBEDDING and kind != ModelKind.RERANKER:
                        raise InvalidModelTypeError(f"{model_id} has no classifier head")
                    kv_kw = self._kv_cache_plan(cfg, dev)
                    kv_kw["weight_quant"] = self._weight_quant_plan(cfg, dev)
                    tp = self._tensor_parallel_context(cfg, dev)
                    if tp is not None:
                        kv_kw["tp"] = tp
                    if self._weight_paging and cfg.is_moe and tp is None and not kv_kw.get("weight_quant"):
                        kv_kw["expert_slots"] = self.config.expert_slots or max(4 * cfg.num_experts_per_tok,
                                                                                cfg.num_experts // 4)
                    model = DecoderModel(cfg, weights, device=dev, dtype=dt,
                                         max_positions=min(cfg.max_position_embeddings, self.config.max_model_len), **kv_kw)
                    ec = EngineConfig(max_num_seqs=self.config.max_num_seqs, max_model_len=self.config.max_model_len,
                                      max_batch_tokens=self.config.max_batch_tokens,
                                      prefill_chunk=self.config.max_batch_tokens,
                                      enable_prefix_cache=self.config.enable_prefix_cache,
                                      use_cuda_graphs=self.config.use_cuda_graphs, seed=self.config.seed,
                                      debug=self.config.debug or self._env_debug())
                    if dev.type != "cuda":
                        ec.num_pages = max(64, self.config.max_num_seqs * ((ec.max_model_len + 15) // 16) // 4)
                    engine = LLMEngine(model, ec, tokenizer=tokenizer)
                else:
                    if kind == ModelKind.CHAT:
                        raise InvalidModelTypeError(f"{model_id} is an encoder and cannot generate")
                    model, engine = EncoderModel(cfg, weights, device=dev, dtype=dt), None
            except torch.cuda.OutOfMemoryError as e:  # pragma: no cover - needs a GPU
                raise OutOfMemoryError(str(e)) from e
            self._state = _State(model_id, kind, loaded, model, engine, tokenizer, be)

    def _tensor_parallel_context(self, cfg, dev):
        """``ClientBuilder.distributed(DistributedConfig)``: with ``parallel.tp`` = world size > 1 every rank of the job
        (one process per GPU, started by ``torch.distributed.run``) builds its shard of the model over a
        ``TPContext`` and makes the same client calls with the same arguments; every rank returns the same result.
        Pipeline stages, expert parallelism and context-parallel prefill are reached through the engine-level APIs
        (``engine.pp``, ``EPContext``, ``CpPrefill``). Reference: DistributedConfig on the client builder
        (src/client_fragments/builder.inc.rs:88-220)."""
        d = self._distributed
        if d is None:
            return None
        import os
        import torch.distributed as dist
        world = dist.get_world_size() if dist.is_initialized() else int(os.environ.get("WORLD_SIZE", "1"))
        d.validate(world)
        p = d.parallel
        if p.pp > 1 or p.cp > 1 or (p.ep > 1 and not p.ep_shares_tp):
            raise GllmError("Client: only tensor-parallel layouts (tp = world size) are built by the client; pipeline, "
                            "expert-parallel and context-parallel layouts go through the engine-level APIs")
        if p.tp == 1:
            return None
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if dev.type == "cuda":
                dist.init_process_group("nccl", device_id=dev)
            else:
                dist.init_process_group("gloo")
        from .parallel.tensor_parallel import TPContext, mode_for_comm_config
        return TPContext(dist.get_rank(), world, dev, mode=mode_for_comm_config(d.comm) if dev.type == "cuda" else "nccl",
                         max_tokens=self.config.max_batch_tokens, hidden=cfg.hidden_size)

    @staticmethod
    def _env_debug() -> bool:
        """GLLM_DEBUG_JIT=1 in the environment turns the debug serving mode on, like ``ClientBuilder.debug_jit()``."""
        import os
        return os.environ.get("GLLM_DEBUG_JIT", "0") not in ("", "0", "false", "False")

    _BITS_4 = ("q4", "q5", "iq4", "q3", "iq3", "q2", "iq2", "iq1", "awq", "gptq", "nvfp4", "mxfp4", "int4")
    _BITS_8 = ("q8", "q6", "fp8", "mxfp8", "int8")

    def _weight_quant_plan(self, cfg, dev) -> Optional[str]:
        """``DecoderModel(weight_quant=...)`` for this checkpoint on this device (see ``ClientConfig.weight_quant``)."""
        from .models.weights import can_fuse
        want = (self.config.weight_quant or "bf16").lower()
        if want in ("bf16", "none", ""):
            return None
        if want not in ("auto", "mxfp8", "nvfp4"):
            raise ValueError(f"weight_quant must be bf16, auto, mxfp8 or nvfp4, got {want!r}")
        if want == "auto":
            if dev.type != "cuda":
                return None
            tags = (cfg.quant or "").lower()
            want = "nvfp4" if any(t in tags for t in self._BITS_4) else ("mxfp8" if any(t in tags for t in self._BITS_8) else "")
            if not want:
                return None
        mult = 256 if want == "nvfp4" else 128
        shapes_ok = (can_fuse(cfg, 1) and not cfg.is_mla and cfg.hidden_size % mult == 0 and
                     (cfg.is_moe or cfg.intermediate_size % mult == 0) and (cfg.num_heads * cfg.head_dim) % mult == 0)
        if not shapes_ok:
            if self.config.weight_quant.lower() == "auto":
                return None
            raise ValueError(f"{want}: the model's shapes do not fit the block-scaled fused layer")
        return want

    def _kv_cache_plan(self, cfg, dev) -> dict:
        """Precision of the KV cache for this model on this device. ``auto`` asks the KV decision matrix
        (kv_cache/decision.py) whether the bf16 cache for max_num_seqs x max_model_len tokens fits beside the weights;
        when it does not, or when the checkpoint asks for it, the cache is fp8 (e4m3), the low-precision tier the
        attention kernels read directly. The chosen variant is kept in ``self.kv_plan``."""
        from .kv_cache.decision import HardwareProfile, KvDecisionMatrix
        pref = (self.config.kv_cache_dtype or "auto").lower()
        hw = HardwareProfile()
        if dev.type == "cuda":
            hw = HardwareProfile(hbm_bytes=int(torch.cuda.get_device_properties(dev).total_memory))
        tokens = self.config.max_num_seqs * self.config.max_model_len
        bf16_per_token = cfg.kv_bytes_per_token() * (2 if cfg.kv_cache_dtype in ("fp8", "fp8_e4m3") else 1)
        variant = KvDecisionMatrix(hw).choose(bf16_per_token * tokens, cfg.param_count() * 2,
                                              long_context=self.config.max_model_len > 32768,
                                              latency_sensitive=self.config.intent == "latency")
        want_fp8 = pref in ("fp8", "fp8_e4m3") or (pref == "auto" and (variant.kivi or cfg.kv_cache_dtype in ("fp8", "fp8_e4m3")))
        self.kv_plan = {"variant": variant, "kv_cache_dtype": "fp8" if want_fp8 and dev.type == "cuda" else "bf16",
                        "bf16_bytes": bf16_per_token * tokens}
        if want_fp8 and dev.type == "cuda" and not cfg.is_mla:
            return dict(kv_dtype=torch.float8_e4m3fn, kv_scale=float(self.config.kv_scale))
        return {}

    def unload_model(self):
        with self._lock:
            self._state = None
            if torch.cuda.is_available():
                torch.cuda.empty_cache()

    def swap_model(self, model_id: str, kind: Optional[ModelKind] = None):
        self.unload_model()
        self.load_model(model_id, kind)

    def _st(self) -> _State:
        st = self._state
        if st is None:
            raise NoModelLoadedError("no model is loaded")
        return st

    # ---- tokenizer ------------------------------------------------------------------------------
    def encode(self, text: str) -> List[int]:
        return self._st().tokenizer.encode(text)

    def decode(self, ids: Sequence[int]) -> str:
        return self._st().tokenizer.decode(ids)

    # ---- generation -----------------------------------------------------------------------------
    def generate(self, prompt) -> GenerationBuilder:
        return GenerationBuilder(self, prompt)

    def _prompt_ids(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            return self._st().tokenizer.encode(prompt)
        return [int(t) for t in prompt]

    def _hook_fn(self, hooks: List[GenerationHook]):
        if not hooks:
            return None

        def fn(rid, tok, n):
            for h in hooks:
                d = h.post_step(tok, n)
                if d != HookDecision.CONTINUE:
                    return d.value
            return None
        return fn

    def _execute_generation(self, b: GenerationBuilder, stream_cb=None) -> GenerationResponse:
        st = self._st()
        if st.engine is None:
            raise InvalidModelTypeError("generate() needs a decoder model")
        ids = self._prompt_ids(b._prompt)
        eos = st.tokenizer.eos_ids(st.model.cfg.eos_token_ids) + list(b._stop)
        if b._images or b._audio:
            return self._execute_multimodal(b, ids, eos)
        stop_hook = StopStringHook(st.tokenizer.decode, b._stop_strings) if b._stop_strings else None
        hooks = list(b._hooks) + ([stop_hook] if stop_hook else [])
        with self._lock:
            try:
                rid = st.engine.add_request(ids, max_tokens=b._max_tokens, temperature=b._temperature, top_k=b._top_k,
                                            top_p=b._top_p, eos_ids=eos, session_id=b._session_id,
                                            hook=self._hook_fn(hooks), stream=stream_cb)
            except ValueError as e:
                raise RuntimeGllmError(str(e)) from e
            keep_cb = st.engine.cfg.callbacks
            if b._callbacks is not None:
                st.engine.cfg.callbacks = b._callbacks       # the lock is held: this request runs alone
            try:
                st.engine.run_until_done()
            finally:
                st.engine.cfg.callbacks = keep_cb
            res: GenerateResult = st.engine.results.pop(rid)
        toks = res.token_ids
        if toks and toks[-1] in eos and res.finish_reason == "eos":
            toks = toks[:-1]
        text = st.tokenizer.decode(toks)
        thinking, answer = split_thinking_content(text) if b._reasoning else ("", text)
        reason = res.finish_reason
        if stop_hook is not None and stop_hook.hit:
            answer, reason = stop_hook.cut(answer), "stop"
        t = res.telemetry
        return GenerationResponse(text=answer, token_ids=toks, finish_reason=reason, thinking=thinking,
                                  prompt_tokens=t.prompt_tokens, cached_prefix_tokens=t.cached_prefix_tokens,
                                  ttft_ms=t.ttft_ms, tpot_ms=t.tpot_ms)

    def _execute_multimodal(self, b: GenerationBuilder, ids, eos) -> GenerationResponse:
        """Prompts with image / audio inputs: the encoder's features replace the placeholder tokens' embeddings and
        the sequence runs on a private KV cache (client_impl.inc.rs generate_with_multimodal)."""
        from .engine.simple_generate import generate_single
        st = self._st()
        enc = self._multimodal_encoder
        if enc is None:
            raise InvalidModelTypeError("image / audio inputs need set_multimodal_encoder(...) first")
        images = torch.stack([torch.as_tensor(i) for i in b._images]) if b._images else None
        waves = torch.stack([torch.as_tensor(a) for a in b._audio]) if b._audio else None
        table = st.model.embed
        if st.model.cfg.embedding_scale not in (None, 0, 1.0):
            table = table.float() * st.model.cfg.embedding_scale
        with self._lock:
            ids2, embeds = enc.prepare(ids, table, images=images, waves=waves)
            toks = generate_single(st.model, ids2, b._max_tokens, input_embeds=embeds, temperature=b._temperature,
                                   top_k=b._top_k, top_p=b._top_p, eos_ids=eos)
        reason = "eos" if toks and toks[-1] in eos else "length"
        if reason == "eos":
            toks = toks[:-1]
        text = st.tokenizer.decode(toks)
        thinking, answer = split_thinking_content(text) if b._reasoning else ("", text)
        return GenerationResponse(text=answer, token_ids=toks, finish_reason=reason, thinking=thinking,
                                  prompt_tokens=len(ids2), cached_prefix_tokens=0, ttft_ms=0.0, tpot_ms=0.0)

    def _execute_generation_stream(self, b: GenerationBuilder) -> GenerationStream:
        st = self._st()
        stream = GenerationStream()
        pending: List[int] = []
        emitted = [""]

        def on_token(rid, tok):
            pending.append(tok)
            text = st.tokenizer.decode(pending)
            if text and not text.endswith("�"):
                stream._push(text[len(emitted[0]):])
                emitted[0] = text

        def work():
            try:
                stream._finish(self._execute_generation(b, on_token))
            except BaseException as e:  # delivered to the consumer
                stream._finish(error=e)
        threading.Thread(target=work, daemon=True).start()
        return stream

    def generate_batch(self, requests: Sequence[GenerateRequest]) -> List[GenerateResult]:
        """All requests in one scheduler run (continuous batching); results in request order."""
        st = self._st()
        if st.engine is None:
            raise InvalidModelTypeError("generate_batch() needs a decoder model")
        with self._lock:
            ids = []
            for r in requests:
                p = r.prompt_token_ids if r.prompt_token_ids is not None else st.tokenizer.encode(r.prompt)
                eos = st.tokenizer.eos_ids(st.model.cfg.eos_token_ids) + list(r.stop_token_ids or [])
                ids.append(st.engine.add_request(p, max_tokens=r.max_tokens, temperature=r.temperature, top_k=r.top_k,
                                                 top_p=r.top_p, eos_ids=eos, session_id=r.session_id))
            st.engine.run_until_done()
            out = [st.engine.results.pop(i) for i in ids]
        for r in out:
            r.text = st.tokenizer.decode(r.token_ids)
        return out

    # ---- embeddings / rerank / classify ---------------------------------------------------------
    def embed(self, texts) -> "EmbeddingsBuilder":
        return EmbeddingsBuilder(self, [texts] if isinstance(texts, str) else list(texts))

    def rerank(self, query: str, documents: Sequence[str]) -> "RerankBuilder":
        return RerankBuilder(self, query, list(documents))

    def classify(self, texts) -> "ClassifyBuilder":
        return ClassifyBuilder(self, [texts] if isinstance(texts, str) else list(texts))

    def _embed_raw(self, texts: List[str], pooling: Optional[str] = None) -> torch.Tensor:
        st = self._st()
        seqs = [st.tokenizer.encode(t) or [st.tokenizer.pad_id] for t in texts]
        if st.engine is None:
            return st.model.embed_batch(seqs, pooling).float().cpu()
        return self._decoder_hidden(seqs, pooling or "last")

    def _decoder_hidden(self, seqs, pooling: str, layer: Optional[int] = None) -> torch.Tensor:
        """Decoder-based embedding / mid-layer extraction: one flat prefill without touching the serving pool."""
        from . import ops
        from .engine.batch import ForwardBatch
        st = self._st()
        m, dev = st.model, st.model.device
        lens = [len(s) for s in seqs]
        T = sum(lens)
        pages = [(n + 15) // 16 for n in lens]
        kv = m.alloc_kv_cache(sum(pages) + 1)
        bt = torch.zeros((len(seqs), max(pages)), dtype=torch.int32, device=dev)
        slot = torch.empty(T, dtype=torch.int32, device=dev)
        starts, p0, o = [], 0, 0
        for i, n in enumerate(lens):
            bt[i, :pages[i]] = torch.arange(p0, p0 + pages[i], dtype=torch.int32, device=dev)
            slot[o:o + n] = p0 * 16 + torch.arange(n, dtype=torch.int32, device=dev)
            starts.append(o)
            o += n
            p0 += pages[i]
        q_start = torch.tensor(starts, dtype=torch.int32, device=dev)
        q_len = torch.tensor(lens, dtype=torch.int32, device=dev)
        batch = ForwardBatch(token_ids=torch.tensor([t for s in seqs for t in s], dtype=torch.int32, device=dev),
                             positions=torch.cat([torch.arange(n, dtype=torch.int32, device=dev) for n in lens]),
                             slot_mapping=slot, block_tables=bt, ctx_lens=q_len, q_start=q_start, q_len=q_len,
                             max_q_len=max(lens))
        if layer is None:
            x = m.forward(batch, kv, return_hidden=True)
            x = m.final_hidden(x)
        else:
            m.forward(batch, kv, return_hidden=True, capture_layers={layer})
            x = m.captured[layer]
        return ops.pool(x.contiguous(), q_start, q_len, pooling).float().cpu()

    def encode_to_layer(self, texts: Sequence[str], layer: int, pooling: str = "mean") -> torch.Tensor:
        st = self._st()
        return self._decoder_hidden([st.tokenizer.encode(t) for t in texts], pooling, layer)

    def score_tokens(self, prompt: str, candidates: Sequence[int]) -> List[float]:
        """Logits of candidate next tokens after ``prompt`` (head routing, generative reranking)."""
        from .engine.batch import ForwardBatch
        st = self._st()
        m, dev = st.model, st.model.device
        ids = st.tokenizer.encode(prompt)
        n = len(ids)
        kv = m.alloc_kv_cache((n + 15) // 16 + 1)
        batch = ForwardBatch(token_ids=torch.tensor(ids, dtype=torch.int32, device=dev),
                             positions=torch.arange(n, dtype=torch.int32, device=dev),
                             slot_mapping=torch.arange(n, dtype=torch.int32, device=dev),
                             block_tables=torch.arange((n + 15) // 16, dtype=torch.int32, device=dev)[None],
                             ctx_lens=torch.tensor([n], dtype=torch.int32, device=dev),
                             q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                             q_len=torch.tensor([n], dtype=torch.int32, device=dev), max_q_len=n,
                             logits_rows=torch.tensor([n - 1], dtype=torch.int64, device=dev))
        logits = m.forward(batch, kv)[0].float().cpu()
        return [float(logits[int(c)]) for c in candidates]

    def _rerank_scores(self, query: str, docs: List[str]) -> List[float]:
        st = self._st()
        if st.engine is None:
            seqs = [st.tokenizer.encode_pair(query, d) for d in docs]
            logits = st.model.score_batch(seqs).float().cpu()
            return [float(x) for x in (logits[:, 0] if logits.shape[1] == 1 else logits[:, -1])]
        # generative decoder reranker: "q d" -> logit(yes) - logit(no) (executor_api.rs:655-688)
        yes = st.tokenizer.token_to_id("yes") or st.tokenizer.encode("yes", False)[0]
        no = st.tokenizer.token_to_id("no") or st.tokenizer.encode("no", False)[0]
        out = []
        for d in docs:
            y, n = self.score_tokens(f"{query} {d}", [yes, no])
            out.append(y - n)
        return out

    # ---- pipelines ------------------------------------------------------------------------------
    def rag(self, question: str, documents: Sequence[str], top_n: int = 3, max_tokens: int = 256) -> GenerationResponse:
        """embed -> rerank -> generate (client_impl.inc.rs:1499-1573). Auxiliary clients set with the builder's
        ``reranker()`` / ``generator()`` are used when present, else this client's own model."""
        docs = list(documents)
        rr = self._aux.get("reranker", self)
        ranked = rr.rerank(question, docs).top_n(top_n).generate()
        ctx = "\n".join(docs[r.index] for r in ranked)
        gen = self._aux.get("generator", self)
        return gen.generate(f"Context:\n{ctx}\n\nQuestion: {question}\nAnswer:").max_tokens(max_tokens).generate()

    def set_multimodal_encoder(self, encoder):
        self._multimodal_encoder = encoder

    # ---- diagnostics ----------------------------------------------------------------------------
    def diagnostics(self) -> dict:
        st = self._st()
        d = {"model": st.model_id, "kind": st.kind.value, "backend": st.backend.name, "device": str(st.model.device)}
        if st.engine is not None:
            d.update(stats=dict(st.engine.stats), free_pages=st.engine.batcher.num_free_pages,
                     cached_pages=st.engine.batcher.cached_pages, fused=st.model.fused)
        return d


@dataclass
class EmbedConfig:
    normalize: bool = True
    dimension: Optional[int] = None
    pooling: Optional[str] = None


class EmbeddingsBuilder:
    def __init__(self, client: Client, texts: List[str]):
        self._c, self._texts, self._cfg = client, texts, EmbedConfig()
        self._rerank_query: Optional[str] = None
        self._top_n: Optional[int] = None

    def normalize(self, on: bool = True):
        self._cfg.normalize = on
        return self

    def dimension(self, d: int):
        self._cfg.dimension = int(d)
        return self

    def pooling(self, mode: str):
        self._cfg.pooling = mode
        return self

    def rerank_query(self, q: str):
        self._rerank_query = q
        return self

    def top_n(self, n: int):
        self._top_n = int(n)
        return self

    def generate(self):
        e = self._c._embed_raw(self._texts, self._cfg.pooling)
        if self._cfg.dimension:  # Matryoshka truncation happens before normalisation
            e = e[:, : self._cfg.dimension]
        if self._cfg.normalize:
            e = e / e.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        if self._rerank_query is not None:
            q = self._c.embed([self._rerank_query]).normalize(self._cfg.normalize).generate()[0]
            scores = (e @ torch.as_tensor(q)).tolist()
            order = sorted(range(len(scores)), key=lambda i: -scores[i])[: self._top_n or len(scores)]
            return [RerankResult(index=i, score=scores[i], document=self._texts[i]) for i in order]
        return [row.tolist() for row in e]


@dataclass
class RerankResult:
    index: int
    score: float
    document: str = ""


class RerankBuilder:
    def __init__(self, client: Client, query: str, docs: List[str]):
        self._c, self._q, self._docs, self._top_n = client, query, docs, None
        self._return_documents = True

    def top_n(self, n: int):
        self._top_n = int(n)
        return self

    def return_documents(self, on: bool):
        self._return_documents = on
        return self

    def generate(self) -> List[RerankResult]:
        scores = self._c._rerank_scores(self._q, self._docs)
        order = sorted(range(len(scores)), key=lambda i: -scores[i])[: self._top_n or len(scores)]
        return [RerankResult(i, scores[i], self._docs[i] if self._return_documents else "") for i in order]


@dataclass
class ClassifyResult:
    label: int
    score: float
    probabilities: List[float] = field(default_factory=list)


class ClassifyBuilder:
    def __init__(self, client: Client, texts: List[str]):
        self._c, self._texts = client, texts

    def generate(self) -> List[ClassifyResult]:
        st = self._c._st()
        if st.engine is not None:
            raise InvalidModelTypeError("classify() needs a model with a classifier head")
        seqs = [st.tokenizer.encode(t) or [st.tokenizer.pad_id] for t in self._texts]
        logits = st.model.score_batch(seqs).float().cpu()
        out = []
        for row in logits:
            row = torch.where(torch.isnan(row), torch.full_like(row, float("-inf")), row)  # NaN never wins
            p = torch.softmax(row, -1)
            k = int(p.argmax())
            out.append(ClassifyResult(k, float(p[k]), p.tolist()))
        return out


class AsyncClient:
    """Every call returns a ``concurrent.futures.Future``. With ``continuous=True`` generation requests go to a serving
    loop that owns the engine (``engine.serving.ServingLoop``): calls from many threads are batched together step by
    step instead of running one after the other; the future resolves to a ``GenerationResponse`` all the same."""

    def __init__(self, client: Client, workers: int = 1, continuous: bool = False):
        self._c = client
        self._pool = cf.ThreadPoolExecutor(max_workers=workers)
        self._loop = None
        if continuous:
            from .engine.serving import ServingLoop
            st = client._st()
            if st.engine is None:
                raise InvalidModelTypeError("continuous generation needs a decoder model")
            self._loop = ServingLoop(st.engine)

    def _generate_continuous(self, prompt, kw) -> "cf.Future":
        c, st = self._c, self._c._st()
        b = c.generate(prompt)
        for k, v in kw.items():
            getattr(b, k)(v)
        ids = c._prompt_ids(b._prompt)
        eos = st.tokenizer.eos_ids(st.model.cfg.eos_token_ids) + list(b._stop)
        stream, on_token = None, None
        if b._stream:          # pieces of text arrive on ``future.stream`` while the request runs in the shared batch
            stream, pending, emitted = GenerationStream(), [], [""]

            def on_token(rid, tok):
                pending.append(tok)
                text = st.tokenizer.decode(pending)
                if text and not text.endswith("\ufffd"):
                    stream._push(text[len(emitted[0]):])
                    emitted[0] = text
        stop_hook = StopStringHook(st.tokenizer.decode, b._stop_strings) if b._stop_strings else None
        hooks = list(b._hooks) + ([stop_hook] if stop_hook else [])
        inner = self._loop.submit(ids, max_tokens=b._max_tokens, temperature=b._temperature, top_k=b._top_k, top_p=b._top_p,
                                  eos_ids=eos, session_id=b._session_id, hook=c._hook_fn(hooks), stream=on_token)
        outer: "cf.Future" = cf.Future()
        outer.stream = stream

        def done(f):
            try:
                res = f.result()
            except Exception as exc:
                if stream is not None:
                    stream._finish(error=exc)
                outer.set_exception(exc)
                return
            toks = res.token_ids
            if toks and toks[-1] in eos and res.finish_reason == "eos":
                toks = toks[:-1]
            text = st.tokenizer.decode(toks)
            thinking, answer = split_thinking_content(text) if b._reasoning else ("", text)
            t, reason = res.telemetry, res.finish_reason
            if stop_hook is not None and stop_hook.hit:
                answer, reason = stop_hook.cut(answer), "stop"
            resp = GenerationResponse(text=answer, token_ids=toks, finish_reason=reason, thinking=thinking,
                                      prompt_tokens=t.prompt_tokens, cached_prefix_tokens=t.cached_prefix_tokens,
                                      ttft_ms=t.ttft_ms, tpot_ms=t.tpot_ms)
            if stream is not None:
                if len(text) > len(emitted[0]) and text.startswith(emitted[0]):
                    stream._push(text[len(emitted[0]):])       # a tail that was held back as an incomplete character
                stream._finish(resp)
            outer.set_result(resp)
        inner.add_done_callback(done)
        outer.inner = inner
        return outer

    def cancel(self, fut: "cf.Future", reason: str = "aborted") -> bool:
        """Continuous mode: end a submitted generation early."""
        return self._loop is not None and self._loop.cancel(getattr(fut, "inner", fut), reason)

    def generate(self, prompt, **kw) -> "cf.Future":
        if self._loop is not None:
            return self._generate_continuous(prompt, kw)

        def run():
            b = self._c.generate(prompt)
            for k, v in kw.items():
                getattr(b, k)(v)
            return b.generate()
        return self._pool.submit(run)

    def embed(self, texts, **kw) -> "cf.Future":
        return self._pool.submit(lambda: self._c.embed(texts).generate())

    def rerank(self, query, docs, top_n=None) -> "cf.Future":
        return self._pool.submit(lambda: (self._c.rerank(query, docs).top_n(top_n) if top_n else self._c.rerank(query, docs)).generate())

    def generate_batch(self, requests) -> "cf.Future":
        return self._pool.submit(lambda: self._c.generate_batch(requests))

    def shutdown(self):
        if self._loop is not None:
            self._loop.shutdown()
        self._pool.shutdown(wait=True)
