"""Model loader: resolve a model id or path, detect the weight format, expose tensors under canonical names,
derive the ``ModelConfig`` and the tokenizer.

Reference parity: ``Loader::from_source_with_config(id).load()`` (src/loader/fragments/loader_impl.inc.rs:83-
321), ``LoaderConfig`` with cache dir ``~/.gllm/models`` or ``$GLLM_CACHE_DIR``, HF -> ModelScope fallback,
checksum policy, GGUF file filter (types.inc.rs:133-176), ``WeightFormat{SafeTensors,Gguf,Onnx,PyTorch,Gllm}``
(types.inc.rs:730-788), architecture detection from tensors when metadata is missing.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..models import arch as arch_mod
from ..models.config import ModelConfig
from . import gguf as gguf_mod
from . import pairing
from . import safetensors as st_mod
from .name_map import TensorRole, match_tensor_role


class WeightFormat(str, Enum):
    SAFETENSORS = "safetensors"
    GGUF = "gguf"
    ONNX = "onnx"
    PYTORCH = "pytorch"
    GLLM = "gllm"


class ModelNotFound(FileNotFoundError):
    pass


@dataclass
class LoaderConfig:
    cache_dir: Path = field(default_factory=lambda: Path(os.environ.get("GLLM_CACHE_DIR", Path.home() / ".gllm" / "models")))
    source: str = "huggingface"       # huggingface | modelscope
    fallback: bool = True             # try the other hub when the first one fails
    verify_checksums: bool = True
    gguf_file_filter: Optional[str] = None   # substring / regex picking one quantisation of a multi-file repo
    offline: bool = field(default_factory=lambda: os.environ.get("HF_HUB_OFFLINE", "0") == "1")
    dtype: torch.dtype = torch.bfloat16
    static_compression: str = field(default_factory=lambda: os.environ.get("GLLM_STATIC_COMPRESSION", ""))
    #   "" | "dead_columns": FFN neurons whose gate / up row or down column is zero are dropped when the layer is packed
    device_weight_budget: Optional[int] = None    # bytes of device memory for weights: a tier plan is attached when set
    host_weight_budget: int = 256 << 30

    @staticmethod
    def from_env() -> "LoaderConfig":
        return LoaderConfig()


def detect_format(path: Path, gguf_filter: Optional[str] = None):
    """-> (WeightFormat, [files])"""
    if path.is_file():
        suf = path.suffix.lower()
        fmt = {".gguf": WeightFormat.GGUF, ".safetensors": WeightFormat.SAFETENSORS, ".onnx": WeightFormat.ONNX,
               ".bin": WeightFormat.PYTORCH, ".pt": WeightFormat.PYTORCH, ".pth": WeightFormat.PYTORCH,
               ".gllm": WeightFormat.GLLM}.get(suf)
        if fmt is None:
            raise ValueError(f"unknown weight file type: {path}")
        return fmt, [path]
    for pattern, fmt in (("*.gllm", WeightFormat.GLLM), ("*.safetensors", WeightFormat.SAFETENSORS),
                         ("*.gguf", WeightFormat.GGUF), ("*.onnx", WeightFormat.ONNX),
                         ("pytorch_model*.bin", WeightFormat.PYTORCH)):
        files = sorted(path.glob(pattern))
        if fmt == WeightFormat.GGUF and gguf_filter and files:
            rx = re.compile(gguf_filter, re.I)
            files = [f for f in files if rx.search(f.name)] or files
        if files:
            return fmt, files
    raise ModelNotFound(f"no weight files under {path}")


class TensorProvider:
    """Uniform access to a checkpoint: canonical name -> tensor, lazily materialised."""

    def __init__(self):
        self.external_to_canon: Dict[str, str] = {}
        self.canon_to_external: Dict[str, str] = {}
        self.shapes: Dict[str, tuple] = {}
        self.quant_summary: Dict[str, int] = {}

    def has(self, name: str) -> bool:
        return name in self.canon_to_external or name in getattr(self, "_derived", {})

    def names(self):
        return list(self.canon_to_external)

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError


class SafeTensorsProvider(TensorProvider):
    def __init__(self, path, dtype=torch.bfloat16):
        super().__init__()
        self.model = st_mod.SafeTensorsModel(path)
        self.dtype = dtype
        names = list(self.model.keys())
        self.groups = {g.prefix: g for g in pairing.detect_groups(names)}
        consumed = set()
        for g in self.groups.values():
            consumed.update(g.members.values())
            self.quant_summary[g.kind] = self.quant_summary.get(g.kind, 0) + 1
        self._group_of: Dict[str, pairing.QuantGroup] = {}
        for n in names:
            dt, shape = self.model.meta(n)
            self.shapes[n] = shape
        for prefix, g in self.groups.items():
            role, layer, canon, _ = match_tensor_role(prefix + ".weight")
            if canon:
                self.canon_to_external[canon] = prefix
                self._group_of[canon] = g
            if "bias" in g.members:
                _, _, cb, _ = match_tensor_role(prefix + ".bias")
                if cb:
                    self.canon_to_external[cb] = g.members["bias"]
        for n in names:
            if n in consumed and not n.endswith("_bias"):
                continue
            role, layer, canon, suffix = match_tensor_role(n)
            if canon and canon not in self.canon_to_external:
                self.canon_to_external[canon] = n
                self.external_to_canon[n] = canon

    def get(self, name: str) -> torch.Tensor:
        if name in self._group_of:
            w = pairing.dequant_group(self._group_of[name], self.model.tensor)
            return w.to(self.dtype)
        ext = self.canon_to_external[name]
        t = self.model.tensor(ext)
        if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.float()
        if t.is_floating_point() and not name.rsplit(".", 1)[-1].endswith("norm"):
            t = t.to(self.dtype)
        return t.clone() if not t.is_floating_point() else t

    def raw_group(self, name: str):
        """The quantised members of a weight (for GPU paths that keep it quantised)."""
        g = self._group_of.get(name)
        return None if g is None else {k: self.model.tensor(v) for k, v in g.members.items()}


def _unpermute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """GGUF llama-family files store q/k rows permuted for interleaved RoPE; undo it for half-split RoPE."""
    out, inn = w.shape
    hd = out // n_head
    return w.reshape(n_head, hd // 2, 2, inn).transpose(1, 2).reshape(out, inn)


class GgufProvider(TensorProvider):
    PERMUTED_ARCHS = ("llama", "mistral", "mixtral")

    def __init__(self, files, dtype=torch.bfloat16):
        super().__init__()
        self.files = gguf_mod.open_multi(files)
        self.dtype = dtype
        self.metadata = {}
        for f in self.files:
            self.metadata.update(f.metadata)
        self._where = {}
        for f in self.files:
            for n, ti in f.tensors.items():
                self._where[n] = f
                self.shapes[n] = ti.shape
                self.quant_summary[ti.type_name] = self.quant_summary.get(ti.type_name, 0) + 1
                role, layer, canon, suffix = match_tensor_role(n)
                if canon:
                    if ".experts.stacked." in canon:
                        canon = canon  # expanded lazily in get()
                    self.canon_to_external[canon] = n
                    self.external_to_canon[n] = canon
        self.arch = str(self.metadata.get("general.architecture", "llama"))
        self.n_head = int(self.metadata.get(f"{self.arch}.attention.head_count", 0) or 0)
        kv = self.metadata.get(f"{self.arch}.attention.head_count_kv", self.n_head)
        self.n_head_kv = int(max(kv) if isinstance(kv, (list, tuple)) else kv or self.n_head)

    def has(self, name: str) -> bool:
        if name in self.canon_to_external:
            return True
        m = re.match(r"(L\d+)\.experts\.(\d+)\.(\w+)$", name)
        return bool(m) and f"{m.group(1)}.experts.stacked.{m.group(3)}" in self.canon_to_external

    def get(self, name: str) -> torch.Tensor:
        m = re.match(r"(L\d+)\.experts\.(\d+)\.(\w+)$", name)
        if m and name not in self.canon_to_external:
            stacked = self.get(f"{m.group(1)}.experts.stacked.{m.group(3)}")
            return stacked[int(m.group(2))]
        ext = self.canon_to_external[name]
        t = self._where[ext].tensor(ext)
        base = name.rsplit(".", 1)[-1]
        if self.arch in self.PERMUTED_ARCHS and base in ("q_proj", "k_proj") and t.dim() == 2:
            t = _unpermute_qk(t, self.n_head if base == "q_proj" else self.n_head_kv)
        if base.endswith("norm"):
            return t.float()
        return t.to(self.dtype)

    def raw(self, name: str):
        ext = self.canon_to_external[name]
        f = self._where[ext]
        return f.tensors[ext], f.raw(ext)


@dataclass
class LoadedModel:
    path: Path
    format: WeightFormat
    config: ModelConfig
    weights: TensorProvider
    tokenizer: Optional[object]
    features: Optional[arch_mod.ArchFeatures] = None
    tier_plan: Optional[list] = None      # loader/weight_tier.py placements when a device budget was given

    def plan_tiers(self, device_budget: int, host_budget: int = 256 << 30, bytes_per_element: int = 2):
        """Which tensors stay on the device, which go to pinned host memory and which stay memory-mapped, for a device
        budget in bytes (loader/weight_tier.py: attention, norms, router and embeddings always stay resident)."""
        from .weight_tier import plan_weight_tiers
        sizes = {}
        for name, shape in self.weights.shapes.items():
            n = 1
            for d in shape:
                n *= int(d)
            sizes[name] = n * bytes_per_element
        self.tier_plan = plan_weight_tiers(sizes, device_budget, host_budget)
        return self.tier_plan


class Loader:
    def __init__(self, source: str, config: Optional[LoaderConfig] = None):
        self.source, self.cfg = source, config or LoaderConfig.from_env()

    @staticmethod
    def from_source_with_config(source: str, config: Optional[LoaderConfig] = None) -> "Loader":
        return Loader(source, config)

    # ------------------------------------------------------------------------------------------
    def resolve(self) -> Path:
        p = Path(self.source).expanduser()
        if p.exists():
            return p
        from .hub import resolve_model
        return resolve_model(self.source, self.cfg)

    def load(self) -> LoadedModel:
        path = self.resolve()
        fmt, files = detect_format(path, self.cfg.gguf_file_filter)
        root = path if path.is_dir() else path.parent
        tokenizer = None
        if fmt == WeightFormat.GGUF:
            prov = GgufProvider(files, self.cfg.dtype)
            cfg = ModelConfig.from_gguf_metadata(prov.metadata)
            try:
                from ..tokenizer import TokenizerHandle
                tokenizer = TokenizerHandle.from_gguf(prov.files[0])
            except Exception:
                tokenizer = None
        elif fmt == WeightFormat.SAFETENSORS:
            prov = SafeTensorsProvider(path, self.cfg.dtype)
            cfg = self._config_for(root, prov)
        elif fmt == WeightFormat.GLLM:
            from .gllm_format import GllmProvider
            prov = GllmProvider(files[0], self.cfg.dtype)
            cfg = ModelConfig.from_hf_dict(prov.metadata.get("config", {})) if prov.metadata.get("config") else \
                self._config_for(root, prov)
        elif fmt == WeightFormat.PYTORCH:
            from .pytorch_bin import PytorchProvider
            prov = PytorchProvider(files, self.cfg.dtype)
            cfg = self._config_for(root, prov)
        else:
            from .onnx import OnnxProvider
            prov = OnnxProvider(files[0], self.cfg.dtype)
            cfg = self._config_for(root, prov)
        feats = arch_mod.analyze_architecture(prov.shapes)
        self._reconcile(cfg, feats, prov)
        if tokenizer is None:
            tj = root / "tokenizer.json"
            if tj.exists():
                from ..tokenizer import TokenizerHandle
                tokenizer = TokenizerHandle.from_file(tj)
        if prov.quant_summary and not cfg.quant:
            cfg.quant = "+".join(sorted(prov.quant_summary))
        if self.cfg.static_compression:
            cfg.static_compression = self.cfg.static_compression
        loaded = LoadedModel(path=path, format=fmt, config=cfg, weights=prov, tokenizer=tokenizer, features=feats)
        if self.cfg.device_weight_budget is not None:
            loaded.plan_tiers(self.cfg.device_weight_budget, self.cfg.host_weight_budget)
        return loaded

    # ------------------------------------------------------------------------------------------
    def _config_for(self, root: Path, prov: TensorProvider) -> ModelConfig:
        cj = root / "config.json"
        if cj.exists():
            return ModelConfig.from_json_file(cj)
        gc = getattr(getattr(prov, "model", None), "gllm_config", lambda: None)()
        if gc:
            return ModelConfig.from_hf_dict(gc)
        feats = arch_mod.analyze_architecture(prov.shapes)
        return arch_mod.config_from_features(feats)

    @staticmethod
    def _reconcile(cfg: ModelConfig, f: arch_mod.ArchFeatures, prov: TensorProvider):
        """Tensor facts win over metadata where they disagree (the reference is tensor driven)."""
        if f.vocab_size and cfg.vocab_size != f.vocab_size:
            cfg.vocab_size = f.vocab_size
        if f.num_layers and cfg.num_layers != f.num_layers:
            cfg.num_layers = f.num_layers
        if f.hidden_size and cfg.hidden_size != f.hidden_size:
            cfg.hidden_size = f.hidden_size
        cfg.qk_norm = cfg.qk_norm or f.qk_norm
        cfg.attention_bias = f.attention_bias if f.roles.get(TensorRole.ATTN_QUERY.value) else cfg.attention_bias
        cfg.attention_sinks = cfg.attention_sinks or f.attention_sinks
        if f.is_decoder and not prov.has("lm_head"):
            cfg.tie_word_embeddings = True
        if f.num_experts and not cfg.num_experts:
            cfg.num_experts = f.num_experts
        if f.moe_intermediate and not cfg.moe_intermediate_size:
            cfg.moe_intermediate_size = f.moe_intermediate
        if f.q_out and cfg.num_heads and cfg.head_dim * cfg.num_heads != f.q_out and not cfg.is_mla:
            cfg.head_dim = f.q_out // cfg.num_heads
