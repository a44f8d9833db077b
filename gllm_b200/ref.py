"""ctypes front end of the scalar C++ CPU reference (``csrc/ref/cpuref.cpp``): correctness oracle and timed CPU
baseline for small Llama-style models.

    python -m gllm_b200.ref --model smollm2-135m --prompt-len 32 --new-tokens 32

prints tokens/s of greedy decoding on the host CPU (fp32, paged KV, random-init weights of that shape).
"""
from __future__ import annotations

import ctypes
import json
import time
from ctypes import POINTER, c_float, c_int, c_void_p
from pathlib import Path
from typing import List, Sequence

import torch

_LIB = Path(__file__).resolve().parent / "_lib" / "libgllm_cpuref.so"
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not _LIB.exists():
            raise RuntimeError(f"{_LIB} missing: run `python -m gllm_b200.build`")
        L = ctypes.CDLL(str(_LIB))
        L.gllm_ref_create.restype = c_void_p
        L.gllm_ref_create.argtypes = [c_int] * 8 + [c_float, c_float, c_void_p, c_void_p, c_void_p, c_int]
        L.gllm_ref_set_layer.argtypes = [c_void_p, c_int, c_void_p]
        L.gllm_ref_destroy.argtypes = [c_void_p]
        L.gllm_ref_reset.argtypes = [c_void_p]
        L.gllm_ref_forward.restype = c_int
        L.gllm_ref_forward.argtypes = [c_void_p, c_void_p, c_int, c_void_p]
        L.gllm_ref_generate_greedy.restype = c_int
        L.gllm_ref_generate_greedy.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        L.gllm_ref_sample.restype = c_int
        L.gllm_ref_sample.argtypes = [c_void_p, c_int, c_float, c_int, c_float, c_float]
        L.gllm_ref_moe_gate_topk.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p]
        _lib = L
    return _lib


class CpuReferenceModel:
    """Dense Llama / Qwen3-style decoder in scalar fp32 C++."""

    def __init__(self, cfg, src, num_pages: int = 64):
        if cfg.is_moe or cfg.is_mla or cfg.rotary_dim != cfg.head_dim or cfg.hidden_act != "silu":
            raise ValueError("the scalar reference covers dense RMSNorm / full-RoPE / SwiGLU decoders")
        self.cfg = cfg
        f = lambda name: src.get(name).float().contiguous()
        self._keep = []

        def keep(t):
            self._keep.append(t)
            return t.data_ptr()
        embed = f("embed_tokens")
        head = f("lm_head") if src.has("lm_head") and not cfg.tie_word_embeddings else embed
        self.h = lib().gllm_ref_create(cfg.num_layers, cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim,
                                       cfg.intermediate_size, cfg.vocab_size, 1 if cfg.qk_norm else 0, cfg.rms_norm_eps,
                                       cfg.rope_theta, keep(embed), keep(head), keep(f("final_norm")), num_pages)
        names = ["input_norm", "post_attn_norm", "q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "gate_proj",
                 "up_proj", "down_proj"]
        for l in range(cfg.num_layers):
            ptrs = (c_void_p * 11)()
            for i, n in enumerate(names):
                if n in ("q_norm", "k_norm") and not cfg.qk_norm:
                    ptrs[i] = None
                else:
                    ptrs[i] = keep(f(f"L{l}.{n}"))
            lib().gllm_ref_set_layer(self.h, l, ptrs)

    def reset(self):
        lib().gllm_ref_reset(self.h)

    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        t = torch.tensor(list(tokens), dtype=torch.int32)
        out = torch.empty(self.cfg.vocab_size, dtype=torch.float32)
        n = lib().gllm_ref_forward(self.h, t.data_ptr(), t.numel(), out.data_ptr())
        if n < 0:
            raise RuntimeError("sequence longer than the reference KV pool")
        return out

    def generate_greedy(self, prompt: Sequence[int], max_new: int, eos: int = -1) -> List[int]:
        t = torch.tensor(list(prompt), dtype=torch.int32)
        out = torch.zeros(max_new, dtype=torch.int32)
        n = lib().gllm_ref_generate_greedy(self.h, t.data_ptr(), t.numel(), max_new, eos, out.data_ptr())
        return out[:max(n, 0)].tolist()

    def __del__(self):
        try:
            lib().gllm_ref_destroy(self.h)
        except Exception:
            pass


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    l = logits.float().contiguous()
    return int(lib().gllm_ref_sample(l.data_ptr(), l.numel(), temperature, top_k, top_p, u))


def moe_gate_topk(logits: torch.Tensor, k: int):
    l = logits.float().contiguous()
    ids, w = torch.zeros(k, dtype=torch.int32), torch.zeros(k, dtype=torch.float32)
    lib().gllm_ref_moe_gate_topk(l.data_ptr(), l.numel(), k, ids.data_ptr(), w.data_ptr())
    return ids, w


def main():
    import argparse
    from .models.config import preset
    from .models.weights import RandomWeights
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="smollm2-135m")
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--new-tokens", type=int, default=32)
    a = ap.parse_args()
    cfg = preset(a.model)
    m = CpuReferenceModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=0), num_pages=(a.prompt_len + a.new_tokens) // 16 + 2)
    prompt = list(range(1, a.prompt_len + 1))
    t0 = time.perf_counter()
    m.forward(prompt)
    t1 = time.perf_counter()
    m.reset()
    out = m.generate_greedy(prompt, a.new_tokens)
    t2 = time.perf_counter()
    decode_s = (t2 - t1) - (t1 - t0)
    print(json.dumps({"model": a.model, "impl": "scalar C++ fp32 CPU reference", "prompt_tokens": a.prompt_len,
                      "new_tokens": len(out), "prefill_s": round(t1 - t0, 3),
                      "decode_ms_per_token": round(1e3 * decode_s / max(len(out) - 1, 1), 2),
                      "decode_tokens_per_s": round(max(len(out) - 1, 1) / max(decode_s, 1e-9), 2)}))


if __name__ == "__main__":
    main()
