"""Checkpoint formats, quantised block codecs, pairing, name mapping and the end-to-end Loader (CPU only)."""
import json
import struct

import numpy as np
import pytest
import torch

from gllm_b200.loader import Loader, LoaderConfig, WeightFormat
from gllm_b200.loader import gguf, pairing, quant, safetensors as st
from gllm_b200.loader.name_map import TensorRole, match_tensor_role
from gllm_b200.models import arch
from gllm_b200.models.config import ModelConfig, preset
from gllm_b200.models.weights import RandomWeights


def test_safetensors_roundtrip_and_sharded(tmp_path):
    t = {"a.weight": torch.randn(4, 6).to(torch.bfloat16), "b": torch.arange(5, dtype=torch.int32),
         "c": torch.randn(3, 2).to(torch.float8_e4m3fn), "e": torch.zeros(0, 4)}
    st.save_file({k: t[k] for k in ("a.weight", "b")}, tmp_path / "model-00001-of-00002.safetensors", {"gllm_config": "{\"x\":1}"})
    st.save_file({k: t[k] for k in ("c", "e")}, tmp_path / "model-00002-of-00002.safetensors")
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        "a.weight": "model-00001-of-00002.safetensors", "b": "model-00001-of-00002.safetensors",
        "c": "model-00002-of-00002.safetensors", "e": "model-00002-of-00002.safetensors"}}))
    m = st.SafeTensorsModel(tmp_path)
    assert set(m.keys()) == set(t) and m.gllm_config() == {"x": 1}
    for k in t:
        got = m.tensor(k)
        assert got.dtype == t[k].dtype and got.shape == t[k].shape
        assert torch.equal(got.view(torch.uint8) if got.numel() else got, t[k].view(torch.uint8) if got.numel() else t[k])
    (tmp_path / "bad.safetensors").write_bytes(struct.pack("<Q", 10 ** 12) + b"{}")
    with pytest.raises(st.SafeTensorsError):
        st.SafeTensorsFile(tmp_path / "bad.safetensors")


def _ref_q4_k(block: bytes) -> np.ndarray:
    """Independent decoder: d, dmin, 12 scale bytes (6-bit sc/m), 128 nibble bytes; 64-element groups."""
    d, dmin = np.frombuffer(block[:4], np.float16).astype(np.float32)
    sc = np.frombuffer(block[4:16], np.uint8)
    qs = np.frombuffer(block[16:], np.uint8)
    out = np.zeros(256, np.float32)
    for j in range(8):
        if j < 4:
            s, m = sc[j] & 63, sc[j + 4] & 63
        else:
            s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)
            m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
        q = qs[(j // 2) * 32:(j // 2) * 32 + 32]
        nib = (q & 0xF) if j % 2 == 0 else (q >> 4)
        out[j * 32:(j + 1) * 32] = d * s * nib - dmin * m
    return out


def _ref_q6_k(block: bytes) -> np.ndarray:
    ql, qh = np.frombuffer(block[:128], np.uint8), np.frombuffer(block[128:192], np.uint8)
    sc = np.frombuffer(block[192:208], np.int8)
    d = np.frombuffer(block[208:210], np.float16).astype(np.float32)[0]
    out = np.zeros(256, np.float32)
    for i in range(256):
        half, r = divmod(i, 128)
        quarter, l = divmod(r, 32)
        lo = ql[half * 64 + l + (32 if quarter in (1, 3) else 0)]
        lo4 = (lo & 0xF) if quarter < 2 else (lo >> 4)
        hi2 = (qh[half * 32 + l] >> (2 * quarter)) & 3
        out[i] = d * sc[half * 8 + quarter * 2 + l // 16] * (int(lo4 | (hi2 << 4)) - 32)
    return out


def test_k_quant_decoders_match_independent_reference():
    rng = np.random.RandomState(0)
    for name, ref in (("Q4_K", _ref_q4_k), ("Q6_K", _ref_q6_k)):
        t = quant.BY_NAME[name]
        raw = rng.randint(0, 256, size=t.block_bytes * 3, dtype=np.uint8)
        for b in range(3):  # keep the fp16 scale fields finite
            o = b * t.block_bytes
            pos = [0, 2] if name == "Q4_K" else [208]
            for p in pos:
                raw[o + p:o + p + 2] = np.frombuffer(np.float16(rng.rand() + 0.1).tobytes(), np.uint8)
        got = quant.dequantize(t.id, raw.tobytes(), 768).numpy()
        want = np.concatenate([ref(raw[b * t.block_bytes:(b + 1) * t.block_bytes].tobytes()) for b in range(3)])
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name,tol", [("Q8_0", 0.01), ("Q4_0", 0.12), ("Q4_K", 0.1), ("Q6_K", 0.03), ("MXFP4", 0.3),
                                      ("NVFP4", 0.2)])
def test_quantise_dequantise_roundtrip(name, tol):
    rng = np.random.RandomState(1)
    x = rng.randn(4, 512).astype(np.float32)
    raw = quant.QUANTIZERS[name](x)
    t = quant.BY_NAME[name]
    assert len(raw) == quant.nbytes(t.id, x.size)
    y = quant.dequantize(t.id, raw, x.size).numpy().reshape(x.shape)
    assert np.abs(y - x).max() <= tol * np.abs(x).max() + 1e-6
    assert np.corrcoef(x.ravel(), y.ravel())[0, 1] > 0.97


def test_every_supported_type_decodes_whole_blocks():
    rng = np.random.RandomState(2)
    for t in quant.TYPES.values():
        if not t.supported or t.block_elems == 1:
            continue
        raw = bytearray(rng.randint(0, 256, size=t.block_bytes * 2, dtype=np.uint8).tobytes())
        y = quant.dequantize(t.id, bytes(raw), t.block_elems * 2)
        assert y.shape == (t.block_elems * 2,)
    if quant.codebook_backend_available():      # lattice-codebook types decode through the gguf package's tables
        assert quant.dequantize(quant.BY_NAME["IQ2_XXS"].id, b"\0" * 66, 256).shape == (256,)
    else:
        with pytest.raises(NotImplementedError):
            quant.dequantize(quant.BY_NAME["IQ2_XXS"].id, b"\0" * 66, 256)
    with pytest.raises(NotImplementedError):     # a format nobody can decode stays an explicit error
        quant.dequantize(quant.BY_NAME["SQUEEZE"].id, b"\0" * 72, 128)
    # hand-built classic blocks (split nibbles: low nibble -> element j, high -> element j+16)
    blk = np.float16(0.5).tobytes() + bytes([0x1F] * 16)
    y = quant.dequantize(2, blk, 32).numpy()
    assert np.allclose(y[:16], (15 - 8) * 0.5) and np.allclose(y[16:], (1 - 8) * 0.5)
    blk = np.float16(2.0).tobytes() + struct.pack("<I", 0x00010001) + bytes([0x00] * 16)   # Q5_0: 5th bit of e0, e16
    y = quant.dequantize(6, blk, 32).numpy()
    assert y[0] == (16 - 16) * 2.0 and y[1] == -32.0 and y[16] == 0.0 and y[17] == -32.0
    blk = bytes([127]) + bytes([0x92] * 16)               # MXFP4: scale 2^0, codes 2 (=1.0) and 9 (= -0.5)
    y = quant.dequantize(39, blk, 32).numpy()
    assert np.allclose(y[:16], 1.0) and np.allclose(y[16:], -0.5)


def test_gguf_roundtrip_metadata_and_quantised_tensors(tmp_path):
    rng = np.random.RandomState(3)
    w = rng.randn(8, 256).astype(np.float32)
    md = {"general.architecture": "qwen3", "general.alignment": 64, "qwen3.block_count": 2,
          "qwen3.embedding_length": 256, "qwen3.attention.head_count": 2, "qwen3.attention.head_count_kv": 1,
          "qwen3.rope.freq_base": 1e6, "qwen3.context_length": 4096, "qwen3.feed_forward_length": 512,
          "qwen3.attention.layer_norm_rms_epsilon": 1e-6, "tokenizer.ggml.tokens": ["a", "b", "c"],
          "tokenizer.ggml.eos_token_id": 2, "flag": True}
    gguf.write_gguf(tmp_path / "m.gguf", md, {
        "blk.0.attn_q.weight": ("Q4_K", (8, 256), quant.quantize_q4_k(w)),
        "blk.0.ffn_down.weight": ("Q6_K", (8, 256), quant.quantize_q6_k(w)),
        "token_embd.weight": torch.from_numpy(w), "output_norm.weight": torch.ones(256).to(torch.float16)}, alignment=64)
    f = gguf.GgufFile(tmp_path / "m.gguf")
    assert f.version == 3 and f.alignment == 64 and f.architecture() == "qwen3" and f.get("flag") is True
    assert f.tokenizer_tokens() == ["a", "b", "c"] and f.arch_get("block_count") == 2
    assert f.tensors["blk.0.attn_q.weight"].shape == (8, 256) and f.tensors["blk.0.attn_q.weight"].type_name == "Q4_K"
    assert torch.equal(f.tensor("token_embd.weight"), torch.from_numpy(w))
    assert np.abs(f.tensor("blk.0.attn_q.weight").numpy() - w).max() < 0.12 * np.abs(w).max()
    assert np.abs(f.tensor("blk.0.ffn_down.weight").numpy() - w).max() < 0.04 * np.abs(w).max()
    cfg = ModelConfig.from_gguf_metadata(f.metadata)
    assert (cfg.arch, cfg.num_layers, cfg.hidden_size, cfg.num_kv_heads, cfg.qk_norm, cfg.vocab_size) == \
           ("qwen3", 2, 256, 1, True, 3) and cfg.eos_token_ids == [2]
    (tmp_path / "bad.gguf").write_bytes(b"NOPE" + b"\0" * 32)
    with pytest.raises(gguf.GgufError):
        gguf.GgufFile(tmp_path / "bad.gguf")


def test_awq_gptq_mxfp4_nvfp4_fp8_pairing():
    torch.manual_seed(4)
    N, K, g = 16, 256, 128
    q = torch.randint(0, 16, (K, N))
    z = torch.randint(0, 16, (K // g, N))
    s = torch.rand(K // g, N) * 0.1 + 0.01
    want = ((q - z.repeat_interleave(g, 0)).float() * s.repeat_interleave(g, 0)).t()

    def pack(vals, order):  # [R, C] nibbles -> [R, C/8] int32 with `order[i]` = position of logical element i
        r = vals.reshape(vals.shape[0], -1, 8).to(torch.int64)
        w = sum(r[:, :, i] << (4 * order[i]) for i in range(8))
        return torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)
    awq_pos = [pairing._AWQ_ORDER.index(i) for i in range(8)]
    got = pairing.dequant_awq(pack(q, awq_pos), s.half(), pack(z, awq_pos))
    torch.testing.assert_close(got, (((q - z.repeat_interleave(g, 0)).float()) * s.half().float().repeat_interleave(g, 0)).t())
    qw_gptq = pack(q.t().contiguous(), list(range(8))).t().contiguous()       # [K/8, N]
    got = pairing.dequant_gptq(qw_gptq, s.half(), pack((z - 1) & 0xF, list(range(8))), torch.arange(K) // g)
    torch.testing.assert_close(got, (((q - z.repeat_interleave(g, 0)).float()) * s.half().float().repeat_interleave(g, 0)).t())
    names = ["m.q.qweight", "m.q.scales", "m.q.qzeros", "m.q.g_idx", "m.k.qweight", "m.k.scales", "m.k.qzeros",
             "e.gate_up_proj_blocks", "e.gate_up_proj_scales", "e.gate_up_proj_bias", "d.weight", "d.weight_scale_inv",
             "f.weight", "f.weight_scale", "f.weight_scale_2"]
    kinds = {g_.prefix: g_.kind for g_ in pairing.detect_groups(names)}
    assert kinds == {"m.q": "gptq", "m.k": "awq", "e.gate_up_proj": "mxfp4", "d": "fp8_block", "f": "nvfp4_or_fp8"}
    # MXFP4: SafeTensors nibble order vs GGUF order decode to the same values
    blocks = torch.randint(0, 256, (4, 2, 16), dtype=torch.uint8)
    scales = torch.randint(120, 134, (4, 2), dtype=torch.uint8)
    a = pairing.dequant_mxfp4_st(blocks, scales)
    b = quant.dequantize(39, pairing.repack_mxfp4_to_gguf(blocks, scales), 4 * 64).reshape(4, 64)
    torch.testing.assert_close(a, b)
    # NVFP4: HF layout vs repacked 36-byte blocks
    w8 = torch.randint(0, 256, (4, 64), dtype=torch.uint8)
    sc = torch.rand(4, 8).clamp_min(0.1).to(torch.float8_e4m3fn).view(torch.uint8)
    a = pairing.dequant_nvfp4(w8, sc, torch.tensor([1.0]))
    b = quant.dequantize(53, pairing.repack_nvfp4_blocks(w8, sc), 4 * 128).reshape(4, 128)
    torch.testing.assert_close(a, b)
    # block FP8 and MXFP8 quantise -> dequantise
    w = torch.randn(200, 300)
    q8, si = pairing.quantize_fp8_block(w)
    assert si.shape == (2, 3) and (pairing.dequant_fp8_block(q8, si) - w).abs().max() < 0.07 * w.abs().max()
    w = torch.randn(8, 128)
    q8, e = pairing.quantize_mxfp8(w)
    assert (pairing.dequant_mxfp8(q8, e) - w).abs().max() < 0.07 * w.abs().max()


def test_name_roles_hf_gguf_bert():
    cases = {
        "model.layers.3.self_attn.q_proj.weight": (TensorRole.ATTN_QUERY, 3, "L3.q_proj"),
        "model.layers.0.self_attn.q_proj.bias": (TensorRole.ATTN_QUERY, 0, "L0.q_proj_bias"),
        "model.layers.1.self_attn.k_norm.weight": (TensorRole.ATTN_K_NORM, 1, "L1.k_norm"),
        "model.layers.2.mlp.experts.17.down_proj.weight": (TensorRole.MOE_EXPERT_DOWN, 2, "L2.experts.17.down_proj"),
        "model.layers.2.mlp.gate.weight": (TensorRole.MOE_ROUTER, 2, "L2.router"),
        "model.layers.5.self_attn.kv_a_proj_with_mqa.weight": (TensorRole.MLA_KV_COMPRESS, 5, "L5.kv_a_proj"),
        "model.embed_tokens.weight": (TensorRole.EMBEDDING, None, "embed_tokens"),
        "lm_head.weight": (TensorRole.OUTPUT_HEAD, None, "lm_head"), "model.norm.weight": (TensorRole.FINAL_NORM, None, "final_norm"),
        "blk.7.attn_q.weight": (TensorRole.ATTN_QUERY, 7, "L7.q_proj"), "blk.7.ffn_gate_exps.weight": (TensorRole.MOE_EXPERT_GATE, 7, "L7.experts.stacked.gate_proj"),
        "token_embd.weight": (TensorRole.EMBEDDING, None, "embed_tokens"), "output.weight": (TensorRole.OUTPUT_HEAD, None, "lm_head"),
        "bert.encoder.layer.1.attention.self.query.weight": (TensorRole.ATTN_QUERY, 1, "L1.q_proj"),
        "bert.encoder.layer.1.output.dense.weight": (TensorRole.FFN_DOWN, 1, "L1.down_proj"),
        "bert.embeddings.word_embeddings.weight": (TensorRole.EMBEDDING, None, "embed_tokens"),
        "model.layers.0.mlp.down_proj.qweight": (TensorRole.FFN_DOWN, 0, "L0.down_proj.qweight"),
    }
    for name, (role, layer, canon) in cases.items():
        r, l, c, _ = match_tensor_role(name)
        assert (r, l, c) == (role, layer, canon), name
    assert match_tensor_role("some.unrelated.tensor")[0] == TensorRole.UNKNOWN


def test_analyze_architecture_from_shapes():
    shapes = {"model.embed_tokens.weight": (32000, 512), "model.norm.weight": (512,)}
    for i in range(3):
        p = f"model.layers.{i}."
        shapes.update({p + "self_attn.q_proj.weight": (512, 512), p + "self_attn.k_proj.weight": (128, 512),
                       p + "self_attn.v_proj.weight": (128, 512), p + "self_attn.o_proj.weight": (512, 512),
                       p + "self_attn.q_norm.weight": (64,), p + "self_attn.k_norm.weight": (64,),
                       p + "input_layernorm.weight": (512,), p + "post_attention_layernorm.weight": (512,),
                       p + "mlp.gate.weight": (8, 512)})
        for e in range(8):
            shapes.update({p + f"mlp.experts.{e}.gate_proj.weight": (96, 512), p + f"mlp.experts.{e}.up_proj.weight": (96, 512),
                           p + f"mlp.experts.{e}.down_proj.weight": (512, 96)})
    f = arch.analyze_architecture(shapes)
    assert f.is_decoder and f.tied_embeddings and f.num_layers == 3 and f.qk_norm and f.ffn_type == "moe"
    assert f.num_experts == 8 and f.moe_intermediate == 96 and f.hidden_size == 512 and f.vocab_size == 32000
    cfg = arch.config_from_features(f, head_dim=64)
    assert (cfg.arch, cfg.num_heads, cfg.num_kv_heads, cfg.num_experts, cfg.tie_word_embeddings) == ("qwen3_moe", 8, 2, 8, True)
    enc = {"bert.embeddings.word_embeddings.weight": (30522, 128), "bert.embeddings.position_embeddings.weight": (512, 128),
           "bert.encoder.layer.0.attention.self.query.weight": (128, 128), "classifier.weight": (1, 128)}
    f = arch.analyze_architecture(enc)
    assert not f.is_decoder and f.has_classifier and f.num_labels == 1 and f.norm_type == "layer"
    assert arch.canonical_arch("Qwen3MoE") == "qwen3_moe" and arch.canonical_arch("xlm-roberta") == "bert"


def _hf_state(cfg, seed=0):
    src = RandomWeights(cfg, "cpu", torch.float32, seed=seed)
    sd = {"model.embed_tokens.weight": src.get("embed_tokens"), "model.norm.weight": src.get("final_norm")}
    if not cfg.tie_word_embeddings:
        sd["lm_head.weight"] = src.get("lm_head")
    m = {"q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj", "o_proj": "self_attn.o_proj",
         "q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm", "input_norm": "input_layernorm",
         "post_attn_norm": "post_attention_layernorm", "gate_proj": "mlp.gate_proj", "up_proj": "mlp.up_proj",
         "down_proj": "mlp.down_proj"}
    for i in range(cfg.num_layers):
        for c, h in m.items():
            if src.has(f"L{i}.{c}"):
                sd[f"model.layers.{i}.{h}.weight"] = src.get(f"L{i}.{c}")
    return src, sd


def test_loader_end_to_end_safetensors_gguf_gllm_bin(tmp_path):
    cfg = preset("tiny-qwen3")
    src, sd = _hf_state(cfg)
    d = tmp_path / "hf"
    d.mkdir()
    st.save_file(sd, d / "model.safetensors")
    (d / "config.json").write_text(json.dumps({
        "model_type": "qwen3", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
        "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 512, "vocab_size": 1024, "rope_theta": 1e6,
        "rms_norm_eps": 1e-6, "max_position_embeddings": 2048, "eos_token_id": 2, "tie_word_embeddings": False}))
    lm = Loader.from_source_with_config(str(d), LoaderConfig(dtype=torch.float32)).load()
    assert lm.format == WeightFormat.SAFETENSORS and lm.config.qk_norm and lm.config.num_layers == 2
    for n in ("embed_tokens", "L1.q_proj", "L0.k_norm", "L1.down_proj", "lm_head", "final_norm"):
        assert torch.equal(lm.weights.get(n).float(), src.get(n).float()), n
    # same model through GGUF (F32), .gllm (Q8_0) and a torch.save'd state dict
    md = {"general.architecture": "qwen3", "qwen3.block_count": 2, "qwen3.embedding_length": 256,
          "qwen3.attention.head_count": 4, "qwen3.attention.head_count_kv": 2, "qwen3.attention.key_length": 128,
          "qwen3.feed_forward_length": 512, "qwen3.rope.freq_base": 1e6, "qwen3.attention.layer_norm_rms_epsilon": 1e-6,
          "qwen3.context_length": 2048}
    gmap = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight", "lm_head.weight": "output.weight"}
    lmap = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
            "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm", "input_layernorm": "attn_norm",
            "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}
    gt = {}
    for k, v in sd.items():
        if k in gmap:
            gt[gmap[k]] = v
        else:
            _, _, i, rest = k.split(".", 3)
            gt[f"blk.{i}.{lmap[rest[:-len('.weight')]]}.weight"] = v
    gguf.write_gguf(tmp_path / "m.gguf", md, gt)
    lg = Loader(str(tmp_path / "m.gguf"), LoaderConfig(dtype=torch.float32)).load()
    assert lg.format == WeightFormat.GGUF and lg.config.head_dim == 128 and lg.config.vocab_size == 1024
    for n in ("embed_tokens", "L1.q_proj", "L0.k_norm", "L1.down_proj", "lm_head"):
        assert torch.equal(lg.weights.get(n).float(), src.get(n).float()), n
    from gllm_b200.loader.gllm_format import convert_to_gllm
    convert_to_gllm(lm, tmp_path / "m.gllm", quantize="Q8_0")
    l2 = Loader(str(tmp_path / "m.gllm"), LoaderConfig(dtype=torch.float32)).load()
    assert l2.format == WeightFormat.GLLM and l2.weights.quant_summary.get("Q8_0", 0) > 0
    w, w0 = l2.weights.get("L0.q_proj").float(), src.get("L0.q_proj").float()
    assert (w - w0).abs().max() < 0.01 * w0.abs().max() and torch.equal(l2.weights.get("embed_tokens").float(), src.get("embed_tokens"))
    b = tmp_path / "pt"
    b.mkdir()
    torch.save(sd, b / "pytorch_model.bin")
    (b / "config.json").write_text((d / "config.json").read_text())
    lp = Loader(str(b), LoaderConfig(dtype=torch.float32)).load()
    assert lp.format == WeightFormat.PYTORCH and torch.equal(lp.weights.get("L1.up_proj"), src.get("L1.up_proj"))


def test_gguf_llama_qk_rows_are_unpermuted(tmp_path):
    from gllm_b200.loader.loader import _unpermute_qk
    n_head, hd, inn = 2, 8, 4
    w = torch.arange(n_head * hd * inn, dtype=torch.float32).reshape(n_head * hd, inn)
    perm = w.reshape(n_head, 2, hd // 2, inn).transpose(1, 2).reshape(n_head * hd, inn)   # what the converter stores
    assert torch.equal(_unpermute_qk(perm, n_head), w)


def test_restricted_unpickler_refuses_code(tmp_path):
    import pickle
    import zipfile
    from gllm_b200.loader.pytorch_bin import load_state_dict
    class Evil:
        def __reduce__(self):
            return (print, ("pwned",))
    with zipfile.ZipFile(tmp_path / "evil.bin", "w") as z:
        z.writestr("archive/data.pkl", pickle.dumps({"x": Evil()}))
    with pytest.raises(pickle.UnpicklingError):
        load_state_dict(tmp_path / "evil.bin")


def test_onnx_initializers(tmp_path):
    from gllm_b200.loader.onnx import fused_patterns, read_onnx
    def vi(n):
        out = b""
        while True:
            b7 = n & 0x7F
            n >>= 7
            out += bytes([b7 | (0x80 if n else 0)])
            if not n:
                return out
    def ld(fn, payload):
        return vi((fn << 3) | 2) + vi(len(payload)) + payload
    def tensor(name, arr):
        b = b"".join(vi((1 << 3) | 0) + vi(d) for d in arr.shape) + vi((2 << 3) | 0) + vi(1)
        return b + ld(8, name.encode()) + ld(9, arr.astype("<f4").tobytes())
    def node(op, ins, outs):
        return b"".join(ld(1, i.encode()) for i in ins) + b"".join(ld(2, o.encode()) for o in outs) + ld(4, op.encode())
    w = np.arange(12, dtype=np.float32).reshape(3, 4)
    graph = ld(1, node("MatMul", ["x", "encoder.layer.0.attention.self.query.weight"], ["y"])) + \
        ld(1, node("Add", ["y", "b"], ["z"])) + ld(5, tensor("encoder.layer.0.attention.self.query.weight", w))
    (tmp_path / "m.onnx").write_bytes(ld(7, graph))
    tensors, nodes = read_onnx(tmp_path / "m.onnx")
    assert np.array_equal(tensors["encoder.layer.0.attention.self.query.weight"].numpy(), w)
    assert [n["op_type"] for n in nodes] == ["MatMul", "Add"] and fused_patterns(nodes)["linear"] == 1


def test_codebook_gguf_types_decode_through_the_format_library():
    """IQ1 / IQ2 / IQ3 blocks (lattice codebooks) decode through the tables of the ``gguf`` package when it is there;
    the block geometry is ours. The block scale is linear: doubling the fp16 ``d`` field doubles every value."""
    import numpy as np
    from gllm_b200.loader import quant as Q
    if not Q.codebook_backend_available():
        import pytest
        pytest.skip("gguf package not installed")
    rng = np.random.RandomState(0)
    for name in ("IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S"):
        t = Q.BY_NAME[name]
        raw = rng.randint(0, 256, size=(3, t.block_bytes), dtype=np.uint8)
        raw[:, 0:2] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
        a = Q.dequantize(t.id, raw.tobytes(), 3 * t.block_elems)
        raw[:, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
        b = Q.dequantize(t.id, raw.tobytes(), 3 * t.block_elems)
        assert a.shape == (3 * t.block_elems,) and torch.isfinite(a).all() and a.abs().max() > 0
        torch.testing.assert_close(b, 2 * a)
    m = Q.BY_NAME["IQ1_M"]
    out = Q.dequantize(m.id, rng.randint(0, 256, size=(2, m.block_bytes), dtype=np.uint8).tobytes(), 2 * m.block_elems)
    assert out.shape == (512,)


def test_onnx_graph_import_recovers_fused_ops_and_names_anonymous_weights(tmp_path):
    """A one-layer BERT-style export written node by node, with initializer names that say nothing
    (``onnx::MatMul_7``): decomposed LayerNorm, erf-GELU, MatMul+Add and the softmax attention core are recovered as
    fused ops and the structure alone names every weight."""
    from gllm_b200.loader.onnx import OnnxProvider, import_graph

    def vi(n):
        out = b""
        while True:
            b7 = n & 0x7F
            n >>= 7
            out += bytes([b7 | (0x80 if n else 0)])
            if not n:
                return out
    ld = lambda fn, payload: vi((fn << 3) | 2) + vi(len(payload)) + payload

    def tensor(name, arr):
        b = b"".join(vi((1 << 3) | 0) + vi(d) for d in arr.shape) + vi((2 << 3) | 0) + vi(1)
        return b + ld(8, name.encode()) + ld(9, arr.astype("<f4").tobytes())
    node = lambda op, ins, outs: b"".join(ld(1, i.encode()) for i in ins) + b"".join(ld(2, o.encode()) for o in outs) + ld(4, op.encode())
    H = 8
    rng = np.random.RandomState(0)
    inits, nodes, k = {}, [], [0]

    def w(shape):
        k[0] += 1
        name = f"onnx::MatMul_{k[0]}"
        inits[name] = np.asarray(rng.randn(*shape), dtype=np.float32)
        return name

    def layernorm(x, out):
        g, b, eps, two = w((H,)), w((H,)), w(()), w(())
        nodes.extend([("ReduceMean", [x], [out + "_m"]), ("Sub", [x, out + "_m"], [out + "_c"]),
                      ("Pow", [out + "_c", two], [out + "_p"]), ("ReduceMean", [out + "_p"], [out + "_v"]),
                      ("Add", [out + "_v", eps], [out + "_e"]), ("Sqrt", [out + "_e"], [out + "_s"]),
                      ("Div", [out + "_c", out + "_s"], [out + "_n"]), ("Mul", [out + "_n", g], [out + "_g"]),
                      ("Add", [out + "_g", b], [out])])
        return g, b

    def linear(x, out, n_in, n_out):
        wt, bs = w((n_in, n_out)), w((n_out,))
        nodes.extend([("MatMul", [x, wt], [out + "_mm"]), ("Add", [out + "_mm", bs], [out])])
        return wt, bs
    table = w((30, H))
    nodes.append(("Gather", [table, "input_ids"], ["emb"]))
    g0, _ = layernorm("emb", "h0")
    q, _ = linear("h0", "q", H, H)
    kk, _ = linear("h0", "k", H, H)
    v, _ = linear("h0", "v", H, H)
    sc = w(())
    nodes.extend([("Transpose", ["k"], ["kt"]), ("MatMul", ["q", "kt"], ["s"]), ("Div", ["s", sc], ["ss"]),
                  ("Add", ["ss", "mask"], ["sm"]), ("Softmax", ["sm"], ["p"]), ("MatMul", ["p", "v"], ["ctx"])])
    o, _ = linear("ctx", "ao", H, H)
    nodes.append(("Add", ["ao", "h0"], ["r1"]))
    g1, _ = layernorm("r1", "h1")
    up, _ = linear("h1", "u", H, 4 * H)
    c2, c1, ch = w(()), w(()), w(())
    nodes.extend([("Div", ["u", c2], ["u_d"]), ("Erf", ["u_d"], ["u_e"]), ("Add", ["u_e", c1], ["u_a"]),
                  ("Mul", ["u", "u_a"], ["u_m"]), ("Mul", ["u_m", ch], ["act"])])
    dn, _ = linear("act", "d", 4 * H, H)
    nodes.append(("Add", ["d", "h1"], ["r2"]))
    g2, _ = layernorm("r2", "h2")
    graph = b"".join(ld(1, node(*n)) for n in nodes) + b"".join(ld(5, tensor(n, a)) for n, a in inits.items())
    (tmp_path / "enc.onnx").write_bytes(ld(7, graph))
    tensors, ops, names = import_graph(tmp_path / "enc.onnx")
    kinds = [o.kind for o in ops if o.kind != "other"]
    assert kinds == ["embedding", "layernorm", "linear", "linear", "linear", "attention", "linear", "add", "layernorm",
                     "linear", "gelu", "linear", "add", "layernorm"]
    assert sum(len(o.nodes) for o in ops) == len(nodes)                  # every node belongs to exactly one op
    want = {"embed_tokens": table, "embed_norm": g0, "L0.q_proj": q, "L0.k_proj": kk, "L0.v_proj": v, "L0.o_proj": o,
            "L0.post_attn_norm": g1, "L0.up_proj": up, "L0.down_proj": dn, "L0.post_ffn_norm": g2}
    assert {k_: names[k_] for k_ in want} == want and "L0.q_proj_bias" in names and "L0.post_ffn_norm_bias" in names
    prov = OnnxProvider(tmp_path / "enc.onnx", dtype=torch.float32)
    # MatMul weights are stored [in, out] in the export; the provider hands out [out, in]
    assert torch.equal(prov.get("L0.up_proj"), torch.from_numpy(inits[up]).t())


def _ref_gllm_bytes(name=b"L0.q_proj", shape=(2, 4), payload=None, data_off=4096, rel=0, count=1, dir_off=64,
                    meta_off=None, version=1, magic=0x4D4C4C47):
    """A .gllm file in the reference's byte layout, field by field (header offsets 0/4/8/12/20/24/32/40, 72-byte
    entries, names after the directory, MessagePack metadata, page-aligned data region)."""
    import struct
    import msgpack
    payload = payload if payload is not None else torch.arange(8, dtype=torch.float32).numpy().tobytes()
    strings_off = dir_off + 72 * count
    meta = msgpack.packb({"config": {"arch": "llama"}}, use_bin_type=True)
    meta_off = strings_off + len(name) if meta_off is None else meta_off
    buf = bytearray(data_off + rel + len(payload))
    struct.pack_into("<I", buf, 0, magic)
    struct.pack_into("<I", buf, 4, version)
    struct.pack_into("<I", buf, 8, 0)
    struct.pack_into("<Q", buf, 12, meta_off)
    struct.pack_into("<I", buf, 20, count)
    struct.pack_into("<Q", buf, 24, dir_off)
    struct.pack_into("<Q", buf, 32, data_off)
    struct.pack_into("<I", buf, 40, 4096)
    e = dir_off
    struct.pack_into("<I", buf, e + 0, 0)               # name_offset
    struct.pack_into("<H", buf, e + 4, len(name))       # name_len
    buf[e + 6] = len(shape)                              # ndim
    buf[e + 7] = 0                                       # dtype: F32
    for i, d in enumerate(shape):
        struct.pack_into("<Q", buf, e + 8 + 8 * i, d)
    buf[e + 40] = 0                                      # quant_format: none
    struct.pack_into("<Q", buf, e + 48, rel)             # data offset inside the data region
    struct.pack_into("<Q", buf, e + 56, 0)               # compressed size
    struct.pack_into("<Q", buf, e + 64, len(payload))    # original size
    buf[strings_off:strings_off + len(name)] = name
    if meta_off + len(meta) <= data_off:
        buf[meta_off:meta_off + len(meta)] = meta
    buf[data_off + rel:data_off + rel + len(payload)] = payload
    return bytes(buf)


def test_gllm_reference_layout_byte_exact_and_bounds_checks(tmp_path):
    """The reader takes a file laid out byte for byte as the reference writes it, and refuses files whose directory,
    names, metadata or payloads leave the file, whose names repeat, or whose magic / version are wrong."""
    from gllm_b200.loader.gllm_format import GllmFile, GllmFormatError, write_gllm
    p = tmp_path / "ref.gllm"
    p.write_bytes(_ref_gllm_bytes())
    f = GllmFile(p)
    assert f.layout == "reference" and f.page_size == 4096 and f.metadata["config"]["arch"] == "llama"
    torch.testing.assert_close(f.tensor("L0.q_proj"), torch.arange(8, dtype=torch.float32).reshape(2, 4))
    bad = {
        "magic": _ref_gllm_bytes(magic=0xBADBAD),
        "version": _ref_gllm_bytes(version=99),
        "directory": _ref_gllm_bytes(count=1000),
        "payload": _ref_gllm_bytes(rel=1 << 20)[:8192],
        "names": _ref_gllm_bytes(name=b"x" * 5000),
        "metadata": _ref_gllm_bytes(meta_off=1 << 30),
        "short": b"GLLM",
    }
    for what, raw in bad.items():
        q = tmp_path / f"bad_{what}.gllm"
        q.write_bytes(raw)
        with pytest.raises(GllmFormatError):
            GllmFile(q)
    # the writer produces the same layout: header fields at the reference's offsets, 72-byte entries
    import struct
    w = tmp_path / "w.gllm"
    write_gllm(w, {"a": torch.ones(3, 5, dtype=torch.bfloat16), "b": torch.arange(4, dtype=torch.int32)}, {"k": 1})
    raw = w.read_bytes()
    assert struct.unpack_from("<I", raw, 0)[0] == 0x4D4C4C47 and struct.unpack_from("<I", raw, 4)[0] == 1
    assert struct.unpack_from("<I", raw, 20)[0] == 2 and struct.unpack_from("<Q", raw, 24)[0] == 64
    data_off = struct.unpack_from("<Q", raw, 32)[0]
    assert data_off % 4096 == 0 and raw[64 + 7] == 2 and raw[64 + 6] == 2          # first entry: bf16, two dimensions
    g = GllmFile(w)
    assert g.metadata == {"k": 1} and g.tensor("b").tolist() == [0, 1, 2, 3] and g.tensor("a").dtype == torch.bfloat16


def test_gllm_private_layout_still_reads(tmp_path):
    """Files written by earlier versions of this package (magic "GLLMB200") are still readable."""
    import msgpack
    from gllm_b200.loader.gllm_format import PRIVATE_ENTRY, PRIVATE_HEADER, PRIVATE_MAGIC, GllmFile
    t = torch.arange(6, dtype=torch.float32)
    name, meta = b"final_norm", msgpack.packb({"v": 2}, use_bin_type=True)
    eoff = PRIVATE_HEADER.size
    soff = eoff + PRIVATE_ENTRY.size
    moff = soff + len(name)
    doff = (moff + len(meta) + 255) // 256 * 256
    raw = PRIVATE_HEADER.pack(PRIVATE_MAGIC, 1, 1, eoff, soff, len(name), moff, len(meta), doff)
    raw += PRIVATE_ENTRY.pack(0, len(name), 100, 1, 0, 6, 0, 0, 0, 0, 24) + name + meta
    raw += b"\0" * (doff - len(raw)) + t.numpy().tobytes()
    p = tmp_path / "old.gllm"
    p.write_bytes(raw)
    f = GllmFile(p)
    assert f.layout == "private" and f.metadata == {"v": 2}
    torch.testing.assert_close(f.tensor("final_norm"), t)
